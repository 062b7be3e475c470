"""chat subpackage."""
