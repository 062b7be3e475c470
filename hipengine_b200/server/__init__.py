"""server subpackage."""
