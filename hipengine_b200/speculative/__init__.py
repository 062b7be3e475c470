"""speculative subpackage."""
