"""generation subpackage."""
