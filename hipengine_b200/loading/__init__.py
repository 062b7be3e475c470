"""loading subpackage."""
