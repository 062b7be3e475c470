"""ref subpackage."""
