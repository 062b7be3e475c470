"""tokenization subpackage."""
