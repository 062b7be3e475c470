"""kvcache subpackage."""
