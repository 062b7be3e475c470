"""models subpackage."""


def make_executor(weights, **kw):
    """Executor class for the checkpoint's architecture."""
    if weights.config.arch == "gemma4":
        from .gemma4 import Gemma4Executor
        return Gemma4Executor(weights, **kw)
    from .executor import HybridExecutor
    return HybridExecutor(weights, **kw)
