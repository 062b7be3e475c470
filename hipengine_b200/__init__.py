"""hipengine_b200: a Blackwell-native (sm_100a) LLM inference and serving engine.

Public surface mirrors the reference package root (``hipengine/__init__.py:20-34``):
``LLM``, ``SamplingParams``, ``ExecutionProfile``, ``ResidentPreparationError``, ``UnsupportedModalityError``.
Unlike the reference, PyTorch is the framework layer here, so importing the
package imports torch; the heavy pieces (CUDA extension, server) load lazily.
"""
from __future__ import annotations

__version__ = "0.1.0"

_LAZY = {
    "LLM": "hipengine_b200.llm",
    "SamplingParams": "hipengine_b200.llm",
    "ResidentPreparationError": "hipengine_b200.llm",
    "UnsupportedModalityError": "hipengine_b200.llm",
    "ExecutionProfile": "hipengine_b200.config",
    "EngineConfig": "hipengine_b200.config",
}

__all__ = sorted(_LAZY) + ["__version__"]


def __getattr__(name: str):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    from importlib import import_module
    value = getattr(import_module(mod), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
