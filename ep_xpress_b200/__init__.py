"""Blackwell-native expert-parallel dispatch/combine for MoE inference.

Importing this package neither compiles nor initialises CUDA; attributes are
resolved lazily (same rule as the reference, ep_xpress/__init__.py:13-20).
"""

__version__ = "0.1.0"

_EXPORTS = {
    "Config": ("config", "Config"),
    "Context": ("context", "Context"),
    "DispatchBatch": ("context", "DispatchBatch"),
    "Pending": ("context", "Pending"),
    "RouteHandle": ("context", "RouteHandle"),
    "NCCLCommHandle": ("comm", "NCCLCommHandle"),
    "get_nccl_comm_handle": ("comm", "get_nccl_comm_handle"),
    "EmulatedGroup": ("parallel.emulated", "EmulatedGroup"),
}

__all__ = sorted(_EXPORTS)


def __getattr__(name):
    try:
        module, attribute = _EXPORTS[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    import importlib
    value = getattr(importlib.import_module(f"{__name__}.{module}"), attribute)
    globals()[name] = value
    return value
