"""B200 (sm_100a) implementation of the E5M2EffMA hot path: FP8 (E5M2 / E4M3) GEMM, GEMV, casts
and fused Adam / AdamW behind the C interface of include/e5m2effma.h.

The Python layer is a thin wrapper over that C interface (module `capi`), mirroring the
functional interface of the reference's binding (binds/python/e5m2effma/__init__.py:58-131):
`matmul`, `linear`, `cast`, `adam_step` and the `AdamW` optimizer.  torch is used for device
memory and streams only.  There is no CPU path and no alternative backend: a missing library or
a GPU other than compute capability 10.0 raises.
"""
__version__ = "0.2.0"
__all__ = ["capi", "matmul", "linear", "cast", "adam_step", "adam_step_multi", "AdamW", "get_include", "__version__"]


def __getattr__(name):
    """The binding (and with it libe5m2effma.so) is loaded on first use of any public name."""
    if name == "capi":
        import importlib
        return importlib.import_module(".capi", __name__)
    if name in __all__:
        from . import functional
        return getattr(functional, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
