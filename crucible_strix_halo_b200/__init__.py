"""B200 (sm_100a) attention hot path of the Crucible engine: QSA sparse gated attention and Gated DeltaNet,
behind a C ABI (include/crucible_attn.h).  This package holds the CUDA sources (csrc/), the in-tree build
(build.py), the ctypes binding (capi.py) and torch-tensor convenience wrappers (layers.py).  There is no CPU
fallback: using the binding without the built library raises ImportError."""


def __getattr__(name):   # capi loads the shared library; keep `python -m crucible_strix_halo_b200.build` importable without it
    if name in ("capi", "layers"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
