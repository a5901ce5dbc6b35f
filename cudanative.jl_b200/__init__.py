"""B200-native replacement for the FP16 x FP16 -> FP32 tensor-core GEMM path of CUDAnative.jl.

* ``wmma``  -- host-side mirror of ``CUDAnative.WMMA`` (Config, load_a/b/c, mma, store_d,
  fill_c, fragment broadcasting) over the library's 16x16x16 unit.
* ``gemm``  -- the tiled GEMM ``D = alpha*op(A)*op(B) + beta*C`` and its N-sharded multi-GPU form.
* ``bfloat16`` -- host-side bfloat16 (bit patterns in uint16) for the bfloat16 variants of ``gemm``.
* ``rng``   -- the counter-based synthetic matrices used by tests and benchmarks.
* ``_lib``  -- ctypes binding of ``libb200wmma.so`` (the C ABI declared in include/b200wmma.h).

All arithmetic runs in hand-written sm_100a kernels inside ``libb200wmma.so``; nothing here
computes on the CPU or through PyTorch operators.
"""
from . import _lib  # noqa: F401
from ._lib import B200Error  # noqa: F401

__all__ = ["B200Error", "_lib", "bfloat16", "build", "gemm", "rng", "wmma"]


def __getattr__(name):
    # submodules load lazily so that `build` can be imported before the library exists
    if name in ("build", "gemm", "rng", "wmma", "array", "bfloat16"):
        import importlib

        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
