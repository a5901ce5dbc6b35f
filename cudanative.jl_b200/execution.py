"""``@cuda``-style launches for kernels written against the host-level WMMA mirror.

Reference: src/execution.jl of CUDAnative.jl.  ``@cuda threads=32 kernel(a_dev, b_dev, c_dev, d_dev)``
(examples/wmma/high-level.jl:46) converts every argument with ``cudaconvert`` (:99-139), compiles the
function once per argument-type tuple (``cufunction``, :296-298, cached) into a ``HostKernel`` (:203-207) and
calls it with the launch keywords ``threads``, ``blocks``, ``shmem``, ``config``, ``stream``, ``cooperative``
(:152-166, :60-63); ``config`` is a callback that receives the kernel and returns some of those keywords
(:209-215).  The launch is asynchronous on ``stream``; any other keyword is an ``ArgumentError`` (:64-67).

Here a "kernel" is a Python function whose body is made of the fragment operations of ``wmma`` --
each of them a call into ``libb200wmma.so`` that enqueues device work.  ``cuda(...)`` keeps the
conventions: same keywords and defaults, same errors for unknown ones, the same conversion and caching
steps, work enqueued on the launch's stream and nothing waited for.  A WMMA operation is a one-warp
operation, so the function body runs once per warp of the launch (``blocks`` x ``threads / 32`` times)
with ``threadIdx()`` / ``blockIdx()`` set for that warp.  A block of fewer than 32 threads (the default is
``threads=1``) has no full warp: its body still runs once, and a WMMA operation inside it is refused
(in the reference that is undefined behaviour: ``wmma.*.sync`` needs all 32 lanes).
"""
from __future__ import annotations

import contextvars
from collections import namedtuple

import numpy as np

from . import _lib
from .array import CuHostArray, DevicePtr

Dim3 = namedtuple("Dim3", "x y z")

LAUNCH_KEYWORDS = ("cooperative", "blocks", "threads", "config", "shmem", "stream")
COMPILER_KEYWORDS = ("minthreads", "maxthreads", "blocks_per_sm", "maxregs", "name")

_stream = contextvars.ContextVar("b200_stream", default=None)
_indices = contextvars.ContextVar("b200_indices", default=None)


def current_stream():
    """The stream the fragment operations enqueue on: the launch's ``stream`` inside a kernel body,
    otherwise the default stream (``CuDefaultStream()``, src/execution.jl:165)."""
    return _stream.get()


def _index(name: str) -> Dim3:
    idx = _indices.get()
    if idx is None:
        raise RuntimeError(f"{name}() is only defined inside a kernel launched with cuda(...)")
    return idx[name]


def threadIdx() -> Dim3:
    """1-based index of the warp's first thread inside its block, as Julia counts (src/device/cuda/indexing.jl)."""
    return _index("threadIdx")


def blockIdx() -> Dim3:
    return _index("blockIdx")


def blockDim() -> Dim3:
    return _index("blockDim")


def gridDim() -> Dim3:
    return _index("gridDim")


def require_full_warp(op: str) -> None:
    """Called by every fragment operation: inside a launch whose blocks have fewer than 32 threads
    there is no warp that could execute it."""
    idx = _indices.get()
    if idx is not None and not idx["full_warp"]:
        raise _lib.B200Error(_lib.UNSUPPORTED, f"{op}: WMMA operations are executed by whole warps; "
                                               f"this kernel was launched with {idx['block_threads']} threads per block")


def _dim3(value, what: str) -> Dim3:
    if isinstance(value, (int, np.integer)):
        value = (int(value),)
    value = tuple(int(v) for v in value)
    if not 1 <= len(value) <= 3 or any(v < 1 for v in value):
        raise ValueError(f"{what} must be 1 to 3 positive integers")
    return Dim3(*(value + (1, 1, 1))[:3])


class CuDeviceArray:
    """What a ``CuHostArray`` becomes on its way into a kernel (the reference converts host handles
    to device-side ones with Adapt, src/execution.jl:99-139): a typed device pointer plus dims, with
    the owner kept alive for as long as the view exists."""

    __slots__ = ("ptr", "shape", "dtype", "_owner")

    def __init__(self, owner: CuHostArray):
        self.ptr = DevicePtr(owner.dtype, owner.ptr, owner)
        self.shape = owner.shape
        self.dtype = owner.dtype
        self._owner = owner


def cudaconvert(arg):
    """Called for every kernel argument; everything but a ``CuHostArray`` passes unchanged."""
    if isinstance(arg, CuHostArray):
        return CuDeviceArray(arg)
    return arg


class HostKernel:
    """A kernel function bound to an argument-type tuple (src/execution.jl:203-207).  Calling it
    launches: ``kernel(*args, threads=32, stream=s)``."""

    def __init__(self, f, tt: tuple):
        self.f = f
        self.tt = tt
        self.launches = 0

    def __call__(self, *args, **kwargs):
        for key in kwargs:
            if key not in LAUNCH_KEYWORDS:
                raise TypeError(f"Unsupported keyword argument '{key}'")
        config = kwargs.pop("config", None)
        if config is not None:
            # the callback sees the kernel and may set any of the launch keywords; its values win
            kwargs.update(dict(config(self)))
            for key in kwargs:
                if key not in LAUNCH_KEYWORDS or key == "config":
                    raise TypeError(f"Unsupported keyword argument '{key}' returned by config")
        threads = _dim3(kwargs.get("threads", 1), "threads")
        blocks = _dim3(kwargs.get("blocks", 1), "blocks")
        shmem = int(kwargs.get("shmem", 0))
        if shmem < 0:
            raise ValueError("shmem must be non-negative")
        if len(args) != len(self.tt) or tuple(type(a) for a in args) != self.tt:
            raise TypeError("kernel called with arguments that do not match the types it was compiled for")
        block_threads = threads.x * threads.y * threads.z
        if block_threads > 1024:
            raise ValueError("Number of threads per block exceeds 1024")
        # full warps run the body once each; a block without one still runs it once (its WMMA calls raise)
        warps = max(1, block_threads // 32)
        stream = kwargs.get("stream", None)
        token_s = _stream.set(stream)
        try:
            for bz in range(blocks.z):
                for by in range(blocks.y):
                    for bx in range(blocks.x):
                        for w in range(warps):
                            lin = w * 32  # first thread of the warp, linear index inside the block
                            tid = Dim3(lin % threads.x + 1, lin // threads.x % threads.y + 1,
                                       lin // (threads.x * threads.y) + 1)
                            token_i = _indices.set({"threadIdx": tid, "blockIdx": Dim3(bx + 1, by + 1, bz + 1),
                                                    "blockDim": threads, "gridDim": blocks,
                                                    "full_warp": block_threads >= 32, "block_threads": block_threads})
                            try:
                                self.f(*args)
                            finally:
                                _indices.reset(token_i)
        finally:
            _stream.reset(token_s)
        self.launches += 1
        return None


_kernel_cache: dict = {}


def cufunction(f, tt: tuple, **compiler_kwargs) -> HostKernel:
    """``cufunction(f, tt)``: the kernel object for ``f`` and an argument-type tuple, made once and
    cached (src/execution.jl:296-298).  The compiler keywords of the reference are accepted and have
    nothing to act on here (there is no code generation)."""
    for key in compiler_kwargs:
        if key not in COMPILER_KEYWORDS:
            raise TypeError(f"Unsupported keyword argument '{key}'")
    key = (f, tuple(tt))
    kernel = _kernel_cache.get(key)
    if kernel is None:
        kernel = _kernel_cache[key] = HostKernel(f, tuple(tt))
    return kernel


def cuda(f, *args, **kwargs) -> None:
    """``@cuda [kwargs...] f(args...)``: convert the arguments, get the cached kernel, launch it.
    Keywords: ``threads`` (1), ``blocks`` (1), ``shmem`` (0), ``config``, ``stream`` (default stream),
    ``cooperative``, plus the reference's compiler keywords.  ``dynamic=True`` (device-side launch) does not
    exist on the host."""
    if not callable(f):
        raise TypeError("second argument to cuda should be a function call")
    if kwargs.pop("dynamic", False):
        raise _lib.B200Error(_lib.UNSUPPORTED, "cuda launch: dynamic parallelism is a device-side launch")
    compiler = {k: kwargs.pop(k) for k in list(kwargs) if k in COMPILER_KEYWORDS}
    for key in kwargs:
        if key not in LAUNCH_KEYWORDS:
            raise TypeError(f"Unsupported keyword argument '{key}'")
    kernel_args = tuple(cudaconvert(a) for a in args)
    kernel = cufunction(f, tuple(type(a) for a in kernel_args), **compiler)
    kernel(*kernel_args, **kwargs)


def synchronize(stream=None) -> None:
    """Wait for ``stream`` (default: the default stream), the reference's ``synchronize()``."""
    _lib.check(_lib.lib().b200_stream_sync(stream), "synchronize")
