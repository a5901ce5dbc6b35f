"""Host-side mirror of ``CUDAnative.WMMA`` over the library's 16x16x16 unit.

Reference: src/device/cuda/wmma.jl of CUDAnative.jl.  Names, argument order and error behaviour
follow the high-level API there:

    FragmentLayout / RowMajor / ColMajor / Unspecified      :313-338
    MatrixA / MatrixB / Accumulator                           :343-346
    Fragment{M,N,K,FS,T,L,U} with ``.x`` and indexing         :358-368
    Config{M,N,K,d_type}                                      :394
    load_a / load_b / load_c(addr, stride, layout, config)    :507-530
    mma(a, b, c, config)                                      :558-583
    store_d(addr, d, stride, layout, config)                  :613-632
    fill_c(value, config)                                     :654-667
    flatten / unflatten                                       :264-294
    ``scalar .* fragment`` broadcasting                        :678-716

In the reference these are device functions inlined into a user kernel and a Fragment is one
thread's registers.  Here each call launches a one-warp kernel of libb200wmma.so and a Fragment
is the whole warp's register image in device memory (32 lanes x FS elements, FS = 16 for A/B and
8 for C/D as in wmma.jl:413-420); which matrix element sits in which slot is unspecified, as in
the reference (docs/src/device/wmma.md:47-49).  A Fragment can also be built from a plain tuple,
which gives the per-thread value semantics that the reference's host-only broadcasting tests use
(test/device/wmma.jl:178-184).

``wmma_16x16x16`` runs the whole load -> scale -> mma -> store body of the reference's example
kernel (examples/wmma/high-level.jl:30-44) as one launch.
"""
from __future__ import annotations

import numpy as np

from . import _lib
from .array import CuHostArray, DevicePtr, Float16, Float32, pointer  # noqa: F401
from .execution import current_stream, require_full_warp


# ---- layouts, uses ---------------------------------------------------------------------------
class FragmentLayout:
    """Abstract storage layout of a matrix."""


class RowMajor(FragmentLayout):
    """Row major (C style) order."""


class ColMajor(FragmentLayout):
    """Column major (Julia style) order."""


class Unspecified(FragmentLayout):
    """Unspecified order; not valid for all WMMA operations."""


class FragmentUse:
    pass


class MatrixA(FragmentUse):
    pass


class MatrixB(FragmentUse):
    pass


class Accumulator(FragmentUse):
    pass


_LAYOUT_CODE = {ColMajor: _lib.COL_MAJOR, RowMajor: _lib.ROW_MAJOR}
_TYPE_CODE = {np.dtype(np.float16): _lib.F16, np.dtype(np.float32): _lib.F32}
_USE_CODE = {MatrixA: _lib.MATRIX_A, MatrixB: _lib.MATRIX_B, Accumulator: _lib.ACCUMULATOR}
_MATRIX_OF_USE = {"a": MatrixA, "b": MatrixB, "c": Accumulator, "d": Accumulator}
# wmma.jl:413-420
_NUM_ELEMS = {("a", np.dtype(np.float16)): 16, ("b", np.dtype(np.float16)): 16,
              ("c", np.dtype(np.float16)): 8, ("c", np.dtype(np.float32)): 8,
              ("d", np.dtype(np.float16)): 8, ("d", np.dtype(np.float32)): 8}


def _layout_code(L) -> int:
    try:
        return _LAYOUT_CODE[L]
    except (KeyError, TypeError):
        raise ValueError(f"Invalid layout for WMMA: {getattr(L, '__name__', L)}") from None


def _frag_elems(matrix: str, T) -> int:
    try:
        dt = np.dtype(T)
    except TypeError:
        raise ValueError(f"Invalid element type for WMMA: {T}") from None
    if dt not in _TYPE_CODE:
        raise ValueError(f"Invalid element type for WMMA: {dt}")
    try:
        return _NUM_ELEMS[(matrix, dt)]
    except KeyError:
        raise ValueError(f"Invalid type {dt} for matrix {matrix}") from None


class Config:
    """``Config{M, N, K, d_type}``: everything WMMA operations cannot infer from their arguments.
    Only (16, 16, 16) is a legal shape (wmma.jl:450-456); d_type is Float16 or Float32."""

    __slots__ = ("M", "N", "K", "d_type")

    def __init__(self, M: int, N: int, K: int, d_type):
        self.M, self.N, self.K = int(M), int(N), int(K)
        self.d_type = np.dtype(d_type)

    def __class_getitem__(cls, params):
        return cls(*params)

    def __repr__(self):
        return f"Config{{{self.M},{self.N},{self.K},{self.d_type.name}}}"

    def __eq__(self, other):
        return isinstance(other, Config) and (self.M, self.N, self.K, self.d_type) == (other.M, other.N, other.K, other.d_type)

    def __hash__(self):
        return hash((self.M, self.N, self.K, self.d_type))


def _check_shape(config: Config) -> None:
    if (config.M, config.N, config.K) != (16, 16, 16):
        raise ValueError(f"Invalid shape for WMMA: (M, N, K) = ({config.M}, {config.N}, {config.K})")


# ---- fragments ---------------------------------------------------------------------------------
class Fragment:
    """Intermediate result of WMMA operations.

    Device form: ``buf`` is a CuHostArray of 32 x FS elements (lane-major).  Host form: ``values``
    is one thread's tuple.  ``x`` / ``[]`` read elements; the ordering is unspecified."""

    __slots__ = ("M", "N", "K", "FS", "T", "L", "U", "buf", "values")
    __array_ufunc__ = None  # numpy scalars defer to __rmul__ / __radd__ instead of iterating us

    def __init__(self, M, N, K, FS, T, L, U, data=None):
        self.M, self.N, self.K, self.FS = int(M), int(N), int(K), int(FS)
        self.T = np.dtype(T)
        self.L, self.U = L, U
        self.buf = None
        self.values = None
        if isinstance(data, CuHostArray):
            self.buf = data
        elif data is not None:
            vals = tuple(self.T.type(v) for v in data)
            if len(vals) != self.FS:
                raise ValueError(f"fragment of size {self.FS} built from {len(vals)} values")
            self.values = vals

    def _like(self, data) -> "Fragment":
        return Fragment(self.M, self.N, self.K, self.FS, self.T, self.L, self.U, data)

    @property
    def on_device(self) -> bool:
        return self.buf is not None

    @property
    def x(self):
        """Host form: the tuple.  Device form: a (32, FS) array, one row per lane."""
        if self.values is not None:
            return self.values
        return np.ascontiguousarray(self.buf.to_host().reshape(32, self.FS))

    def __getitem__(self, i):
        return self.x[i]

    def __len__(self):
        return self.FS

    def __eq__(self, other):
        if not isinstance(other, Fragment):
            return NotImplemented
        same_type = (self.M, self.N, self.K, self.FS, self.T, self.L, self.U) == \
                    (other.M, other.N, other.K, other.FS, other.T, other.L, other.U)
        return same_type and np.array_equal(np.asarray(self.x), np.asarray(other.x))

    def __hash__(self):
        return id(self)

    def __repr__(self):
        where = "device" if self.on_device else "host"
        return (f"Fragment{{{self.M},{self.N},{self.K},{self.FS},{self.T.name},"
                f"{self.L.__name__},{self.U.__name__}}}<{where}>")

    # scalar .* frag, scalar .+ frag (wmma.jl:678-716): elementwise in the fragment's type,
    # result is a Fragment of the same type
    def _bcast(self, op: int, scalar) -> "Fragment":
        if self.values is not None:
            s = self.T.type(scalar)
            f = (lambda v: self.T.type(s * v)) if op == 0 else (lambda v: self.T.type(s + v))
            return self._like(tuple(f(v) for v in self.values))
        require_full_warp("fragment broadcast")
        out = CuHostArray(self.T, shape=(32 * self.FS,))
        _lib.check(_lib.lib().b200_wmma_bcast(current_stream(), op, _TYPE_CODE[self.T], self.FS, float(scalar),
                                              self.buf.ptr, out.ptr), "broadcast")
        return self._like(out)

    def __mul__(self, scalar):
        return self._bcast(0, scalar)

    __rmul__ = __mul__

    def __add__(self, scalar):
        return self._bcast(1, scalar)

    __radd__ = __add__


def _new_frag(matrix: str, T, L, config: Config) -> Fragment:
    fs = _frag_elems(matrix, T)
    buf = CuHostArray(np.dtype(T), shape=(32 * fs,))
    return Fragment(config.M, config.N, config.K, fs, T, L, _MATRIX_OF_USE[matrix], buf)


def _load(matrix: str, addr, stride, layout, config: Config) -> Fragment:
    addr = DevicePtr.of(addr)
    code = _layout_code(layout)
    _check_shape(config)
    require_full_warp(f"load_{matrix}")
    frag = _new_frag(matrix, addr.dtype, Unspecified if matrix == "c" else layout, config)
    _lib.check(_lib.lib().b200_wmma_load(current_stream(), _USE_CODE[frag.U], code, _TYPE_CODE[addr.dtype], addr.addr,
                                         int(stride), frag.buf.ptr), f"load_{matrix}")
    return frag


def load_a(addr, stride, layout, config: Config) -> Fragment:
    """Load matrix ``a`` (16x16 Float16) from ``addr`` with leading dimension ``stride``."""
    return _load("a", addr, stride, layout, config)


def load_b(addr, stride, layout, config: Config) -> Fragment:
    """Load matrix ``b`` (16x16 Float16)."""
    return _load("b", addr, stride, layout, config)


def load_c(addr, stride, layout, config: Config) -> Fragment:
    """Load the accumulator ``c`` (16x16 Float16 or Float32); its fragment layout is Unspecified."""
    return _load("c", addr, stride, layout, config)


def fill_c(value, config: Config) -> Fragment:
    """A ``c`` fragment filled with ``value`` (a numpy float16 / float32 scalar picks the type)."""
    T = np.dtype(type(value)) if isinstance(value, np.generic) else np.dtype(np.float32)
    _check_shape(config)
    require_full_warp("fill_c")
    frag = _new_frag("c", T, Unspecified, config)
    _lib.check(_lib.lib().b200_wmma_fill_c(current_stream(), _TYPE_CODE[frag.T], float(value), frag.buf.ptr), "fill_c")
    return frag


def mma(a: Fragment, b: Fragment, c: Fragment, config: Config) -> Fragment:
    """``D = A * B + C`` on the tensor cores; D's element type comes from ``config``."""
    if not (isinstance(a, Fragment) and a.U is MatrixA and isinstance(b, Fragment) and b.U is MatrixB
            and isinstance(c, Fragment) and c.U is Accumulator and c.L is Unspecified):
        raise TypeError("mma(a, b, c, config): a must be a MatrixA, b a MatrixB and c an Accumulator "
                        "fragment with Unspecified layout")  # the reference's MethodError
    for f in (a, b, c):
        if (f.M, f.N, f.K) != (config.M, config.N, config.K):
            raise TypeError("mma: fragment shape does not match the Config")
        if not f.on_device:
            raise TypeError("mma needs device fragments (from load_* or fill_c)")
    _check_shape(config)
    _layout_code(a.L), _layout_code(b.L)
    require_full_warp("mma")
    d = _new_frag("d", config.d_type, Unspecified, config)
    _lib.check(_lib.lib().b200_wmma_mma(current_stream(), _TYPE_CODE[c.T], _TYPE_CODE[d.T], a.buf.ptr, b.buf.ptr,
                                        c.buf.ptr, d.buf.ptr), "mma")
    return d


def store_d(addr, d: Fragment, stride, layout, config: Config) -> None:
    """Store the result fragment ``d`` to ``addr`` with leading dimension ``stride``."""
    addr = DevicePtr.of(addr)
    if not (isinstance(d, Fragment) and d.U is Accumulator and d.L is Unspecified and d.on_device):
        raise TypeError("store_d: d must be a device Accumulator fragment")
    if addr.dtype != d.T or config.d_type != d.T:
        raise TypeError("store_d: pointer, fragment and Config element types must agree")
    code = _layout_code(layout)
    _check_shape(config)
    require_full_warp("store_d")
    _lib.check(_lib.lib().b200_wmma_store_d(current_stream(), code, _TYPE_CODE[d.T], addr.addr, d.buf.ptr, int(stride)),
               "store_d")


# ---- the low-level wrappers (wmma.jl:104-257) under their reference names ------------------------
# 24 loads, 12 stores, 16 multiply-accumulates, e.g. llvm_wmma_load_a_col_m16n16k16_stride_f16(addr, stride),
# llvm_wmma_mma_col_col_m16n16k16_f32_f32(a, b, c), llvm_wmma_store_d_col_m16n16k16_stride_f32(addr, d, stride).
# In the reference they move per-thread register tuples; here they move Fragments, like the high-level API
# they back.  The `_global` forms take the same pointers as the generic ones.  The `_shared` forms need a
# shared-memory address, which only device code has: they exist (so that a script naming them imports) and
# refuse the call; the linkable device library carries the real ones.
_ELT = {"f16": np.dtype(np.float16), "f32": np.dtype(np.float32)}
_LAYOUT_OF = {"col": ColMajor, "row": RowMajor}
LLVM_WRAPPERS: list = []


def _define_llvm_wrappers() -> None:
    unit = Config(16, 16, 16, np.float32)

    def shared_refusal(name):
        def fn(*_args):
            raise _lib.B200Error(_lib.UNSUPPORTED, f"{name}: a shared-memory address exists only in device code; "
                                                   f"link b200_{name[5:]} from the device library instead")
        return fn

    def check_ptr(name, addr, elt):
        addr = DevicePtr.of(addr)
        if addr.dtype != _ELT[elt]:
            raise TypeError(f"{name}: expected a pointer to {_ELT[elt].name}, got {addr.dtype.name}")
        return addr

    def make_load(name, mat, layout, elt):
        def fn(src_addr, stride):
            return _load(mat, check_ptr(name, src_addr, elt), stride, _LAYOUT_OF[layout], unit)
        return fn

    def make_store(name, layout, elt):
        def fn(dst_addr, data, stride):
            return store_d(check_ptr(name, dst_addr, elt), data, stride, _LAYOUT_OF[layout], Config(16, 16, 16, _ELT[elt]))
        return fn

    def make_mma(name, a_layout, b_layout, d_elt, c_elt):
        def fn(a, b, c):
            if isinstance(a, Fragment) and isinstance(b, Fragment) and (a.L is not _LAYOUT_OF[a_layout] or b.L is not _LAYOUT_OF[b_layout]):
                raise TypeError(f"{name}: fragments were loaded as {a.L.__name__} / {b.L.__name__}")
            if isinstance(c, Fragment) and c.T != _ELT[c_elt]:
                raise TypeError(f"{name}: expected a {_ELT[c_elt].name} accumulator")
            return mma(a, b, c, Config(16, 16, 16, _ELT[d_elt]))
        return fn

    table = {}
    for space in ("", "_global", "_shared"):
        for layout in ("col", "row"):
            for mat, elts in (("a", ("f16",)), ("b", ("f16",)), ("c", ("f16", "f32"))):
                for elt in elts:
                    name = f"llvm_wmma_load_{mat}_{layout}_m16n16k16{space}_stride_{elt}"
                    table[name] = shared_refusal(name) if space == "_shared" else make_load(name, mat, layout, elt)
            for elt in ("f16", "f32"):
                name = f"llvm_wmma_store_d_{layout}_m16n16k16{space}_stride_{elt}"
                table[name] = shared_refusal(name) if space == "_shared" else make_store(name, layout, elt)
    for a_layout in ("col", "row"):
        for b_layout in ("col", "row"):
            for d_elt in ("f16", "f32"):
                for c_elt in ("f16", "f32"):
                    name = f"llvm_wmma_mma_{a_layout}_{b_layout}_m16n16k16_{d_elt}_{c_elt}"
                    table[name] = make_mma(name, a_layout, b_layout, d_elt, c_elt)
    for name, fn in table.items():
        fn.__name__ = fn.__qualname__ = name
        globals()[name] = fn
        LLVM_WRAPPERS.append(name)


_define_llvm_wrappers()


def synchronize() -> None:
    """Wait for the default stream (the reference's ``synchronize()``)."""
    _lib.check(_lib.lib().b200_stream_sync(None), "synchronize")


# ---- flatten / unflatten (wmma.jl:264-294) ------------------------------------------------------
class VecElement:
    """Mirror of Julia's ``VecElement{T}``: a value marked as an LLVM vector lane."""

    __slots__ = ("value",)

    def __init__(self, value):
        self.value = value

    def __eq__(self, other):
        return isinstance(other, VecElement) and self.value == other.value

    def __hash__(self):
        return hash(("VecElement", self.value))

    def __repr__(self):
        return f"VecElement({self.value!r})"


def flatten(x) -> tuple:
    """Nested tuples / VecElements -> one flat tuple of plain values."""
    if isinstance(x, VecElement):
        return (x.value,)
    if isinstance(x, tuple):
        out = []
        for item in x:
            out.extend(flatten(item))
        return tuple(out)
    return (x,)


def unflatten(spec, flat):
    """Inverse of flatten.  ``spec`` describes the nested type: a scalar type (``int``,
    ``float``, ``np.float16`` ...), ``(VecElement, T)`` for ``VecElement{T}``, or
    ``(n, inner_spec)`` for ``NTuple{n, inner}``."""
    flat = tuple(flat)
    value, rest = _unflatten(spec, flat)
    if rest:
        raise ValueError("unflatten: too many values for the requested type")
    return value


def _unflatten(spec, flat):
    if isinstance(spec, tuple) and len(spec) == 2 and spec[0] is VecElement:
        return VecElement(spec[1](flat[0])), flat[1:]
    if isinstance(spec, tuple) and len(spec) == 2 and isinstance(spec[0], int):
        items = []
        for _ in range(spec[0]):
            v, flat = _unflatten(spec[1], flat)
            items.append(v)
        return tuple(items), flat
    return spec(flat[0]), flat[1:]


# ---- the whole unit as one launch -----------------------------------------------------------------
LOWER_WARP = _lib.LOWER_WARP
LOWER_TCGEN05 = _lib.LOWER_TCGEN05


def wmma_16x16x16(a, b, c, d, *, a_layout=ColMajor, b_layout=ColMajor, c_layout=ColMajor, d_layout=ColMajor,
                  alpha=None, beta=None, lda=16, ldb=16, ldc=16, ldd=16, lowering=LOWER_WARP, stream=None) -> None:
    """``d = mma(alpha .* load_a(a), load_b(b), beta .* load_c(c))`` in one kernel.

    ``c=None`` is the ``fill_c(0)`` (MUL) case of test/device/wmma.jl:212-216.  ``alpha`` scales the
    Float16 A fragment and ``beta`` the C fragment in C's type, exactly where the reference's test
    applies them (test/device/wmma.jl:223-224); ``None`` skips the broadcast."""
    pa, pb, pd = DevicePtr.of(a), DevicePtr.of(b), DevicePtr.of(d)
    pc = DevicePtr.of(c) if c is not None else None
    if pa.dtype != np.float16 or pb.dtype != np.float16:
        raise ValueError("Invalid element type for WMMA: a and b must be Float16")
    c_type = _TYPE_CODE[pc.dtype] if pc is not None else _TYPE_CODE[pd.dtype]
    _lib.check(_lib.lib().b200_wmma_16x16x16(
        stream, lowering, _layout_code(a_layout), _layout_code(b_layout), _layout_code(c_layout),
        _layout_code(d_layout), c_type, _TYPE_CODE[pd.dtype], 1 if pc is not None else 0,
        0 if alpha is None else 1, 0.0 if alpha is None else float(alpha),
        0 if beta is None else 1, 0.0 if beta is None else float(beta),
        pa.addr, lda, pb.addr, ldb, pc.addr if pc is not None else None, ldc, pd.addr, ldd), "wmma_16x16x16")
