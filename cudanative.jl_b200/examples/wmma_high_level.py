"""examples/wmma/high-level.jl of CUDAnative.jl, statement for statement (its lines 20-49).

    a_dev = CuArray(a) ...                      ->  the same
    function kernel(a_dev, b_dev, c_dev, d_dev)  ->  def kernel(a_dev, b_dev, c_dev, d_dev)
    @cuda threads=32 kernel(a_dev, ...)          ->  cuda(kernel, a_dev, ..., threads=32)
    d = Array(d_dev)                             ->  the same
"""
import numpy as np

from cudanative_jl_b200 import wmma as WMMA
from cudanative_jl_b200.array import Array, CuArray, pointer, similar
from cudanative_jl_b200.execution import cuda


def kernel(a_dev, b_dev, c_dev, d_dev):
    conf = WMMA.Config[16, 16, 16, np.float32]

    a_frag = WMMA.load_a(pointer(a_dev), 16, WMMA.ColMajor, conf)
    b_frag = WMMA.load_b(pointer(b_dev), 16, WMMA.ColMajor, conf)
    c_frag = WMMA.load_c(pointer(c_dev), 16, WMMA.ColMajor, conf)

    c_frag = np.float32(0.5) * c_frag

    d_frag = WMMA.mma(a_frag, b_frag, c_frag, conf)

    WMMA.store_d(pointer(d_dev), d_frag, 16, WMMA.ColMajor, conf)

    return


def main(seed: int = 0):
    """Returns (a, b, c, d) as host arrays; the reference's check is
    ``all(isapprox.(a * b + 0.5 * c, d; rtol=0.01))``."""
    rand = np.random.default_rng(seed)
    a = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
    b = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
    c = np.asfortranarray(rand.random((16, 16)).astype(np.float32))

    a_dev = CuArray(a)
    b_dev = CuArray(b)
    c_dev = CuArray(c)
    d_dev = similar(c_dev)

    cuda(kernel, a_dev, b_dev, c_dev, d_dev, threads=32)
    d = Array(d_dev)
    return a, b, c, d


if __name__ == "__main__":
    a, b, c, d = main()
    ref = a.astype(np.float32) @ b.astype(np.float32) + 0.5 * c
    assert np.all(np.abs(ref - d) <= 0.01 * np.maximum(np.abs(ref), np.abs(d)))
    print("ok")
