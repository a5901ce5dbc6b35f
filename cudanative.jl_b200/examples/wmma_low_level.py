"""examples/wmma/low-level.jl of CUDAnative.jl, statement for statement (its lines 20-45): the same
product through the low-level wrappers, D = A * B + C."""
import numpy as np

from cudanative_jl_b200 import wmma as WMMA
from cudanative_jl_b200.array import Array, CuArray, pointer, similar
from cudanative_jl_b200.execution import cuda


# Matrix multiply-accumulate kernel (D = A * B + C)
def kernel(a_dev, b_dev, c_dev, d_dev):
    a_frag = WMMA.llvm_wmma_load_a_col_m16n16k16_stride_f16(pointer(a_dev), 16)
    b_frag = WMMA.llvm_wmma_load_b_col_m16n16k16_stride_f16(pointer(b_dev), 16)
    c_frag = WMMA.llvm_wmma_load_c_col_m16n16k16_stride_f32(pointer(c_dev), 16)

    d_frag = WMMA.llvm_wmma_mma_col_col_m16n16k16_f32_f32(a_frag, b_frag, c_frag)

    WMMA.llvm_wmma_store_d_col_m16n16k16_stride_f32(pointer(d_dev), d_frag, 16)
    return


def main(seed: int = 0):
    rand = np.random.default_rng(seed)
    # Generate input matrices
    a = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
    a_dev = CuArray(a)
    b = np.asfortranarray(rand.random((16, 16)).astype(np.float16))
    b_dev = CuArray(b)
    c = np.asfortranarray(rand.random((16, 16)).astype(np.float32))
    c_dev = CuArray(c)

    # Allocate space for result
    d_dev = similar(c_dev)

    cuda(kernel, a_dev, b_dev, c_dev, d_dev, threads=32)
    return a, b, c, Array(d_dev)


if __name__ == "__main__":
    a, b, c, d = main()
    ref = a.astype(np.float32) @ b.astype(np.float32) + c
    assert np.all(np.abs(ref - d) <= 0.01 * np.maximum(np.abs(ref), np.abs(d)))
    print("ok")
