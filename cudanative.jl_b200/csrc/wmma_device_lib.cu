// Device-side fragment library: the 52 low-level WMMA wrappers of CUDAnative.jl as linkable
// `extern "C" __device__` functions for sm_100a.
//
// Reference: src/device/cuda/wmma.jl generates
//   llvm_wmma_load_{a,b,c}_{col,row}_m16n16k16[_global|_shared]_stride_{f16,f32}   (:104-137, 24 functions)
//   llvm_wmma_store_d_{col,row}_m16n16k16[_global|_shared]_stride_{f16,f32}        (:162-191, 12 functions)
//   llvm_wmma_mma_{col,row}_{col,row}_m16n16k16_{f16,f32}_{f16,f32}                 (:222-257, 16 functions)
// each a `ccall("extern llvm.nvvm.wmma...", llvmcall, ...)` that the NVPTX back-end turns into one
// wmma.* instruction.  Here the same names, prefixed b200_, are real device functions: a Julia kernel
// reaches them the way the reference reaches libcudadevrt (src/device/cuda/libcudadevrt.jl:12-16:
// `ccall("extern <symbol>", llvmcall, ...)`) after adding this object or its PTX to the CuLink
// invocation of src/execution.jl:325-332.  All 32 lanes of a warp must call with identical arguments,
// as for the reference's intrinsics (wmma.jl:500-504).
//
// Register fragments have the reference's sizes: 8 x <2 x half> for A, B (16 halves per lane),
// 4 x <2 x half> for Float16 C / D and 8 x float for Float32 C / D (wmma.jl:23-30).  Layout is handled
// by the load: a fragment holds the same logical elements whatever layout it was loaded with, so the
// sixteen mma variants differ only in their C / D element types.  `_global` and `_shared` variants take
// state-space addresses (what a Julia DevicePtr{T,AS.Global} / DevicePtr{T,AS.Shared} holds,
// src/device/pointer.jl:11-27); the unsuffixed ones take generic addresses.
//
// The multiply-accumulate is mma.sync.aligned.m16n8k16 x 2: the warp-level tensor-core instruction
// that sm_100a offers to code which keeps its operands in registers.  Products of whole matrices
// belong on the tcgen05 kernels of gemm_sm100.cuh instead.
#include <cuda_fp16.h>

#include "wmma_frag.cuh"

using namespace b200;

extern "C" {

// Plain aggregates of 32-bit words, so that they travel by value in .param space exactly like the
// LLVM structs {<2 x half> x 8}, {<2 x half> x 4} and {float x 8} of the reference's wrappers
// (wmma.jl:67-75); each word of the first two packs two binary16 values, low half first.
struct b200_frag_ab { uint32_t x[8]; };  // a.f16 / b.f16: 8 x <2 x half>
struct b200_frag_h { uint32_t x[4]; };   // c.f16 / d.f16: 4 x <2 x half>
struct b200_frag_f { float x[8]; };      // c.f32 / d.f32: 8 x float

}  // extern "C"

namespace {

enum { kGeneric = 0, kGlobal = 1, kShared = 3 };

template <int kAS, typename T>
__device__ __forceinline__ T* as_generic(const void* p) {
    if (kAS == kShared) return static_cast<T*>(__cvta_shared_to_generic(reinterpret_cast<size_t>(p)));
    if (kAS == kGlobal) return static_cast<T*>(__cvta_global_to_generic(reinterpret_cast<size_t>(p)));
    return static_cast<T*>(const_cast<void*>(p));
}

// The hardware lane of the calling thread: right for any block shape (threadIdx.x & 31 would be wrong
// for a block whose x extent is not a multiple of 32, e.g. threads = (16, 2)), as the reference's
// intrinsics are (they are warp-level instructions, src/device/cuda/wmma.jl:500-504).
__device__ __forceinline__ int lane() {
    unsigned l;
    asm("mov.u32 %0, %%laneid;" : "=r"(l));
    return static_cast<int>(l);
}

__device__ __forceinline__ __half half_of(uint32_t word, int hi) {
    return __ushort_as_half(static_cast<unsigned short>(hi ? (word >> 16) : (word & 0xffffu)));
}

template <int kUse, int kLayout, int kAS>
__device__ __forceinline__ b200_frag_ab load_ab(const void* addr, int stride) {
    const __half* p = as_generic<kAS, const __half>(addr);
    b200_frag_ab f;
#pragma unroll
    for (int e = 0; e < 16; e += 2) {
        int r0, c0, r1, c1;
        frag_coord(kUse, lane(), e, r0, c0);
        frag_coord(kUse, lane(), e + 1, r1, c1);
        f.x[e / 2] = pack2(p[mat_off(kLayout, r0, c0, stride)], p[mat_off(kLayout, r1, c1, stride)]);
    }
    return f;
}

template <int kLayout, int kAS>
__device__ __forceinline__ b200_frag_h load_c_h(const void* addr, int stride) {
    const __half* p = as_generic<kAS, const __half>(addr);
    b200_frag_h f;
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        int r0, c0, r1, c1;
        c_coord(lane(), e, r0, c0);
        c_coord(lane(), e + 1, r1, c1);
        f.x[e / 2] = pack2(p[mat_off(kLayout, r0, c0, stride)], p[mat_off(kLayout, r1, c1, stride)]);
    }
    return f;
}

template <int kLayout, int kAS>
__device__ __forceinline__ b200_frag_f load_c_f(const void* addr, int stride) {
    const float* p = as_generic<kAS, const float>(addr);
    b200_frag_f f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        int r, c;
        c_coord(lane(), e, r, c);
        f.x[e] = p[mat_off(kLayout, r, c, stride)];
    }
    return f;
}

template <int kLayout, int kAS>
__device__ __forceinline__ void store_h(void* addr, const b200_frag_h& d, int stride) {
    __half* p = as_generic<kAS, __half>(addr);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        int r, c;
        c_coord(lane(), e, r, c);
        p[mat_off(kLayout, r, c, stride)] = half_of(d.x[e / 2], e & 1);
    }
}

template <int kLayout, int kAS>
__device__ __forceinline__ void store_f(void* addr, const b200_frag_f& d, int stride) {
    float* p = as_generic<kAS, float>(addr);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        int r, c;
        c_coord(lane(), e, r, c);
        p[mat_off(kLayout, r, c, stride)] = d.x[e];
    }
}

__device__ __forceinline__ void unpack_ab(const b200_frag_ab& f, __half (&out)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // slots 8..15 repeat slots 0..7
        out[2 * i] = half_of(f.x[i], 0);
        out[2 * i + 1] = half_of(f.x[i], 1);
    }
}

template <int kCType, int kDType, typename CF, typename DF>
__device__ __forceinline__ DF mma_any(const b200_frag_ab& a, const b200_frag_ab& b, const CF& c) {
    __half ah[8], bh[8];
    float cf[8], df[8];
    unpack_ab(a, ah);
    unpack_ab(b, bh);
    if constexpr (kCType == B200_F16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            cf[2 * i] = __half2float(half_of(c.x[i], 0));
            cf[2 * i + 1] = __half2float(half_of(c.x[i], 1));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) cf[i] = c.x[i];
    }
    warp_mma(ah, bh, cf, kCType, kDType, df);
    DF d;
    if constexpr (kDType == B200_F16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) d.x[i] = pack2(__float2half_rn(df[2 * i]), __float2half_rn(df[2 * i + 1]));
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) d.x[i] = df[i];
    }
    return d;
}

}  // namespace

extern "C" {

// ---- loads: 24 functions ------------------------------------------------------------------------------
#define B200_LOAD_AB(mat, use, lay, laycode, sfx, as)                                                        \
    __device__ b200_frag_ab b200_wmma_load_##mat##_##lay##_m16n16k16##sfx##_stride_f16(const void* addr,     \
                                                                                        int stride) {        \
        return load_ab<use, laycode, as>(addr, stride);                                                      \
    }
#define B200_LOAD_C(lay, laycode, sfx, as)                                                                    \
    __device__ b200_frag_h b200_wmma_load_c_##lay##_m16n16k16##sfx##_stride_f16(const void* addr, int stride) { \
        return load_c_h<laycode, as>(addr, stride);                                                            \
    }                                                                                                          \
    __device__ b200_frag_f b200_wmma_load_c_##lay##_m16n16k16##sfx##_stride_f32(const void* addr, int stride) { \
        return load_c_f<laycode, as>(addr, stride);                                                            \
    }
#define B200_STORE_D(lay, laycode, sfx, as)                                                                   \
    __device__ void b200_wmma_store_d_##lay##_m16n16k16##sfx##_stride_f16(void* addr, b200_frag_h d,           \
                                                                           int stride) {                       \
        store_h<laycode, as>(addr, d, stride);                                                                 \
    }                                                                                                          \
    __device__ void b200_wmma_store_d_##lay##_m16n16k16##sfx##_stride_f32(void* addr, b200_frag_f d,           \
                                                                           int stride) {                       \
        store_f<laycode, as>(addr, d, stride);                                                                 \
    }
#define B200_FOR_EACH_AS(M, ...)       \
    M(__VA_ARGS__, , kGeneric)         \
    M(__VA_ARGS__, _global, kGlobal)   \
    M(__VA_ARGS__, _shared, kShared)

B200_FOR_EACH_AS(B200_LOAD_AB, a, B200_MATRIX_A, col, B200_COL_MAJOR)
B200_FOR_EACH_AS(B200_LOAD_AB, a, B200_MATRIX_A, row, B200_ROW_MAJOR)
B200_FOR_EACH_AS(B200_LOAD_AB, b, B200_MATRIX_B, col, B200_COL_MAJOR)
B200_FOR_EACH_AS(B200_LOAD_AB, b, B200_MATRIX_B, row, B200_ROW_MAJOR)
B200_FOR_EACH_AS(B200_LOAD_C, col, B200_COL_MAJOR)
B200_FOR_EACH_AS(B200_LOAD_C, row, B200_ROW_MAJOR)

// ---- stores: 12 functions -----------------------------------------------------------------------------
B200_FOR_EACH_AS(B200_STORE_D, col, B200_COL_MAJOR)
B200_FOR_EACH_AS(B200_STORE_D, row, B200_ROW_MAJOR)

// ---- mma: 16 functions (a layout, b layout, d type, c type) -------------------------------------------
#define B200_MMA(al, bl)                                                                                              \
    __device__ b200_frag_h b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f16(b200_frag_ab a, b200_frag_ab b,              \
                                                                         b200_frag_h c) {                             \
        return mma_any<B200_F16, B200_F16, b200_frag_h, b200_frag_h>(a, b, c);                                        \
    }                                                                                                                 \
    __device__ b200_frag_h b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f32(b200_frag_ab a, b200_frag_ab b,              \
                                                                         b200_frag_f c) {                             \
        return mma_any<B200_F32, B200_F16, b200_frag_f, b200_frag_h>(a, b, c);                                        \
    }                                                                                                                 \
    __device__ b200_frag_f b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f16(b200_frag_ab a, b200_frag_ab b,              \
                                                                         b200_frag_h c) {                             \
        return mma_any<B200_F16, B200_F32, b200_frag_h, b200_frag_f>(a, b, c);                                        \
    }                                                                                                                 \
    __device__ b200_frag_f b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f32(b200_frag_ab a, b200_frag_ab b,              \
                                                                         b200_frag_f c) {                             \
        return mma_any<B200_F32, B200_F32, b200_frag_f, b200_frag_f>(a, b, c);                                        \
    }
B200_MMA(col, col)
B200_MMA(col, row)
B200_MMA(row, col)
B200_MMA(row, row)

}  // extern "C"
