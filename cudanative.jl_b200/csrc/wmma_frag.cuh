// Register-level pieces of the 16x16x16 WMMA unit shared by the host-launched kernels
// (wmma_unit.cu) and the linkable device library (wmma_device_lib.cu): the slot -> matrix-element
// maps of a fragment and the warp-wide multiply-accumulate on mma.sync.m16n8k16.
//
// Fragment sizes follow CUDAnative.jl src/device/cuda/wmma.jl:413-420 (16 elements per lane for A
// and B, 8 for C and D); which element sits in which slot is private, as the reference leaves it
// unspecified (docs/src/device/wmma.md:47-49): slots follow the register order of
// mma.sync.m16n8k16 (A: 8 halves per lane; B and C/D: two n-blocks of 8 columns) and A/B slots
// 8..15 repeat slots 0..7.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/b200wmma.h"

namespace b200 {

// ---- slot -> (row, col) maps --------------------------------------------------------------
__device__ __forceinline__ void a_coord(int lane, int e, int& row, int& k) {
    e &= 7;
    const int g = lane >> 2, t = lane & 3;
    row = g + ((e >> 1) & 1) * 8;
    k = 2 * t + (e & 1) + ((e >> 2) & 1) * 8;
}
__device__ __forceinline__ void b_coord(int lane, int e, int& k, int& n) {
    e &= 7;
    const int g = lane >> 2, t = lane & 3;
    const int ee = e & 3;
    n = g + 8 * (e >> 2);
    k = 2 * t + (ee & 1) + ((ee >> 1) & 1) * 8;
}
__device__ __forceinline__ void c_coord(int lane, int e, int& row, int& col) {
    const int g = lane >> 2, t = lane & 3;
    const int ee = e & 3;
    row = g + ((ee >> 1) & 1) * 8;
    col = 8 * (e >> 2) + 2 * t + (ee & 1);
}
// linear offset of element (r, c) of a 16x16 matrix with leading dimension `ld`
__device__ __forceinline__ int64_t mat_off(int layout, int r, int c, int64_t ld) {
    return layout == B200_ROW_MAJOR ? r * ld + c : r + c * ld;
}
__device__ __forceinline__ void frag_coord(int use, int lane, int e, int& r, int& c) {
    if (use == B200_MATRIX_A) a_coord(lane, e, r, c);
    else if (use == B200_MATRIX_B) b_coord(lane, e, r, c);
    else c_coord(lane, e, r, c);
}

// ---- mma.sync wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(__half lo, __half hi) {
    return static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

__device__ __forceinline__ void mma_16x8x16_f32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2],
                                                const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}
__device__ __forceinline__ void mma_16x8x16_f16(uint32_t (&d)[2], const uint32_t (&a)[4], const uint32_t (&b)[2],
                                                const uint32_t (&c)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%9};"
        : "=r"(d[0]), "=r"(d[1])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(c[0]), "r"(c[1]));
}

// One warp: d(16x16) = a * b + c from register fragments in this file's slot order.
// c / d travel as float; c_type / d_type say which precision the accumulator lives in.
// (f16, f16): accumulates in binary16 like wmma's .f16.f16 form; every other combination
// accumulates in binary32 and rounds d once if d is binary16.
__device__ __forceinline__ void warp_mma(const __half (&a)[8], const __half (&b)[8], const float (&c)[8],
                                         int c_type, int d_type, float (&d)[8]) {
    uint32_t ar[4] = {pack2(a[0], a[1]), pack2(a[2], a[3]), pack2(a[4], a[5]), pack2(a[6], a[7])};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
        uint32_t br[2] = {pack2(b[nb * 4 + 0], b[nb * 4 + 1]), pack2(b[nb * 4 + 2], b[nb * 4 + 3])};
        if (c_type == B200_F16 && d_type == B200_F16) {
            uint32_t cr[2] = {pack2(__float2half_rn(c[nb * 4 + 0]), __float2half_rn(c[nb * 4 + 1])),
                              pack2(__float2half_rn(c[nb * 4 + 2]), __float2half_rn(c[nb * 4 + 3]))};
            uint32_t dr[2];
            mma_16x8x16_f16(dr, ar, br, cr);
            d[nb * 4 + 0] = __half2float(__ushort_as_half(static_cast<unsigned short>(dr[0] & 0xffff)));
            d[nb * 4 + 1] = __half2float(__ushort_as_half(static_cast<unsigned short>(dr[0] >> 16)));
            d[nb * 4 + 2] = __half2float(__ushort_as_half(static_cast<unsigned short>(dr[1] & 0xffff)));
            d[nb * 4 + 3] = __half2float(__ushort_as_half(static_cast<unsigned short>(dr[1] >> 16)));
        } else {
            float cr[4] = {c[nb * 4 + 0], c[nb * 4 + 1], c[nb * 4 + 2], c[nb * 4 + 3]};
            float dr[4];
            mma_16x8x16_f32(dr, ar, br, cr);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                d[nb * 4 + i] = d_type == B200_F16 ? __half2float(__float2half_rn(dr[i])) : dr[i];
        }
    }
}

}  // namespace b200
