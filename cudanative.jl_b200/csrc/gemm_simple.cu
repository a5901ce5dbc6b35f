// Plain shared-memory GEMM (FP32 FMA on CUDA cores) and the synthetic-matrix fill kernels.
//
// The simple kernel takes any shape, leading dimension and alignment, so it backs the shapes the
// TMA path cannot address (unaligned pointers, K == 0) and serves as an independent on-device
// check of the tcgen05 kernel at sizes a CPU product would take minutes for.  Products of two
// binary16 (or bfloat16) values are exact in binary32, so it differs from the tensor-core result
// only in the order of the FP32 additions.  Batched problems put the matrix index in blockIdx.z.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "rng.cuh"

namespace b200 {
namespace {

constexpr int kTile = 64;   // output tile per block
constexpr int kTileK = 16;  // k per shared-memory step

struct SimpleBatch {
    int64_t count, stride_a, stride_b, stride_c, stride_d;  // strides in elements
};

// 16-bit storage -> binary32: bfloat16 is the upper half of a binary32
__device__ __forceinline__ float widen16(unsigned short raw, int bf16) {
    return bf16 ? __uint_as_float(static_cast<uint32_t>(raw) << 16) : __half2float(__ushort_as_half(raw));
}

template <bool kTransA, bool kTransB>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(int64_t M, int64_t N, int64_t K, float alpha, const unsigned short* __restrict__ A0, int64_t lda,
                   const unsigned short* __restrict__ B0, int64_t ldb, float beta, const void* Cv0, int64_t ldc,
                   void* Dv0, int64_t ldd, int ab_bf16, int c_fmt, int d_fmt, SimpleBatch batch) {
  for (int64_t bz = blockIdx.z; bz < batch.count; bz += gridDim.z) {
    const unsigned short* A = A0 + bz * batch.stride_a;
    const unsigned short* B = B0 + bz * batch.stride_b;
    const int c_bytes = c_fmt == 0 ? 4 : 2, d_bytes = d_fmt == 0 ? 4 : 2;
    const void* Cv = static_cast<const char*>(Cv0) + bz * batch.stride_c * c_bytes;
    void* Dv = static_cast<char*>(Dv0) + bz * batch.stride_d * d_bytes;
    const float* C = static_cast<const float*>(Cv);
    float* D = static_cast<float*>(Dv);
    const unsigned short* Ch = static_cast<const unsigned short*>(Cv);
    __half* Dh = static_cast<__half*>(Dv);
    __nv_bfloat16* Db = static_cast<__nv_bfloat16*>(Dv);
    __shared__ float sA[kTileK][kTile + 1];
    __shared__ float sB[kTileK][kTile + 1];
    const int tx = threadIdx.x & 15;  // 4 rows each
    const int ty = threadIdx.x >> 4;  // 4 cols each
    const int64_t m0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * kTile;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < K; k0 += kTileK) {
        for (int e = threadIdx.x; e < kTile * kTileK; e += 256) {
            int mm, kk;
            if (kTransA) { kk = e % kTileK; mm = e / kTileK; } else { mm = e % kTile; kk = e / kTile; }
            const int64_t m = m0 + mm, k = k0 + kk;
            float v = 0.f;
            if (m < M && k < K) v = widen16(kTransA ? A[k + m * lda] : A[m + k * lda], ab_bf16);
            sA[kk][mm] = v;
        }
        for (int e = threadIdx.x; e < kTile * kTileK; e += 256) {
            int nn, kk;
            if (kTransB) { nn = e % kTile; kk = e / kTile; } else { kk = e % kTileK; nn = e / kTileK; }
            const int64_t n = n0 + nn, k = k0 + kk;
            float v = 0.f;
            if (n < N && k < K) v = widen16(kTransB ? B[n + k * ldb] : B[k + n * ldb], ab_bf16);
            sB[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTileK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[kk][tx * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sB[kk][ty * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t n = n0 + ty * 4 + j;
        if (n >= N) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t m = m0 + tx * 4 + i;
            if (m >= M) continue;
            float v = alpha * acc[i][j];
            if (beta != 0.0f) v = fmaf(beta, c_fmt ? widen16(Ch[m + n * ldc], c_fmt == 2) : C[m + n * ldc], v);
            if (d_fmt == 2) Db[m + n * ldd] = __float2bfloat16_rn(v);
            else if (d_fmt == 1) Dh[m + n * ldd] = __float2half_rn(v);
            else D[m + n * ldd] = v;
        }
    }
    __syncthreads();  // the shared tiles are reused by the next matrix of the batch
  }
}

template <typename T>
__global__ void fill_kernel(T* out, int64_t rows, int64_t cols, int64_t ld, uint64_t seed, uint64_t matrix_id,
                            uint64_t index0, int dist, float scale) {
    const int64_t total = rows * cols;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t j = idx / rows, i = idx - j * rows;
        const float v = synth_value(seed, matrix_id, index0 + static_cast<uint64_t>(idx), dist) * scale;
        if constexpr (sizeof(T) == 4) out[i + j * ld] = v;
        else out[i + j * ld] = T(v);  // __half and __nv_bfloat16 convert with round-to-nearest-even
    }
}

template <typename T>
int fill_launch(cudaStream_t stream, T* dptr, int64_t rows, int64_t cols, int64_t ld, uint64_t seed,
                uint64_t matrix_id, uint64_t index0, int dist, float scale) {
    if (rows < 0 || cols < 0 || ld < rows || (rows * cols > 0 && !dptr)) return fail(B200_INVALID_ARG, "fill: bad matrix");
    if (dist < 0 || dist > 2) return fail(B200_INVALID_ARG, "fill: dist must be 0 (uniform), 1 (normal) or 2 (zeros)");
    const int64_t total = rows * cols;
    if (total == 0) return B200_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fill_kernel<T><<<static_cast<int>(blocks), 256, 0, stream>>>(dptr, rows, cols, ld, seed, matrix_id, index0, dist, scale);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace

int gemm_simple_launch(const GemmProblem& g, cudaStream_t stream, LaunchInfo* info) {
    if (g.M == 0 || g.N == 0) return B200_OK;
    const int64_t gx = (g.M + kTile - 1) / kTile, gy = (g.N + kTile - 1) / kTile;
    if (gy > 65535) return fail(B200_UNSUPPORTED, "simple kernel: N too large for one launch");
    const int64_t count = g.batch > 1 ? g.batch : 1;
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(count < 1024 ? count : 1024));
    const unsigned short* A = static_cast<const unsigned short*>(g.A);
    const unsigned short* B = static_cast<const unsigned short*>(g.B);
    const SimpleBatch batch = {count, g.stride_a, g.stride_b, g.stride_c, g.stride_d};
#define B200_SIMPLE(TA, TB) \
    gemm_simple_kernel<TA, TB><<<grid, 256, 0, stream>>>(g.M, g.N, g.K, g.alpha, A, g.lda, B, g.ldb, g.beta, g.C, g.ldc, g.D, g.ldd, \
                                                         g.ab_type == B200_BF16 ? 1 : 0, elem_fmt(g.c_type), elem_fmt(g.d_type), batch)
    if (g.transA) { if (g.transB) B200_SIMPLE(true, true); else B200_SIMPLE(true, false); }
    else          { if (g.transB) B200_SIMPLE(false, true); else B200_SIMPLE(false, false); }
#undef B200_SIMPLE
    B200_CUDA_TRY(cudaGetLastError());
    if (info) {
        info->kernel = B200_KERNEL_SIMPLE;
        info->tile_n = kTile;
        info->split_k = 1;
        info->ctas = static_cast<int>(gx * gy * grid.z);
        info->cta_pair = 1;
    }
    return B200_OK;
}

int gemm_simple_preload() {
    cudaFuncAttributes at;
    B200_CUDA_TRY(cudaFuncGetAttributes(&at, gemm_simple_kernel<false, false>));
    B200_CUDA_TRY(cudaFuncGetAttributes(&at, gemm_simple_kernel<false, true>));
    B200_CUDA_TRY(cudaFuncGetAttributes(&at, gemm_simple_kernel<true, false>));
    B200_CUDA_TRY(cudaFuncGetAttributes(&at, gemm_simple_kernel<true, true>));
    return B200_OK;
}

}  // namespace b200

extern "C" int b200_fill_f16(b200_stream stream, void* dptr, int64_t rows, int64_t cols, int64_t ld, uint64_t seed,
                             uint64_t matrix_id, uint64_t index0, int dist, float scale) {
    return b200::fill_launch<__half>(static_cast<cudaStream_t>(stream), static_cast<__half*>(dptr), rows, cols, ld,
                                     seed, matrix_id, index0, dist, scale);
}

extern "C" int b200_fill_f32(b200_stream stream, float* dptr, int64_t rows, int64_t cols, int64_t ld, uint64_t seed,
                             uint64_t matrix_id, uint64_t index0, int dist, float scale) {
    return b200::fill_launch<float>(static_cast<cudaStream_t>(stream), dptr, rows, cols, ld, seed, matrix_id, index0,
                                    dist, scale);
}

extern "C" int b200_fill_bf16(b200_stream stream, void* dptr, int64_t rows, int64_t cols, int64_t ld, uint64_t seed,
                              uint64_t matrix_id, uint64_t index0, int dist, float scale) {
    return b200::fill_launch<__nv_bfloat16>(static_cast<cudaStream_t>(stream), static_cast<__nv_bfloat16*>(dptr), rows,
                                            cols, ld, seed, matrix_id, index0, dist, scale);
}
