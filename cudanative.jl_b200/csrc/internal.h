// Declarations shared by the translation units of libb200wmma.so (host side only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/b200wmma.h"

namespace b200 {

// thread-local error text behind b200_last_error()
void set_error(const std::string& msg);
int fail(int status, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define B200_CUDA_TRY(expr)                                  \
    do {                                                     \
        cudaError_t e__ = (expr);                            \
        if (e__ != cudaSuccess) return cuda_fail(e__, #expr); \
    } while (0)

struct GemmProblem {
    int transA, transB;
    int64_t M, N, K;
    float alpha, beta;
    const void* A;
    int64_t lda;
    const void* B;
    int64_t ldb;
    const float* C;
    int64_t ldc;
    float* D;
    int64_t ldd;
    // gated A (optional): columns [j * panel_k, (j + 1) * panel_k) of op(A) may be read only once
    // panel_flags[j] != 0; panel_k is a multiple of 64
    const unsigned int* panel_flags = nullptr;
    int64_t panel_k = 0;
    // element types of C and D in memory (B200_F32 by default); when B200_F16, the C / D pointers
    // above point at binary16 data and ldc / ldd count binary16 elements
    int c_type = B200_F32;
    int d_type = B200_F32;
    // element type of A and B: B200_F16 or B200_BF16 (both operands the same)
    int ab_type = B200_F16;
    // batched problems: `batch` independent products; matrix i of X starts stride_x * i elements after
    // X (a stride of 0 repeats the matrix).  batch == 1 ignores the strides.
    int64_t batch = 1;
    int64_t stride_a = 0, stride_b = 0, stride_c = 0, stride_d = 0;
};

inline int elem_bytes(int type) { return type == B200_F32 ? 4 : 2; }
// 0 = binary32, 1 = binary16, 2 = bfloat16: the encoding the kernels take
inline int elem_fmt(int type) { return type == B200_F32 ? 0 : (type == B200_F16 ? 1 : 2); }

struct GemmPlan {
    int tile_n;    // 64 / 128 / 256
    int cta_pair;  // 1 or 2 CTAs per tile
    int split_k;   // >= 1
    int max_ctas;  // grid cap (0 = SM count)
    int raster_group;  // 0 = default
    unsigned long long wait_budget_ns;
};

struct LaunchInfo {
    int kernel, tile_n, split_k, ctas, cta_pair;
};

// Scratch needed for the plan's split-K partials, in bytes (0 when split_k == 1).
size_t gemm_tcgen05_scratch_bytes(const GemmProblem& g, const GemmPlan& plan);

// True when the TMA/tcgen05 kernel can take the problem (alignment, sizes).
bool gemm_tcgen05_eligible(const GemmProblem& g, std::string* why);

// Enqueue the tcgen05 GEMM (and the split-K reduction when plan.split_k > 1).
int gemm_tcgen05_launch(const GemmProblem& g, const GemmPlan& plan, float* scratch, int* status_word,
                        int sm_count, cudaStream_t stream, LaunchInfo* info);

// Enqueue the plain shared-memory kernel: any shape, any alignment.
int gemm_simple_launch(const GemmProblem& g, cudaStream_t stream, LaunchInfo* info);

}  // namespace b200
