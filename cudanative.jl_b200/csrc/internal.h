// Declarations shared by the translation units of libb200wmma.so (host side only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

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
    // accumulate in binary16 instead of binary32 (tcgen05 kernel only; Float16 A, B, C and D)
    int acc_f16 = 0;
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
    int pdl = 1;       // launch with programmatic stream serialization
};

struct LaunchInfo {
    int kernel, tile_n, split_k, ctas, cta_pair;
};

}  // namespace b200

// The per-device handle behind the C ABI (opaque to callers).
struct b200_handle {
    int device = 0;
    int sm_count = 0;
    int* status_word = nullptr;  // 4 ints on the device
    // options
    int force_kernel = B200_KERNEL_AUTO;
    int max_ctas = 0;
    unsigned long long wait_budget_ns = 2000000000ull;
    int tile_n = 0;
    int split_k = 0;
    int cta_pair = 0;
    int raster_group = 0;
    int check_on_call = 0;
    int pdl = 1;
    int f16_accumulate = 0;
    // workspace of the host-buffer entry point and split-K scratch (grown on demand)
    void* ws[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t ws_bytes[4] = {0, 0, 0, 0};
    float* scratch = nullptr;
    size_t scratch_bytes = 0;
    cudaStream_t streams[3] = {nullptr, nullptr, nullptr};  // upload / multiply / download
    std::vector<cudaEvent_t> events;
    b200::LaunchInfo last = {0, 0, 0, 0, 0};
    // "check on the next call" (B200_OPT_CHECK_ON_CALL): the stream of the previous launch, and an
    // event recorded behind it
    cudaEvent_t last_done = nullptr;
    bool last_pending = false;
    // status-word reads go through a private non-blocking stream and a page-locked word, so that they
    // never wait for unrelated work of the caller (a plain cudaMemcpy joins the legacy default stream)
    cudaStream_t poll_stream = nullptr;
    int* host_word = nullptr;
};

namespace b200 {

// Validate, pick a kernel and enqueue one GEMM on `stream` (the body of every GEMM entry point).
int gemm_dispatch(b200_handle* h, cudaStream_t stream, const GemmProblem& g);
int check_current_device(const b200_handle* h);
// Copies the handle's 4-int device status word to `word` (synchronous) and clears it when non-zero.
int read_status(b200_handle* h, int* word);

// Scratch needed for the plan's split-K partials, in bytes (0 when split_k == 1).
size_t gemm_tcgen05_scratch_bytes(const GemmProblem& g, const GemmPlan& plan);

// True when the TMA/tcgen05 kernel can take the problem (alignment, sizes).
bool gemm_tcgen05_eligible(const GemmProblem& g, std::string* why);

// Enqueue the tcgen05 GEMM (and the split-K reduction when plan.split_k > 1).
int gemm_tcgen05_launch(const GemmProblem& g, const GemmPlan& plan, float* scratch, int* status_word,
                        int sm_count, cudaStream_t stream, LaunchInfo* info);

// Loads every non-batched instantiation of the tcgen05 kernel and the split-K reduction on the current
// device and opts them in to their shared memory, so that no later launch does it.
int gemm_tcgen05_preload();

// Makes the driver load the plain kernel's four layout variants on the current device.
int gemm_simple_preload();

// Enqueue the plain shared-memory kernel: any shape, any alignment.
int gemm_simple_launch(const GemmProblem& g, cudaStream_t stream, LaunchInfo* info);

}  // namespace b200
