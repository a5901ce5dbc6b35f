// C ABI of libb200wmma.so: handle, errors, options, GEMM dispatch, host-buffer path, memory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <vector>
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200 {

// One warp waits on an mbarrier that nothing ever arrives on: exercises the bounded-wait path
// (budget expiry -> status word -> clean exit) without any fault, trap or endless loop.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long budget_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    WaitCtx wc{&abort_flag, status, budget_ns};
    mbar_wait(smem_u32(&bar), 0, wc, kWaitSelftest);
}

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int status, const std::string& msg) {
    g_last_error = msg;
    return status;
}
int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return B200_CUDA_ERROR;
}

}  // namespace b200

using namespace b200;

namespace b200 {

int ensure_buffer(void** p, size_t* have, size_t need) {
    if (need <= *have) return B200_OK;
    if (*p) {
        B200_CUDA_TRY(cudaFree(*p));
        *p = nullptr;
        *have = 0;
    }
    B200_CUDA_TRY(cudaMalloc(p, need));
    *have = need;
    return B200_OK;
}

int validate(const GemmProblem& g) {
    if (g.M < 0 || g.N < 0 || g.K < 0) return fail(B200_INVALID_ARG, "gemm: negative dimension");
    if ((g.transA != 0 && g.transA != 1) || (g.transB != 0 && g.transB != 1))
        return fail(B200_INVALID_ARG, "gemm: transA / transB must be 0 or 1");
    const int64_t a_rows = g.transA ? g.K : g.M, b_rows = g.transB ? g.N : g.K;
    if (g.lda < std::max<int64_t>(1, a_rows)) return fail(B200_INVALID_ARG, "gemm: lda smaller than the rows of stored A");
    if (g.ldb < std::max<int64_t>(1, b_rows)) return fail(B200_INVALID_ARG, "gemm: ldb smaller than the rows of stored B");
    if (g.ldd < std::max<int64_t>(1, g.M)) return fail(B200_INVALID_ARG, "gemm: ldd smaller than M");
    if (g.batch < 0) return fail(B200_INVALID_ARG, "gemm: negative batch count");
    if (g.batch > 1) {
        if (g.stride_a < 0 || g.stride_b < 0 || g.stride_c < 0 || g.stride_d < 0)
            return fail(B200_INVALID_ARG, "gemm: negative batch stride");
        if (g.stride_d < g.ldd * g.N) return fail(B200_INVALID_ARG, "gemm: stride_d smaller than one D matrix (results would overlap)");
    }
    if (g.beta != 0.0f && g.ldc < std::max<int64_t>(1, g.M)) return fail(B200_INVALID_ARG, "gemm: ldc smaller than M");
    if (g.M > 0 && g.N > 0) {
        if (!g.D) return fail(B200_INVALID_ARG, "gemm: D is null");
        if (g.beta != 0.0f && !g.C) return fail(B200_INVALID_ARG, "gemm: C is null but beta != 0");
        if (g.K > 0 && (!g.A || !g.B)) return fail(B200_INVALID_ARG, "gemm: A or B is null");
    }
    return B200_OK;
}

// Tile shape and split heuristics.  Big square-ish problems take 2-CTA 256 x 256 tiles; narrow N
// takes the narrowest tile that covers it, paired along M when there are rows enough.
GemmPlan make_plan(const b200_handle* h, const GemmProblem& g) {
    GemmPlan plan;
    plan.max_ctas = h->max_ctas;
    plan.raster_group = h->raster_group;
    plan.wait_budget_ns = h->wait_budget_ns;
    plan.pdl = h->pdl;
    int tile_n = h->tile_n;
    if (tile_n == 0) tile_n = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);
    int pair = h->cta_pair;
    // 2-CTA tiles halve the B traffic per SM and pay off once the tile is 256 columns wide;
    // narrow (HBM-bound) problems stream better with independent CTAs.
    if (pair == 0) pair = (g.M > 128 && tile_n == 256) ? 2 : 1;
    if (pair == 2 && tile_n < 128) pair = 1;
    if (g.transB && (tile_n / pair) % 64) pair = 1;  // row-major B loads 64 columns per box
    plan.tile_n = tile_n;
    plan.cta_pair = pair;
    plan.split_k = h->split_k > 0 ? h->split_k : 1;
    return plan;
}

// The handle's status word and scratch live on its device and the launch goes to the calling
// thread's current device: the two must be the same.
int check_current_device(const b200_handle* h) {
    int cur = -1;
    B200_CUDA_TRY(cudaGetDevice(&cur));
    if (cur != h->device)
        return fail(B200_INVALID_ARG, "the handle belongs to device " + std::to_string(h->device) +
                                          " but the calling thread's current device is " + std::to_string(cur));
    return B200_OK;
}

int gemm_dispatch(b200_handle* h, cudaStream_t stream, const GemmProblem& g) {
    int rc = validate(g);
    if (rc) return rc;
    if (g.M == 0 || g.N == 0 || g.batch == 0) return B200_OK;
    if ((rc = check_current_device(h))) return rc;
    std::string why;
    const bool eligible = gemm_tcgen05_eligible(g, &why);
    if (g.acc_f16) {
        // only the tensor-core kernel has a binary16 accumulator; the plain kernel and the split-K reduction sum in binary32
        if (!eligible) return fail(B200_UNSUPPORTED, "Float16 accumulation needs the tcgen05 kernel: " + why);
        if (g.K == 0) return fail(B200_UNSUPPORTED, "Float16 accumulation needs K > 0");
        if (h->force_kernel == B200_KERNEL_SIMPLE) return fail(B200_UNSUPPORTED, "Float16 accumulation: the plain kernel accumulates in Float32");
        GemmPlan plan = make_plan(h, g);
        plan.split_k = 1;
        return gemm_tcgen05_launch(g, plan, nullptr, h->status_word, h->sm_count, stream, &h->last);
    }
    int kernel = h->force_kernel;
    const int64_t m_quant = 16 / elem_bytes(g.d_type);
    if (kernel == B200_KERNEL_AUTO && !eligible && (g.M % m_quant) && g.M > m_quant && !g.panel_flags) {
        // Only the row count stands in the way: give the rows that fill whole 16-byte store chunks to
        // the tensor-core kernel and the last few rows to the plain kernel.
        GemmProblem top = g, strip = g;
        top.M = g.M - g.M % m_quant;
        if (gemm_tcgen05_eligible(top, nullptr)) {
            strip.M = g.M % m_quant;
            const int64_t skip = top.M;
            strip.A = static_cast<const char*>(g.A) + 2 * (g.transA ? skip * g.lda : skip);
            if (g.C) strip.C = reinterpret_cast<const float*>(reinterpret_cast<const char*>(g.C) + skip * elem_bytes(g.c_type));
            strip.D = reinterpret_cast<float*>(reinterpret_cast<char*>(g.D) + skip * elem_bytes(g.d_type));
            if ((rc = gemm_simple_launch(strip, stream, nullptr))) return rc;
            return gemm_dispatch(h, stream, top);
        }
    }
    if (kernel == B200_KERNEL_AUTO && !eligible && g.batch > 1) {
        // The batch cannot run as one TMA launch (strides).  If a single matrix can, multiply them one
        // launch each; otherwise all of them go to the plain kernel in one launch.
        GemmProblem one = g;
        one.batch = 1;
        bool one_ok = gemm_tcgen05_eligible(one, nullptr);
        if (!one_ok && (g.M % m_quant) && g.M > m_quant) {
            one.M = g.M - g.M % m_quant;
            one_ok = gemm_tcgen05_eligible(one, nullptr);
            one.M = g.M;
        }
        if (one_ok) {
            for (int64_t i = 0; i < g.batch; ++i) {
                one.A = static_cast<const char*>(g.A) + 2 * i * g.stride_a;
                one.B = static_cast<const char*>(g.B) + 2 * i * g.stride_b;
                if (g.C) one.C = reinterpret_cast<const float*>(reinterpret_cast<const char*>(g.C) + i * g.stride_c * elem_bytes(g.c_type));
                one.D = reinterpret_cast<float*>(reinterpret_cast<char*>(g.D) + i * g.stride_d * elem_bytes(g.d_type));
                if ((rc = gemm_dispatch(h, stream, one))) return rc;
            }
            return B200_OK;
        }
    }
    if (kernel == B200_KERNEL_AUTO) kernel = eligible ? B200_KERNEL_TCGEN05 : B200_KERNEL_SIMPLE;
    if (kernel == B200_KERNEL_TCGEN05) {
        if (!eligible) return fail(B200_UNSUPPORTED, "tcgen05 kernel not eligible: " + why);
        GemmPlan plan = make_plan(h, g);
        const size_t need = gemm_tcgen05_scratch_bytes(g, plan);
        if (need) {
            void* p = h->scratch;
            rc = ensure_buffer(&p, &h->scratch_bytes, need);
            h->scratch = static_cast<float*>(p);
            if (rc) return rc;
        }
        return gemm_tcgen05_launch(g, plan, h->scratch, h->status_word, h->sm_count, stream, &h->last);
    }
    if (kernel == B200_KERNEL_SIMPLE) return gemm_simple_launch(g, stream, &h->last);
    return fail(B200_INVALID_ARG, "unknown kernel selector");
}

int read_status(b200_handle* h, int* word) {
    if (!h->poll_stream) B200_CUDA_TRY(cudaStreamCreateWithFlags(&h->poll_stream, cudaStreamNonBlocking));
    if (!h->host_word) B200_CUDA_TRY(cudaHostAlloc(reinterpret_cast<void**>(&h->host_word), 4 * sizeof(int), cudaHostAllocDefault));
    B200_CUDA_TRY(cudaMemcpyAsync(h->host_word, h->status_word, 4 * sizeof(int), cudaMemcpyDeviceToHost, h->poll_stream));
    B200_CUDA_TRY(cudaStreamSynchronize(h->poll_stream));
    for (int i = 0; i < 4; ++i) word[i] = h->host_word[i];
    if (word[0] != 0) {
        B200_CUDA_TRY(cudaMemsetAsync(h->status_word, 0, 4 * sizeof(int), h->poll_stream));
        B200_CUDA_TRY(cudaStreamSynchronize(h->poll_stream));
    }
    return B200_OK;
}

// B200_OPT_CHECK_ON_CALL: what the reference does in prepare_cuda_call (src/init.jl:37 ->
// src/exceptions.jl:76-89 of CUDAnative.jl) -- before new work is enqueued, look at the failure
// flag of work that has already finished.  Only a launch that is known to be complete is looked
// at (event query), so the call never waits for the GPU.
int poll_previous_launch(b200_handle* h) {
    if (!h->check_on_call || !h->last_pending) return B200_OK;
    cudaError_t e = cudaEventQuery(h->last_done);
    if (e == cudaErrorNotReady) return B200_OK;
    if (e != cudaSuccess) return cuda_fail(e, "cudaEventQuery(previous launch)");
    h->last_pending = false;
    int word[4] = {0, 0, 0, 0};
    int rc = read_status(h, word);
    if (rc) return rc;
    if (word[0] != 0)
        return fail(B200_DEVICE_TIMEOUT, "a bounded wait ran out on the device in an earlier launch of this handle (wait id " +
                                             std::to_string(word[0]) + ", block " + std::to_string(word[1]) +
                                             "); its result is not valid.  This call enqueued nothing.");
    return B200_OK;
}

int note_launch(b200_handle* h, cudaStream_t stream) {
    if (!h->check_on_call) return B200_OK;
    if (!h->last_done) B200_CUDA_TRY(cudaEventCreateWithFlags(&h->last_done, cudaEventDisableTiming));
    B200_CUDA_TRY(cudaEventRecord(h->last_done, stream));
    h->last_pending = true;
    return B200_OK;
}

// What every GEMM entry point of the C ABI runs: optional poll of the previous launch, dispatch,
// bookkeeping for the next poll.
int gemm_entry(b200_handle* h, cudaStream_t stream, const GemmProblem& g) {
    int rc = poll_previous_launch(h);
    if (rc) return rc;
    if ((rc = gemm_dispatch(h, stream, g))) return rc;
    return note_launch(h, stream);
}

}  // namespace b200

extern "C" {

const char* b200_last_error(void) { return g_last_error.c_str(); }

const char* b200_status_string(int status) {
    switch (status) {
        case B200_OK: return "B200_OK";
        case B200_INVALID_ARG: return "B200_INVALID_ARG";
        case B200_UNSUPPORTED: return "B200_UNSUPPORTED";
        case B200_CUDA_ERROR: return "B200_CUDA_ERROR";
        case B200_DEVICE_TIMEOUT: return "B200_DEVICE_TIMEOUT";
        case B200_NO_DEVICE: return "B200_NO_DEVICE";
        case B200_PEER_TIMEOUT: return "B200_PEER_TIMEOUT";
        default: return "B200_UNKNOWN_STATUS";
    }
}

int b200_version(void) { return 100; }

int b200_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDeviceCount");
        return -B200_CUDA_ERROR;
    }
    int good = 0;
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10) ++good;
    }
    return good;
}

int b200_create(b200_handle** out, int device) {
    if (!out) return fail(B200_INVALID_ARG, "b200_create: out is null");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(B200_NO_DEVICE, std::string("b200_create: no CUDA device (") + cudaGetErrorString(e) + ")");
    }
    if (device < 0 || device >= n) return fail(B200_INVALID_ARG, "b200_create: device index out of range");
    int major = 0, minor = 0, sms = 0;
    B200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    if (major != 10)
        return fail(B200_NO_DEVICE, "b200_create: device has compute capability " + std::to_string(major) + "." +
                                        std::to_string(minor) + ", this library holds sm_100a code only");
    B200_CUDA_TRY(cudaSetDevice(device));
    b200_handle* h = new b200_handle();
    h->device = device;
    h->sm_count = sms;
    if (cudaMalloc(&h->status_word, 4 * sizeof(int)) != cudaSuccess || cudaMemset(h->status_word, 0, 4 * sizeof(int)) != cudaSuccess) {
        int rc = cuda_fail(cudaGetLastError(), "b200_create: status word");
        delete h;
        return rc;
    }
    *out = h;
    return B200_OK;
}

int b200_destroy(b200_handle* h) {
    if (!h) return B200_OK;
    cudaSetDevice(h->device);
    for (int i = 0; i < 4; ++i)
        if (h->ws[i]) cudaFree(h->ws[i]);
    if (h->scratch) cudaFree(h->scratch);
    if (h->status_word) cudaFree(h->status_word);
    for (int i = 0; i < 3; ++i)
        if (h->streams[i]) cudaStreamDestroy(h->streams[i]);
    for (cudaEvent_t e : h->events) cudaEventDestroy(e);
    if (h->last_done) cudaEventDestroy(h->last_done);
    if (h->poll_stream) cudaStreamDestroy(h->poll_stream);
    if (h->host_word) cudaFreeHost(h->host_word);
    delete h;
    return B200_OK;
}

int b200_set_option(b200_handle* h, int option, int64_t value) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    switch (option) {
        case B200_OPT_FORCE_KERNEL:
            if (value < B200_KERNEL_AUTO || value > B200_KERNEL_SIMPLE) return fail(B200_INVALID_ARG, "unknown kernel selector");
            h->force_kernel = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_MAX_CTAS:
            if (value < 0) return fail(B200_INVALID_ARG, "max CTAs must be >= 0");
            h->max_ctas = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_WAIT_BUDGET_NS:
            if (value < 1000) return fail(B200_INVALID_ARG, "wait budget below 1 us");
            h->wait_budget_ns = static_cast<unsigned long long>(value);
            return B200_OK;
        case B200_OPT_TILE_N:
            if (value != 0 && value != 64 && value != 128 && value != 256) return fail(B200_INVALID_ARG, "tile_n must be 0, 64, 128 or 256");
            h->tile_n = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_SPLIT_K:
            if (value < 0 || value > 64) return fail(B200_INVALID_ARG, "split_k must be in [0, 64]");
            h->split_k = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_CTA_PAIR:
            if (value < 0 || value > 2) return fail(B200_INVALID_ARG, "cta_pair must be 0, 1 or 2");
            h->cta_pair = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_RASTER_GROUP:
            if (value < 0 || value > 4096) return fail(B200_INVALID_ARG, "raster group must be in [0, 4096]");
            h->raster_group = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_CHECK_ON_CALL:
            if (value != 0 && value != 1) return fail(B200_INVALID_ARG, "check_on_call must be 0 or 1");
            h->check_on_call = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_PDL:
            if (value != 0 && value != 1) return fail(B200_INVALID_ARG, "pdl must be 0 or 1");
            h->pdl = static_cast<int>(value);
            return B200_OK;
        case B200_OPT_F16_ACCUMULATE:
            if (value != 0 && value != 1) return fail(B200_INVALID_ARG, "f16_accumulate must be 0 or 1");
            h->f16_accumulate = static_cast<int>(value);
            return B200_OK;
        default:
            return fail(B200_INVALID_ARG, "unknown option");
    }
}

int b200_get_option(b200_handle* h, int option, int64_t* value) {
    if (!h || !value) return fail(B200_INVALID_ARG, "null handle or value");
    switch (option) {
        case B200_OPT_FORCE_KERNEL: *value = h->force_kernel; return B200_OK;
        case B200_OPT_MAX_CTAS: *value = h->max_ctas; return B200_OK;
        case B200_OPT_WAIT_BUDGET_NS: *value = static_cast<int64_t>(h->wait_budget_ns); return B200_OK;
        case B200_OPT_TILE_N: *value = h->tile_n; return B200_OK;
        case B200_OPT_SPLIT_K: *value = h->split_k; return B200_OK;
        case B200_OPT_CTA_PAIR: *value = h->cta_pair; return B200_OK;
        case B200_OPT_RASTER_GROUP: *value = h->raster_group; return B200_OK;
        case B200_OPT_CHECK_ON_CALL: *value = h->check_on_call; return B200_OK;
        case B200_OPT_PDL: *value = h->pdl; return B200_OK;
        case B200_OPT_F16_ACCUMULATE: *value = h->f16_accumulate; return B200_OK;
        default: return fail(B200_INVALID_ARG, "unknown option");
    }
}

int b200_device_status(b200_handle* h, int* code, int* block, int* detail) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    int word[4] = {0, 0, 0, 0};
    int rc = read_status(h, word);
    if (rc) return rc;
    if (code) *code = word[0];
    if (block) *block = word[1];
    if (detail) *detail = word[2];
    return B200_OK;
}

int b200_selftest_bounded_wait(b200_handle* h, b200_stream stream, int64_t budget_ns) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    if (budget_ns < 1000 || budget_ns > 1000000000ll) return fail(B200_INVALID_ARG, "selftest budget must be within [1 us, 1 s]");
    if (int rc = check_current_device(h)) return rc;
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(h->status_word, static_cast<unsigned long long>(budget_ns));
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_last_launch(b200_handle* h, int* kernel, int* tile_n, int* split_k, int* ctas, int* cta_pair) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    if (kernel) *kernel = h->last.kernel;
    if (tile_n) *tile_n = h->last.tile_n;
    if (split_k) *split_k = h->last.split_k;
    if (ctas) *ctas = h->last.ctas;
    if (cta_pair) *cta_pair = h->last.cta_pair;
    return B200_OK;
}

int b200_gemm_f16f32(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N, int64_t K,
                     float alpha, const void* A, int64_t lda, const void* B, int64_t ldb, float beta, const float* C,
                     int64_t ldc, float* D, int64_t ldd) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    GemmProblem g{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, D, ldd};
    return gemm_entry(h, static_cast<cudaStream_t>(stream), g);
}

int b200_gemm_f16_typed(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N, int64_t K,
                        float alpha, const void* A, int64_t lda, const void* B, int64_t ldb, float beta, const void* C,
                        int64_t ldc, int c_type, void* D, int64_t ldd, int d_type) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    if ((c_type != B200_F16 && c_type != B200_F32) || (d_type != B200_F16 && d_type != B200_F32))
        return fail(B200_INVALID_ARG, "invalid element type for WMMA: C and D must be Float16 or Float32");
    GemmProblem g{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, static_cast<const float*>(C), ldc,
                  static_cast<float*>(D), ldd};
    g.c_type = c_type;
    g.d_type = d_type;
    // Config{16, 16, 16, Float16} with a Float16 C: the .f16.f16 mma variants of the reference
    // (src/device/cuda/wmma.jl:222-257) accumulate in binary16
    g.acc_f16 = (h->f16_accumulate && c_type == B200_F16 && d_type == B200_F16) ? 1 : 0;
    return gemm_entry(h, static_cast<cudaStream_t>(stream), g);
}

namespace {
bool is_elem_type(int t) { return t == B200_F16 || t == B200_F32 || t == B200_BF16; }
}  // namespace

int b200_gemm_strided_batched(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N,
                              int64_t K, float alpha, const void* A, int64_t lda, int64_t stride_a, const void* B,
                              int64_t ldb, int64_t stride_b, int ab_type, float beta, const void* C, int64_t ldc,
                              int64_t stride_c, int c_type, void* D, int64_t ldd, int64_t stride_d, int d_type,
                              int64_t batch) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    if (ab_type != B200_F16 && ab_type != B200_BF16)
        return fail(B200_INVALID_ARG, "invalid element type: A and B must be Float16 or bfloat16");
    if (!is_elem_type(c_type) || !is_elem_type(d_type))
        return fail(B200_INVALID_ARG, "invalid element type: C and D must be Float16, bfloat16 or Float32");
    GemmProblem g{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, static_cast<const float*>(C), ldc,
                  static_cast<float*>(D), ldd};
    g.c_type = c_type;
    g.d_type = d_type;
    g.ab_type = ab_type;
    g.batch = batch;
    g.stride_a = stride_a;
    g.stride_b = stride_b;
    g.stride_c = stride_c;
    g.stride_d = stride_d;
    return gemm_entry(h, static_cast<cudaStream_t>(stream), g);
}

int b200_gemm_ex(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N, int64_t K,
                 float alpha, const void* A, int64_t lda, const void* B, int64_t ldb, int ab_type, float beta,
                 const void* C, int64_t ldc, int c_type, void* D, int64_t ldd, int d_type) {
    return b200_gemm_strided_batched(h, stream, transA, transB, M, N, K, alpha, A, lda, 0, B, ldb, 0, ab_type, beta, C,
                                     ldc, 0, c_type, D, ldd, 0, d_type, 1);
}

int b200_gemm_f16f32_gated(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N, int64_t K,
                           float alpha, const void* A, int64_t lda, const void* B, int64_t ldb, float beta,
                           const float* C, int64_t ldc, float* D, int64_t ldd, const uint32_t* panel_flags,
                           int64_t panel_k) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    if (!panel_flags) return fail(B200_INVALID_ARG, "gated gemm: panel_flags is null");
    GemmProblem g{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, D, ldd};
    g.panel_flags = panel_flags;
    g.panel_k = panel_k;
    int rc = validate(g);
    if (rc) return rc;
    if (M == 0 || N == 0) return B200_OK;
    std::string why;
    if (!gemm_tcgen05_eligible(g, &why)) return fail(B200_UNSUPPORTED, "gated gemm needs the TMA path: " + why);
    const int saved = h->force_kernel, saved_split = h->split_k;
    h->force_kernel = B200_KERNEL_TCGEN05;
    h->split_k = 1;
    rc = gemm_entry(h, static_cast<cudaStream_t>(stream), g);
    h->force_kernel = saved;
    h->split_k = saved_split;
    return rc;
}

int b200_stream_write_u32(b200_stream stream, void* dptr, uint32_t value) {
    if (!dptr || (reinterpret_cast<uintptr_t>(dptr) & 3u)) return fail(B200_INVALID_ARG, "stream_write_u32: null or misaligned address");
    using Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    static Fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        B200_CUDA_TRY(cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !p) return fail(B200_CUDA_ERROR, "cuStreamWriteValue32 entry point not found");
        fn = reinterpret_cast<Fn>(p);
    }
    CUresult r = fn(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(dptr), value, 0);
    if (r != CUDA_SUCCESS) return fail(B200_CUDA_ERROR, "cuStreamWriteValue32 failed (CUresult " + std::to_string(static_cast<int>(r)) + ")");
    return B200_OK;
}

int b200_stream_wait_u32(b200_stream stream, void* dptr, uint32_t value) {
    if (!dptr || (reinterpret_cast<uintptr_t>(dptr) & 3u)) return fail(B200_INVALID_ARG, "stream_wait_u32: null or misaligned address");
    using Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    static Fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        B200_CUDA_TRY(cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !p) return fail(B200_CUDA_ERROR, "cuStreamWaitValue32 entry point not found");
        fn = reinterpret_cast<Fn>(p);
    }
    CUresult r = fn(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(dptr), value, CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS) return fail(B200_CUDA_ERROR, "cuStreamWaitValue32 failed (CUresult " + std::to_string(static_cast<int>(r)) + ")");
    return B200_OK;
}

int b200_gemm_f16f32_host(b200_handle* h, int transA, int transB, int64_t M, int64_t N, int64_t K, float alpha,
                          const void* A, int64_t lda, const void* B, int64_t ldb, float beta, const float* C,
                          int64_t ldc, float* D, int64_t ldd) {
    if (!h) return fail(B200_INVALID_ARG, "null handle");
    GemmProblem hg{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, D, ldd};
    int rc = validate(hg);
    if (rc) return rc;
    if (M == 0 || N == 0) return B200_OK;
    B200_CUDA_TRY(cudaSetDevice(h->device));
    for (int i = 0; i < 3; ++i)
        if (!h->streams[i]) B200_CUDA_TRY(cudaStreamCreateWithFlags(&h->streams[i], cudaStreamNonBlocking));
    cudaStream_t s_up = h->streams[0], s_mm = h->streams[1], s_dn = h->streams[2];
    const int64_t a_cols = transA ? M : K, b_cols = transB ? K : N;
    const bool has_c = (beta != 0.0f);
    const size_t a_bytes = static_cast<size_t>(lda) * a_cols * 2, b_bytes = static_cast<size_t>(ldb) * b_cols * 2;
    const size_t c_bytes = has_c ? static_cast<size_t>(ldc) * N * 4 : 0, d_bytes = static_cast<size_t>(ldd) * N * 4;
    if ((rc = ensure_buffer(&h->ws[0], &h->ws_bytes[0], std::max<size_t>(a_bytes, 16)))) return rc;
    if ((rc = ensure_buffer(&h->ws[1], &h->ws_bytes[1], std::max<size_t>(b_bytes, 16)))) return rc;
    if ((rc = ensure_buffer(&h->ws[2], &h->ws_bytes[2], std::max<size_t>(c_bytes, 16)))) return rc;
    if ((rc = ensure_buffer(&h->ws[3], &h->ws_bytes[3], std::max<size_t>(d_bytes, 16)))) return rc;
    __half* dA = static_cast<__half*>(h->ws[0]);
    __half* dB = static_cast<__half*>(h->ws[1]);
    float* dC = static_cast<float*>(h->ws[2]);
    float* dD = static_cast<float*>(h->ws[3]);

    // The link is full duplex and the GEMM is far faster than either direction, so the call is
    // cut into column slabs: while slab j multiplies, slab j+1's B and C columns are still
    // arriving and slab j-1's D columns are already on their way back.  A is needed by every
    // slab and goes first.  The uploads keep their direction of the link busy from the first byte
    // to the last, so what the call adds to them is whatever is left to do after the last upload:
    // the last slabs shrink (by a third each, down to one tile) to make that one narrow product and
    // one narrow download; a slab's download (4 bytes per element of D) then still ends before the
    // next slab's upload (6 bytes per element for B and C) does.
    std::vector<int64_t> widths;
    {
        const int64_t cap = std::max<int64_t>(256, ((N + 7) / 8 + 255) / 256 * 256);
        int64_t left = N, w = 256;
        while (left > 0) {
            const int64_t take = (left <= w + w / 4) ? left : w;
            widths.push_back(take);
            left -= take;
            w = std::min<int64_t>(cap, (w * 3 / 2 + 255) / 256 * 256);
        }
        std::reverse(widths.begin(), widths.end());
    }
    const int slabs = static_cast<int>(widths.size());
    while (static_cast<int>(h->events.size()) < 2 * slabs + 1) {
        cudaEvent_t e;
        B200_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->events.push_back(e);
    }
    // Host matrices are read window by window: a column-major operand with ld > rows only has
    // ld * (cols - 1) + rows elements, so whole-buffer copies of ld * cols would run past its end.
    auto upload = [&](void* dst, const void* src, int64_t rows, int64_t cols, int64_t ld, int elem) -> int {
        if (rows <= 0 || cols <= 0) return B200_OK;
        if (ld == rows) {
            B200_CUDA_TRY(cudaMemcpyAsync(dst, src, static_cast<size_t>(rows) * cols * elem, cudaMemcpyHostToDevice, s_up));
        } else {
            B200_CUDA_TRY(cudaMemcpy2DAsync(dst, static_cast<size_t>(ld) * elem, src, static_cast<size_t>(ld) * elem,
                                            static_cast<size_t>(rows) * elem, static_cast<size_t>(cols), cudaMemcpyHostToDevice, s_up));
        }
        return B200_OK;
    };
    if (K > 0 && (rc = upload(dA, A, transA ? K : M, a_cols, lda, 2))) return rc;
    B200_CUDA_TRY(cudaEventRecord(h->events[0], s_up));
    B200_CUDA_TRY(cudaStreamWaitEvent(s_mm, h->events[0], 0));
    int64_t n0 = 0;
    for (int j = 0; j < slabs; n0 += widths[j], ++j) {
        const int64_t nc = widths[j];
        if (K > 0) {
            if (!transB) {  // K x N column-major: columns n0 .. n0+nc
                if ((rc = upload(dB + n0 * ldb, static_cast<const __half*>(B) + n0 * ldb, K, nc, ldb, 2))) return rc;
            } else {        // stored N x K: rows n0 .. n0+nc of every column
                B200_CUDA_TRY(cudaMemcpy2DAsync(dB + n0, static_cast<size_t>(ldb) * 2, static_cast<const __half*>(B) + n0,
                                                static_cast<size_t>(ldb) * 2, static_cast<size_t>(nc) * 2,
                                                static_cast<size_t>(K), cudaMemcpyHostToDevice, s_up));
            }
        }
        if (has_c && (rc = upload(dC + n0 * ldc, C + n0 * ldc, M, nc, ldc, 4))) return rc;
        B200_CUDA_TRY(cudaEventRecord(h->events[1 + 2 * j], s_up));
        B200_CUDA_TRY(cudaStreamWaitEvent(s_mm, h->events[1 + 2 * j], 0));
        GemmProblem g{transA, transB, M, nc, K, alpha, beta, dA, lda, transB ? dB + n0 : dB + n0 * ldb, ldb,
                      dC + n0 * ldc, ldc, dD + n0 * ldd, ldd};
        if ((rc = gemm_dispatch(h, s_mm, g))) return rc;
        B200_CUDA_TRY(cudaEventRecord(h->events[2 + 2 * j], s_mm));
        B200_CUDA_TRY(cudaStreamWaitEvent(s_dn, h->events[2 + 2 * j], 0));
        if (ldd == M) {
            B200_CUDA_TRY(cudaMemcpyAsync(D + n0 * ldd, dD + n0 * ldd, static_cast<size_t>(M) * nc * 4,
                                          cudaMemcpyDeviceToHost, s_dn));
        } else {  // only the M x N window of D belongs to the operation
            B200_CUDA_TRY(cudaMemcpy2DAsync(D + n0 * ldd, static_cast<size_t>(ldd) * 4, dD + n0 * ldd,
                                            static_cast<size_t>(ldd) * 4, static_cast<size_t>(M) * 4,
                                            static_cast<size_t>(nc), cudaMemcpyDeviceToHost, s_dn));
        }
    }
    B200_CUDA_TRY(cudaStreamSynchronize(s_dn));
    B200_CUDA_TRY(cudaStreamSynchronize(s_mm));
    B200_CUDA_TRY(cudaStreamSynchronize(s_up));
    int word[4] = {0, 0, 0, 0};
    if ((rc = read_status(h, word))) return rc;
    if (word[0] != 0)
        return fail(B200_DEVICE_TIMEOUT, "gemm: a bounded wait ran out on the device (wait id " + std::to_string(word[0]) +
                                             ", block " + std::to_string(word[1]) + ")");
    return B200_OK;
}

int b200_malloc(void** dptr, size_t bytes) {
    if (!dptr) return fail(B200_INVALID_ARG, "b200_malloc: null out pointer");
    *dptr = nullptr;
    B200_CUDA_TRY(cudaMalloc(dptr, bytes ? bytes : 1));
    return B200_OK;
}
int b200_free(void* dptr) {
    if (dptr) B200_CUDA_TRY(cudaFree(dptr));
    return B200_OK;
}
int b200_host_alloc(void** hptr, size_t bytes) {
    if (!hptr) return fail(B200_INVALID_ARG, "b200_host_alloc: null out pointer");
    *hptr = nullptr;
    B200_CUDA_TRY(cudaHostAlloc(hptr, bytes ? bytes : 1, cudaHostAllocDefault));
    return B200_OK;
}
int b200_host_free(void* hptr) {
    if (hptr) B200_CUDA_TRY(cudaFreeHost(hptr));
    return B200_OK;
}
int b200_memcpy_h2d(void* dst, const void* src, size_t bytes, b200_stream stream) {
    B200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return B200_OK;
}
int b200_memcpy_d2h(void* dst, const void* src, size_t bytes, b200_stream stream) {
    B200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return B200_OK;
}
int b200_ipc_get_handle(void* dptr, void* handle64) {
    if (!dptr || !handle64) return fail(B200_INVALID_ARG, "ipc_get_handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
    cudaIpcMemHandle_t hnd;
    B200_CUDA_TRY(cudaIpcGetMemHandle(&hnd, dptr));
    std::memcpy(handle64, &hnd, sizeof(hnd));
    return B200_OK;
}
int b200_ipc_open_handle(const void* handle64, void** dptr) {
    if (!dptr || !handle64) return fail(B200_INVALID_ARG, "ipc_open_handle: null argument");
    *dptr = nullptr;
    cudaIpcMemHandle_t hnd;
    std::memcpy(&hnd, handle64, sizeof(hnd));
    B200_CUDA_TRY(cudaIpcOpenMemHandle(dptr, hnd, cudaIpcMemLazyEnablePeerAccess));
    return B200_OK;
}
int b200_ipc_close_handle(void* dptr) {
    if (dptr) B200_CUDA_TRY(cudaIpcCloseMemHandle(dptr));
    return B200_OK;
}
int b200_memcpy_d2d(void* dst, const void* src, size_t bytes, b200_stream stream) {
    if (bytes && (!dst || !src)) return fail(B200_INVALID_ARG, "memcpy_d2d: null pointer");
    B200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
    return B200_OK;
}
int b200_memset(void* dst, int byte, size_t bytes, b200_stream stream) {
    B200_CUDA_TRY(cudaMemsetAsync(dst, byte, bytes, static_cast<cudaStream_t>(stream)));
    return B200_OK;
}
int b200_stream_create(b200_stream* out) {
    if (!out) return fail(B200_INVALID_ARG, "stream_create: null out pointer");
    cudaStream_t s = nullptr;
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *out = s;
    return B200_OK;
}
int b200_stream_destroy(b200_stream stream) {
    if (stream) B200_CUDA_TRY(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return B200_OK;
}
int b200_stream_sync(b200_stream stream) {
    B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return B200_OK;
}

}  // extern "C"
