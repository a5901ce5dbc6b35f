// b200_gemm_f16f32_splitk_static: the split-K GEMM for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a product: code
// running inside a memory-pool callback or under an allocator lock, a real-time loop that
// promised its integrator "no driver allocations after start-up", a plug-in whose host process
// owns all device memory and hands out fixed buffers only.  The regular entry points do not fit
// them: the handle allocates a status word when it is created and grows a scratch buffer the
// first time a split-K plan needs one.
//
// This variant takes everything it needs from one array that is part of the library image:
//     static __device__ g_static_scratch[16 MiB + 256 B]
// The first 256 bytes hold the device status word the kernels report a timed-out wait in; the
// rest holds the FP32 partial products of the k-slices.  Every GPU that loads the library carries
// the array until the process exits, which is why it is kept modest: problems whose partials do
// not fit (M rounded up to 4, times N rounded up to the tile width, times the number of k-slices,
// times 4 bytes > 16 MiB) are refused with B200_INVALID_ARG and a message that says so.
//
// The array's name is a host-side stand-in in host code, not a device address, so the host never
// passes it to a kernel: once per device, with that device current, the address is looked up with
// cudaGetSymbolAddress and cached.  That lookup happens on the first call made on a device -- make
// that first call outside of any stream capture.
//
// All calls on one device share the array and it keeps whatever the previous call left there.
// The partials need no clearing because every slice writes its whole window before the reduction
// reads it.  The status word is cleared by whoever reads it (a synchronous call, or
// b200_static_status); an asynchronous caller that never asks keeps the first failure on record.
// Two calls that overlap on the GPU (different streams, or different threads) race on the array:
// serialise them.
//
// "Allocates nothing" has one more condition: the first launch of a kernel makes the driver load
// it, and loading allocates.  b200_static_warmup does all of that up front (symbol lookup, every
// kernel variant the entry point can pick); call it once per device at start-up, outside of any
// stream capture, and nothing after it allocates.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace {

using b200::cuda_fail;  // B200_CUDA_TRY names it unqualified

constexpr size_t kHeaderBytes = 256;
constexpr size_t kPartialBytes = 16u << 20;

static __device__ __align__(256) unsigned char g_static_scratch[kHeaderBytes + kPartialBytes];

// One warp waits, with a budget, on a barrier nothing ever arrives on, and reports into the static
// status word: the way to see b200_static_status work without any fault, trap or endless loop.
__global__ void static_selftest_kernel(int* status, unsigned long long budget_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        b200::mbar_init(b200::smem_u32(&bar), 1);
        b200::fence_mbar_init();
    }
    __syncthreads();
    b200::WaitCtx wc{&abort_flag, status, budget_ns};
    b200::mbar_wait(b200::smem_u32(&bar), 0, wc, b200::kWaitSelftest);
}

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_scratch_addr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};

// Device address of g_static_scratch on the current device (looked up once per device).
int static_scratch(unsigned char** addr, int* sm_count) {
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return b200::fail(B200_UNSUPPORTED, "device index beyond the static table");
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_addr[dev]) {
        int major = 0, sms = 0;
        B200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) return b200::fail(B200_NO_DEVICE, "this library holds sm_100a code only");
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return b200::cuda_fail(e, "cudaGetSymbolAddress(g_static_scratch)");
        if (!p) return b200::fail(B200_CUDA_ERROR, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[dev] = static_cast<unsigned char*>(p);
        g_sm_count[dev] = sms;
    }
    *addr = g_scratch_addr[dev];
    *sm_count = g_sm_count[dev];
    return B200_OK;
}

}  // namespace

extern "C" int b200_gemm_f16f32_splitk_static(b200_stream stream, int transA, int transB, int64_t M, int64_t N,
                                              int64_t K, float alpha, const void* A, int64_t lda, const void* B,
                                              int64_t ldb, float beta, const float* C, int64_t ldc, float* D,
                                              int64_t ldd, int split_k, int sync_and_check) {
    using namespace b200;
    if (M <= 0 || N <= 0 || K <= 0) return fail(B200_INVALID_ARG, "static split-K gemm: M, N and K must be positive");
    if ((transA != 0 && transA != 1) || (transB != 0 && transB != 1))
        return fail(B200_INVALID_ARG, "static split-K gemm: transA / transB must be 0 or 1");
    if (split_k < 2 || split_k > 64) return fail(B200_INVALID_ARG, "static split-K gemm: split_k must be in [2, 64]");
    if (!A || !B || !D || (beta != 0.0f && !C)) return fail(B200_INVALID_ARG, "static split-K gemm: null matrix pointer");
    if (lda < (transA ? K : M) || ldb < (transB ? N : K) || ldd < M || (beta != 0.0f && ldc < M))
        return fail(B200_INVALID_ARG, "static split-K gemm: leading dimension smaller than the stored rows");
    GemmProblem g{transA, transB, M, N, K, alpha, beta, A, lda, B, ldb, C, ldc, D, ldd};
    std::string why;
    if (!gemm_tcgen05_eligible(g, &why)) return fail(B200_UNSUPPORTED, "static split-K gemm: " + why);
    GemmPlan plan = {};
    plan.tile_n = N > 128 ? 256 : (N > 64 ? 128 : 64);
    // the handle path's tile choice: 2-CTA tiles once the tile is 256 columns wide and there are rows enough
    plan.cta_pair = (M > 128 && plan.tile_n == 256) ? 2 : 1;
    plan.split_k = split_k;
    plan.max_ctas = 0;
    plan.raster_group = 0;
    plan.wait_budget_ns = 2000000000ull;
    const size_t need = gemm_tcgen05_scratch_bytes(g, plan);
    if (need > kPartialBytes)
        return fail(B200_INVALID_ARG, "static split-K gemm: the partial products need " + std::to_string(need) +
                                          " bytes but the static scratch holds " + std::to_string(kPartialBytes) +
                                          "; use fewer k-slices, a smaller problem, or b200_gemm_f16f32");
    unsigned char* base = nullptr;
    int sm_count = 0;
    int rc = static_scratch(&base, &sm_count);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = reinterpret_cast<int*>(base);
    float* partials = reinterpret_cast<float*>(base + kHeaderBytes);
    if (need == 0) {
        // K is too short to cut: a single slice needs no partials, only the status word
        plan.split_k = 1;
    }
    if ((rc = gemm_tcgen05_launch(g, plan, partials, status, sm_count, s, nullptr))) return rc;
    if (sync_and_check) {
        B200_CUDA_TRY(cudaStreamSynchronize(s));
        int word[4] = {0, 0, 0, 0};
        B200_CUDA_TRY(cudaMemcpy(word, status, sizeof(word), cudaMemcpyDeviceToHost));
        if (word[0] != 0) B200_CUDA_TRY(cudaMemset(status, 0, sizeof(word)));
        if (word[0] != 0)
            return fail(B200_DEVICE_TIMEOUT, "static split-K gemm: a bounded wait ran out on the device (wait id " +
                                                 std::to_string(word[0]) + ", block " + std::to_string(word[1]) + ")");
    }
    return B200_OK;
}

extern "C" int b200_static_status(int* code, int* block, int* detail) {
    unsigned char* base = nullptr;
    int sm_count = 0;
    int rc = static_scratch(&base, &sm_count);
    if (rc) return rc;
    int word[4] = {0, 0, 0, 0};
    B200_CUDA_TRY(cudaMemcpy(word, base, sizeof(word), cudaMemcpyDeviceToHost));
    if (word[0] != 0) B200_CUDA_TRY(cudaMemset(base, 0, sizeof(word)));
    if (code) *code = word[0];
    if (block) *block = word[1];
    if (detail) *detail = word[2];
    return B200_OK;
}

extern "C" int b200_static_warmup(void) {
    unsigned char* base = nullptr;
    int sm_count = 0;
    int rc = static_scratch(&base, &sm_count);
    if (rc) return rc;
    if ((rc = b200::gemm_tcgen05_preload())) return rc;
    // the array is zero-initialised when the module is loaded; make sure of the status word anyway
    B200_CUDA_TRY(cudaMemset(base, 0, 4 * sizeof(int)));
    return B200_OK;
}

extern "C" int b200_static_selftest_bounded_wait(b200_stream stream, int64_t budget_ns) {
    if (budget_ns < 1000 || budget_ns > 1000000000ll)
        return b200::fail(B200_INVALID_ARG, "selftest budget must be within [1 us, 1 s]");
    unsigned char* base = nullptr;
    int sm_count = 0;
    int rc = static_scratch(&base, &sm_count);
    if (rc) return rc;
    static_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(base),
                                                                            static_cast<unsigned long long>(budget_ns));
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
