// The 16x16x16 WMMA unit: fragment-granular load / fill / broadcast / mma / store kernels and
// the fused one-launch form, in two lowerings.
//
// Reference: CUDAnative.jl src/device/cuda/wmma.jl -- load_a/load_b/load_c (:507-530), mma
// (:558-583), store_d (:613-632), fill_c (:654-667), broadcasting (:678-716).  There each call
// inlines one wmma.{load,mma,store}.sync instruction into the user's kernel; here each call is
// one warp-sized kernel operating on a fragment image in device memory, and the fused entry point
// runs the whole load -> scale -> mma -> store body of the reference's example kernels
// (examples/wmma/high-level.jl:30-44) in a single launch.
//
// Fragment image: 32 lanes x FS elements, FS = 16 (A, B) or 8 (C, D), the sizes of
// wmma.jl:413-420.  Slot -> matrix-element map (private, as the reference leaves it unspecified):
// the register order of mma.sync.m16n8k16 (A: 8 halves per lane; B and C/D: two n-blocks of 8
// columns); A/B slots 8..15 repeat slots 0..7 so that elementwise operations over all FS slots
// stay consistent.
#include <cuda_fp16.h>

#include <mutex>

#include "ptx_sm100.cuh"
#include "wmma_frag.cuh"
#include "internal.h"

namespace b200 {
namespace {

__device__ __forceinline__ float load_elem(const void* p, int elem_type, int64_t off) {
    return elem_type == B200_F16 ? __half2float(static_cast<const __half*>(p)[off]) : static_cast<const float*>(p)[off];
}
__device__ __forceinline__ void store_elem(void* p, int elem_type, int64_t off, float v) {
    if (elem_type == B200_F16) static_cast<__half*>(p)[off] = __float2half_rn(v);
    else static_cast<float*>(p)[off] = v;
}

// ---- fragment-granular kernels (one warp each) ---------------------------------------------
__global__ void frag_load_kernel(int use, int layout, int elem_type, const void* addr, int64_t stride, void* frag) {
    const int lane = threadIdx.x;
    const int fs = (use == B200_ACCUMULATOR) ? 8 : 16;
    for (int e = 0; e < fs; ++e) {
        int r, c;
        frag_coord(use, lane, e, r, c);
        store_elem(frag, elem_type, lane * fs + e, load_elem(addr, elem_type, mat_off(layout, r, c, stride)));
    }
}

__global__ void frag_fill_kernel(int elem_type, float value, void* frag) {
    const int lane = threadIdx.x;
    for (int e = 0; e < 8; ++e) store_elem(frag, elem_type, lane * 8 + e, value);
}

// out[i] = s (op) in[i] in the fragment's own element type (binary16 results are rounded once,
// which is what Float16 arithmetic in the reference's broadcast does).
__global__ void frag_bcast_kernel(int op, int elem_type, int count, float scalar, const void* in, void* out) {
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        float s = scalar;
        if (elem_type == B200_F16) s = __half2float(__float2half_rn(s));
        const float x = load_elem(in, elem_type, i);
        store_elem(out, elem_type, i, op == 0 ? s * x : s + x);
    }
}

__global__ void frag_mma_kernel(int c_type, int d_type, const __half* a_frag, const __half* b_frag,
                                const void* c_frag, void* d_frag) {
    const int lane = threadIdx.x;
    __half a[8], b[8];
    float c[8], d[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        a[e] = a_frag[lane * 16 + e];
        b[e] = b_frag[lane * 16 + e];
        c[e] = load_elem(c_frag, c_type, lane * 8 + e);
    }
    warp_mma(a, b, c, c_type, d_type, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) store_elem(d_frag, d_type, lane * 8 + e, d[e]);
}

__global__ void frag_store_kernel(int layout, int elem_type, void* addr, const void* frag, int64_t stride) {
    const int lane = threadIdx.x;
    for (int e = 0; e < 8; ++e) {
        int r, c;
        c_coord(lane, e, r, c);
        store_elem(addr, elem_type, mat_off(layout, r, c, stride), load_elem(frag, elem_type, lane * 8 + e));
    }
}

struct UnitArgs {
    int a_layout, b_layout, c_layout, d_layout, c_type, d_type, mac, use_alpha, use_beta;
    float alpha, beta;
    const __half* A;
    int64_t lda;
    const __half* B;
    int64_t ldb;
    const void* C;
    int64_t ldc;
    void* D;
    int64_t ldd;
};

// alpha .* a in binary16; beta .* c in C's element type
__device__ __forceinline__ __half scale_a(const UnitArgs& u, __half v) {
    return u.use_alpha ? __hmul(__float2half_rn(u.alpha), v) : v;
}
__device__ __forceinline__ float scaled_c(const UnitArgs& u, int r, int c) {
    if (!u.mac) return 0.0f;  // fill_c(0); beta .* 0 == 0
    float v = load_elem(u.C, u.c_type, mat_off(u.c_layout, r, c, u.ldc));
    if (u.use_beta) {
        if (u.c_type == B200_F16) v = __half2float(__float2half_rn(__half2float(__float2half_rn(u.beta)) * v));
        else v = u.beta * v;
    }
    return v;
}

// ---- fused unit, warp-level lowering ---------------------------------------------------------
__global__ void unit_warp_kernel(UnitArgs u) {
    const int lane = threadIdx.x;
    __half a[8], b[8];
    float c[8], d[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        int r, k, n;
        a_coord(lane, e, r, k);
        a[e] = scale_a(u, u.A[mat_off(u.a_layout, r, k, u.lda)]);
        b_coord(lane, e, k, n);
        b[e] = u.B[mat_off(u.b_layout, k, n, u.ldb)];
        int cr, cc;
        c_coord(lane, e, cr, cc);
        c[e] = scaled_c(u, cr, cc);
    }
    warp_mma(a, b, c, u.c_type, u.d_type, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        int r, cc;
        c_coord(lane, e, r, cc);
        store_elem(u.D, u.d_type, mat_off(u.d_layout, r, cc, u.ldd), d[e]);
    }
}

// ---- fused unit, tcgen05 lowering -------------------------------------------------------------
// One CTA of 128 threads.  A is zero-padded from 16 to 128 rows (tcgen05.mma with M = 128 keeps
// accumulator row i in TMEM lane i), N = K = 16.  Operands sit in shared memory in the
// unswizzled K-major core-matrix layout: 8 rows x 16 bytes form one contiguous 128-byte core
// matrix; the second k-chunk of a row group follows at +128 B (leading byte offset), the next
// 8-row group at +256 B (stride byte offset).  C is written into TMEM with tcgen05.st before the
// MMA accumulates onto it, so the instruction computes a * b + c as WMMA.mma does.
__global__ void __launch_bounds__(128) unit_tcgen05_kernel(UnitArgs u, int* status, unsigned long long budget_ns) {
    __shared__ __align__(1024) uint8_t sA[128 * 16 * 2];
    __shared__ __align__(1024) uint8_t sB[16 * 16 * 2];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5;
    WaitCtx wc{&abort_flag, status, budget_ns};
    if (tid == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    if (warp == 0) {
        __syncwarp();  // thread 0 took the branch above: the allocation is warp-collective (.sync.aligned)
        tmem_alloc<1>(smem_u32(&tmem_slot), 32);
    }

    auto core_off = [](int r, int k) { return (r >> 3) * 256 + (k >> 3) * 128 + (r & 7) * 16 + (k & 7) * 2; };
    {
        const int r = tid;  // one A row per thread
        for (int k = 0; k < 16; ++k) {
            __half v = __float2half_rn(0.0f);
            if (r < 16) v = scale_a(u, u.A[mat_off(u.a_layout, r, k, u.lda)]);
            *reinterpret_cast<__half*>(sA + core_off(r, k)) = v;
        }
        if (tid < 16) {
            const int n = tid;  // B operand rows are the columns of B
            for (int k = 0; k < 16; ++k)
                *reinterpret_cast<__half*>(sB + core_off(n, k)) = u.B[mat_off(u.b_layout, k, n, u.ldb)];
        }
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_slot;
    const uint32_t my_tmem = tmem + (static_cast<uint32_t>(warp * 32) << 16);

    {
        uint32_t cv[16];
#pragma unroll
        for (int n = 0; n < 16; ++n) cv[n] = __float_as_uint(tid < 16 ? scaled_c(u, tid, n) : 0.0f);
        tmem_st_32x32b_x16(my_tmem, cv);
        tmem_wait_st();
    }
    tc_fence_before_sync();
    __syncthreads();

    if (tid == 0) {
        tc_fence_after_sync();
        const uint64_t da = make_smem_desc(smem_u32(sA), 128, 256, kSwizzleNone);
        const uint64_t db = make_smem_desc(smem_u32(sB), 128, 256, kSwizzleNone);
        umma_f16<1>(tmem, da, db, make_idesc_f16_f32(128, 16, 0, 0), 1u);
        umma_commit<1>(smem_u32(&bar));
    }
    const bool ok = mbar_wait(smem_u32(&bar), 0, wc, kWaitUnit);
    const bool all_ok = !__syncthreads_or(!ok);
    tc_fence_after_sync();
    if (all_ok) {
        uint32_t dv[16];
        tmem_ld_32x32b_x16(my_tmem, dv);
        tmem_wait_ld();
        if (tid < 16) {
#pragma unroll
            for (int n = 0; n < 16; ++n)
                store_elem(u.D, u.d_type, mat_off(u.d_layout, tid, n, u.ldd), __uint_as_float(dv[n]));
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem, 32);
    }
}

int check_layout(int l, const char* what) {
    if (l != B200_COL_MAJOR && l != B200_ROW_MAJOR) return fail(B200_INVALID_ARG, std::string("invalid layout for WMMA: ") + what);
    return B200_OK;
}
int check_type(int t, const char* what) {
    if (t != B200_F16 && t != B200_F32) return fail(B200_INVALID_ARG, std::string("invalid element type for WMMA: ") + what);
    return B200_OK;
}

// device status word for the tcgen05 unit (one per process and device is enough: the unit is a
// single CTA and the word only ever holds the first failure).  16 bytes per device, kept until the
// process exits; the table is guarded because WMMA calls may come from several host threads
// (the reference's @cuda is thread-safe, test/device/execution.jl:1057-1078).
int* unit_status_word() {
    static int* word[64] = {};
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!word[dev]) {
        if (cudaMalloc(&word[dev], 4 * sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(word[dev], 0, 4 * sizeof(int));
    }
    return word[dev];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_wmma_16x16x16(b200_stream stream, int lowering, int a_layout, int b_layout, int c_layout,
                                  int d_layout, int c_type, int d_type, int mac, int use_alpha, float alpha,
                                  int use_beta, float beta, const void* A, int64_t lda, const void* B, int64_t ldb,
                                  const void* C, int64_t ldc, void* D, int64_t ldd) {
    int rc;
    if ((rc = check_layout(a_layout, "A")) || (rc = check_layout(b_layout, "B")) || (rc = check_layout(c_layout, "C")) ||
        (rc = check_layout(d_layout, "D")) || (rc = check_type(c_type, "C")) || (rc = check_type(d_type, "D")))
        return rc;
    if (!A || !B || !D || (mac && !C)) return fail(B200_INVALID_ARG, "wmma unit: null matrix pointer");
    if (lda < 16 || ldb < 16 || ldd < 16 || (mac && ldc < 16)) return fail(B200_INVALID_ARG, "wmma unit: stride below 16");
    UnitArgs u{a_layout, b_layout, c_layout, d_layout, c_type, d_type, mac ? 1 : 0, use_alpha ? 1 : 0, use_beta ? 1 : 0,
               alpha, beta, static_cast<const __half*>(A), lda, static_cast<const __half*>(B), ldb, C, ldc, D, ldd};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (lowering == B200_LOWER_WARP) {
        unit_warp_kernel<<<1, 32, 0, s>>>(u);
    } else if (lowering == B200_LOWER_TCGEN05) {
        int* status = unit_status_word();
        if (!status) return fail(B200_CUDA_ERROR, "wmma unit: cannot allocate the device status word");
        unit_tcgen05_kernel<<<1, 128, 0, s>>>(u, status, 2000000000ull);
        B200_CUDA_TRY(cudaGetLastError());
        // this lowering has a bounded in-kernel wait: synchronise so that a wait that ran out
        // is reported by this call rather than lost
        B200_CUDA_TRY(cudaStreamSynchronize(s));
        int word[4] = {0, 0, 0, 0};
        B200_CUDA_TRY(cudaMemcpy(word, status, sizeof(word), cudaMemcpyDeviceToHost));
        if (word[0] != 0) {
            cudaMemset(status, 0, sizeof(word));
            return fail(B200_DEVICE_TIMEOUT, "wmma unit: the wait for tcgen05.mma ran out (wait id " + std::to_string(word[0]) + ")");
        }
    } else {
        return fail(B200_INVALID_ARG, "wmma unit: unknown lowering");
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_wmma_load(b200_stream stream, int use, int layout, int elem_type, const void* addr, int64_t stride,
                              void* frag) {
    int rc;
    if (use < B200_MATRIX_A || use > B200_ACCUMULATOR) return fail(B200_INVALID_ARG, "wmma load: unknown fragment use");
    if ((rc = check_layout(layout, "load")) || (rc = check_type(elem_type, "load"))) return rc;
    if (use != B200_ACCUMULATOR && elem_type != B200_F16)
        return fail(B200_INVALID_ARG, "invalid type Float32 for matrix a/b: only the accumulator may be Float32");
    if (!addr || !frag || stride < 16) return fail(B200_INVALID_ARG, "wmma load: null pointer or stride below 16");
    frag_load_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(use, layout, elem_type, addr, stride, frag);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_wmma_fill_c(b200_stream stream, int elem_type, float value, void* frag) {
    int rc;
    if ((rc = check_type(elem_type, "fill_c"))) return rc;
    if (!frag) return fail(B200_INVALID_ARG, "wmma fill_c: null fragment");
    frag_fill_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(elem_type, value, frag);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_wmma_bcast(b200_stream stream, int op, int elem_type, int frag_size, float scalar,
                               const void* frag_in, void* frag_out) {
    int rc;
    if ((rc = check_type(elem_type, "broadcast"))) return rc;
    if (op != 0 && op != 1) return fail(B200_INVALID_ARG, "wmma broadcast: op must be 0 (mul) or 1 (add)");
    if (frag_size < 1 || frag_size > 16 || !frag_in || !frag_out) return fail(B200_INVALID_ARG, "wmma broadcast: bad fragment");
    frag_bcast_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(op, elem_type, 32 * frag_size, scalar, frag_in, frag_out);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_wmma_mma(b200_stream stream, int c_type, int d_type, const void* a_frag, const void* b_frag,
                             const void* c_frag, void* d_frag) {
    int rc;
    if ((rc = check_type(c_type, "C")) || (rc = check_type(d_type, "D"))) return rc;
    if (!a_frag || !b_frag || !c_frag || !d_frag) return fail(B200_INVALID_ARG, "wmma mma: null fragment");
    frag_mma_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(c_type, d_type, static_cast<const __half*>(a_frag),
                                                                      static_cast<const __half*>(b_frag), c_frag, d_frag);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" int b200_wmma_store_d(b200_stream stream, int layout, int elem_type, void* addr, const void* frag,
                                 int64_t stride) {
    int rc;
    if ((rc = check_layout(layout, "store_d")) || (rc = check_type(elem_type, "store_d"))) return rc;
    if (!addr || !frag || stride < 16) return fail(B200_INVALID_ARG, "wmma store_d: null pointer or stride below 16");
    frag_store_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(layout, elem_type, addr, frag, stride);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
