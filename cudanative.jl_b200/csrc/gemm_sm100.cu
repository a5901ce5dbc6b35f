// Host side of the tcgen05 GEMM: tensor-map construction, kernel selection, launch.
#include "gemm_sm100.cuh"

#include <cudaTypedefs.h>

#include <atomic>
#include <mutex>

#include "internal.h"

namespace b200 {
namespace {

using EncodeFn = PFN_cuTensorMapEncodeTiled_v12000;

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup: no link-time
// dependency on libcuda.
EncodeFn get_encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}

// Matrices of one launch: how many and how far apart (elements); count == 0 asks for a 2-D map.
struct BatchDim {
    int64_t count = 0;
    int64_t stride = 0;
};

// Tensor map over a column-major matrix: dim0 (contiguous) has `inner` elements, dim1 has `outer`
// elements `ld` elements apart; batched problems add dim2 = matrix of the batch (box extent 1).
// A tensor map is a pure function of the arguments below (it describes addresses and shapes, not
// contents), so repeated launches on the same buffers reuse it: a small per-thread cache, most
// recently used first.  Matters for launch-bound sizes only.
struct MapKey {
    const void* base;
    int64_t inner, outer, ld, batch_count, batch_stride;
    uint32_t box_inner, box_outer;
    int dt, sw;
    bool operator==(const MapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && ld == o.ld && batch_count == o.batch_count &&
               batch_stride == o.batch_stride && box_inner == o.box_inner && box_outer == o.box_outer && dt == o.dt && sw == o.sw;
    }
};
struct MapCache {
    static constexpr int kSlots = 16;
    MapKey key[kSlots];
    CUtensorMap map[kSlots];
    int used = 0;
    const CUtensorMap* find(const MapKey& k) {
        for (int i = 0; i < used; ++i)
            if (key[i] == k) {
                if (i > 0) {  // move to front
                    MapKey kk = key[i];
                    CUtensorMap mm = map[i];
                    for (int j = i; j > 0; --j) {
                        key[j] = key[j - 1];
                        map[j] = map[j - 1];
                    }
                    key[0] = kk;
                    map[0] = mm;
                }
                return &map[0];
            }
        return nullptr;
    }
    void insert(const MapKey& k, const CUtensorMap& m) {
        if (used < kSlots) ++used;
        for (int j = used - 1; j > 0; --j) {
            key[j] = key[j - 1];
            map[j] = map[j - 1];
        }
        key[0] = k;
        map[0] = m;
    }
};
thread_local MapCache g_map_cache;

int make_map_2d(CUtensorMap* tm, CUtensorMapDataType dt, int elem_bytes, const void* base, int64_t inner,
                int64_t outer, int64_t ld, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw,
                const char* what, BatchDim batch = BatchDim()) {
    const MapKey mk{base, inner, outer, ld, batch.count, batch.stride, box_inner, box_outer, static_cast<int>(dt), static_cast<int>(sw)};
    if (const CUtensorMap* hit = g_map_cache.find(mk)) {
        *tm = *hit;
        return B200_OK;
    }
    EncodeFn enc = get_encode_fn();
    if (!enc) return fail(B200_CUDA_ERROR, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer),
                          static_cast<cuuint64_t>(batch.count)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * elem_bytes, static_cast<cuuint64_t>(batch.stride) * elem_bytes};
    cuuint32_t box[3] = {box_inner, box_outer, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(tm, dt, batch.count > 0 ? 3 : 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_CUDA_ERROR, std::string("cuTensorMapEncodeTiled failed for ") + what + " (CUresult " +
                                         std::to_string(static_cast<int>(r)) + ")");
    g_map_cache.insert(mk, *tm);
    return B200_OK;
}

// The opt-in to more than 48 KiB of dynamic shared memory is per device and per kernel: made once
// (this also makes the driver load the kernel, which a caller may want to have happen at start-up).
template <int kBN, bool kAMn, bool kBMn, int kCtas, bool kBatch>
int opt_in_shared_memory() {
    static std::atomic<uint64_t> done{0};  // bit d: device d has it
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && (done.load(std::memory_order_relaxed) >> dev) & 1u) return B200_OK;
    B200_CUDA_TRY(cudaFuncSetAttribute(gemm_f16f32_tcgen05<kBN, kAMn, kBMn, kCtas, kBatch>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<kBN, kAMn, kBMn, kCtas>::SMEM_BYTES));
    if (dev < 64) done.fetch_or(uint64_t(1) << dev, std::memory_order_relaxed);
    return B200_OK;
}

template <int kBN, bool kAMn, bool kBMn, int kCtas, bool kBatch>
int launch_kernel(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmD,
                  const GemmParams& p, int grid, cudaStream_t stream, bool pdl) {
    using Cfg = GemmCfg<kBN, kAMn, kBMn, kCtas>;
    auto kern = gemm_f16f32_tcgen05<kBN, kAMn, kBMn, kCtas, kBatch>;
    if (int rc = opt_in_shared_memory<kBN, kAMn, kBMn, kCtas, kBatch>()) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // the kernel orders its own global accesses behind the previous kernel of the stream (griddep_wait)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmD, p));
    return B200_OK;
}

template <int kBN, bool kAMn, bool kBMn, int kCtas>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmD,
               const GemmParams& p, int grid, cudaStream_t stream, bool pdl) {
    if (p.batch > 1) return launch_kernel<kBN, kAMn, kBMn, kCtas, true>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
    return launch_kernel<kBN, kAMn, kBMn, kCtas, false>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
}

template <int kBN, int kCtas>
int launch_layout(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                  const CUtensorMap& tmD, const GemmParams& p, int grid, cudaStream_t stream, bool pdl) {
    if (a_mn) {
        if (b_mn) return launch_one<kBN, true, true, kCtas>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
        return launch_one<kBN, true, false, kCtas>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
    }
    if (b_mn) return launch_one<kBN, false, true, kCtas>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
    return launch_one<kBN, false, false, kCtas>(tmA, tmB, tmC, tmD, p, grid, stream, pdl);
}

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

struct Geometry {
    int tiles_m, tiles_n, kb_total, split_k, kb_per_split;
    int64_t ws_ld;        // leading dimension of the split-K scratch matrix
    int ws_n_stride;      // columns per k-slice in the scratch matrix
};

Geometry geometry(const GemmProblem& g, const GemmPlan& plan) {
    Geometry q;
    const int tile_m = 128 * plan.cta_pair;
    q.tiles_m = static_cast<int>((g.M + tile_m - 1) / tile_m);
    q.tiles_n = static_cast<int>((g.N + plan.tile_n - 1) / plan.tile_n);
    q.kb_total = static_cast<int>((g.K + 63) / 64);
    int s = (plan.split_k < 1 || g.batch > 1) ? 1 : plan.split_k;  // a batch already is parallel work
    if (s > q.kb_total) s = q.kb_total;
    q.kb_per_split = (q.kb_total + s - 1) / s;
    q.split_k = (q.kb_total + q.kb_per_split - 1) / q.kb_per_split;  // no empty slices
    q.ws_ld = round_up(g.M, 4);
    q.ws_n_stride = q.tiles_n * plan.tile_n;
    return q;
}

}  // namespace

namespace {
template <int kBN, int kCtas>
int preload_layouts() {
    int rc;
    if ((rc = opt_in_shared_memory<kBN, false, false, kCtas, false>())) return rc;
    if ((rc = opt_in_shared_memory<kBN, true, false, kCtas, false>())) return rc;
    if constexpr ((kBN / kCtas) % 64 == 0) {
        if ((rc = opt_in_shared_memory<kBN, false, true, kCtas, false>())) return rc;
        if ((rc = opt_in_shared_memory<kBN, true, true, kCtas, false>())) return rc;
    }
    return B200_OK;
}
}  // namespace

int gemm_tcgen05_preload() {
    int rc;
    if ((rc = preload_layouts<256, 2>())) return rc;
    if ((rc = preload_layouts<128, 2>())) return rc;
    if ((rc = preload_layouts<256, 1>())) return rc;
    if ((rc = preload_layouts<128, 1>())) return rc;
    if ((rc = preload_layouts<64, 1>())) return rc;
    cudaFuncAttributes at;
    B200_CUDA_TRY(cudaFuncGetAttributes(&at, gemm_splitk_reduce));
    return B200_OK;
}

size_t gemm_tcgen05_scratch_bytes(const GemmProblem& g, const GemmPlan& plan) {
    const Geometry q = geometry(g, plan);
    if (q.split_k <= 1) return 0;
    return static_cast<size_t>(q.ws_ld) * q.ws_n_stride * q.split_k * sizeof(float);
}

bool gemm_tcgen05_eligible(const GemmProblem& g, std::string* why) {
    auto no = [&](const char* m) {
        if (why) *why = m;
        return false;
    };
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return no("empty problem");
    if (g.M > 0x7fffff00ll || g.N > 0x7fffff00ll || g.K > 0x7fffff00ll) return no("dimension exceeds 2^31");
    if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.D)) & 15u)
        return no("A, B and D must be 16-byte aligned for TMA");
    if (g.beta != 0.0f && (reinterpret_cast<uintptr_t>(g.C) & 15u)) return no("C must be 16-byte aligned for TMA");
    if ((g.lda % 8) || (g.ldb % 8)) return no("lda and ldb must be multiples of 8 elements for TMA");
    const int c_quant = 16 / elem_bytes(g.c_type), d_quant = 16 / elem_bytes(g.d_type);
    if ((g.ldd % d_quant) || (g.beta != 0.0f && (g.ldc % c_quant)))
        return no("ldc and ldd must be multiples of 16 bytes for TMA");
    // bulk tensor stores clip at 16-byte granularity: with a ragged last chunk every column
    // would spill into the rows M .. roundup(M) - 1 of the caller's buffer
    if (g.M % d_quant) return no(d_quant == 8 ? "M must be a multiple of 8 for 16-bit D (bulk stores are 16-byte granular)"
                                              : "M must be a multiple of 4 (bulk stores are 16-byte granular)");
    if (g.batch > 1) {
        // the matrix index becomes a third tensor-map dimension: its stride obeys the same 16-byte
        // rule as a leading dimension, and matrices must not overlap (or repeat: stride 0)
        if (g.panel_flags) return no("gated A is not available for batches");
        if (g.batch * ((g.M + 127) / 128) * ((g.N + 63) / 64) > 0x7fffff00ll) return no("too many tiles for one launch");
        const int64_t a_cols = g.transA ? g.M : g.K, b_cols = g.transB ? g.K : g.N;
        if (g.stride_a < g.lda * a_cols || g.stride_b < g.ldb * b_cols || g.stride_d < g.ldd * g.N ||
            (g.beta != 0.0f && g.stride_c < g.ldc * g.N))
            return no("batch strides must be at least the extent of one matrix");
        if ((g.stride_a % 8) || (g.stride_b % 8) || (g.stride_d % d_quant) || (g.beta != 0.0f && (g.stride_c % c_quant)))
            return no("batch strides must be multiples of 16 bytes for TMA");
    }
    return true;
}

int gemm_tcgen05_launch(const GemmProblem& g, const GemmPlan& plan, float* scratch, int* status_word, int sm_count,
                        cudaStream_t stream, LaunchInfo* info) {
    const Geometry q = geometry(g, plan);
    const bool a_mn = (g.transA == 0);  // column-major M x K: M contiguous
    const bool b_mn = (g.transB != 0);  // stored N x K column-major: N contiguous
    const int bn_local = plan.tile_n / plan.cta_pair;
    if (b_mn && (bn_local % 64)) return fail(B200_UNSUPPORTED, "row-major B needs at least 64 tile columns per CTA");
    if (q.split_k > 1 && !scratch) return fail(B200_INVALID_ARG, "split-K launch without scratch");

    const bool batched = g.batch > 1;
    auto batch_dim = [&](int64_t stride) {
        BatchDim b;
        if (batched) {
            b.count = g.batch;
            b.stride = stride;
        }
        return b;
    };
    auto map_type = [](int type) {
        return type == B200_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                : (type == B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    };
    const CUtensorMapDataType ab_dt = map_type(g.ab_type);

    CUtensorMap tmA, tmB, tmC, tmD;
    int rc;
    if (a_mn)
        rc = make_map_2d(&tmA, ab_dt, 2, g.A, g.M, g.K, g.lda, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B, "A (column-major)",
                         batch_dim(g.stride_a));
    else
        rc = make_map_2d(&tmA, ab_dt, 2, g.A, g.K, g.M, g.lda, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B, "A (row-major)",
                         batch_dim(g.stride_a));
    if (rc) return rc;
    if (b_mn)
        rc = make_map_2d(&tmB, ab_dt, 2, g.B, g.N, g.K, g.ldb, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B, "B (row-major)",
                         batch_dim(g.stride_b));
    else
        rc = make_map_2d(&tmB, ab_dt, 2, g.B, g.K, g.N, g.ldb, 64, bn_local, CU_TENSOR_MAP_SWIZZLE_128B,
                         "B (column-major)", batch_dim(g.stride_b));
    if (rc) return rc;

    GemmParams p = {};
    p.M = static_cast<int>(g.M);
    p.N = static_cast<int>(g.N);
    p.K = static_cast<int>(g.K);
    p.tiles_m = q.tiles_m;
    p.tiles_n = q.tiles_n;
    p.split_k = q.split_k;
    p.kb_total = q.kb_total;
    p.kb_per_split = q.kb_per_split;
    p.raster_group = plan.raster_group > 0 ? plan.raster_group : 8;
    if (g.panel_flags) {
        if (g.panel_k <= 0 || g.panel_k % 64) return fail(B200_INVALID_ARG, "gated gemm: panel_k must be a positive multiple of 64");
        if ((g.K + g.panel_k - 1) / g.panel_k > 32) return fail(B200_INVALID_ARG, "gated gemm: at most 32 panels");
        p.panel_flags = g.panel_flags;
        p.kb_per_panel = static_cast<int>(g.panel_k / 64);
    }
    p.status = status_word;
    p.wait_budget_ns = plan.wait_budget_ns;
    p.ab_bf16 = g.ab_type == B200_BF16 ? 1 : 0;
    p.acc_f16 = g.acc_f16 ? 1 : 0;
    p.batch = static_cast<int>(g.batch);

    if (q.split_k > 1) {
        // partial products go to scratch (k-slice s occupies columns [s * stride, s * stride + N))
        rc = make_map_2d(&tmD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, scratch, g.M, static_cast<int64_t>(q.ws_n_stride) * q.split_k,
                         q.ws_ld, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE, "split-K scratch");
        if (rc) return rc;
        tmC = tmD;
        p.alpha = 1.0f;
        p.beta = 0.0f;
        p.out_n_stride = q.ws_n_stride;
    } else {
        rc = make_map_2d(&tmD, map_type(g.d_type), elem_bytes(g.d_type), g.D, g.M, g.N, g.ldd, 128, 32,
                         CU_TENSOR_MAP_SWIZZLE_NONE, "D", batch_dim(g.stride_d));
        if (rc) return rc;
        if (g.beta != 0.0f) {
            rc = make_map_2d(&tmC, map_type(g.c_type), elem_bytes(g.c_type), g.C, g.M, g.N, g.ldc, 128, 32,
                             CU_TENSOR_MAP_SWIZZLE_NONE, "C", batch_dim(g.stride_c));
            if (rc) return rc;
        } else {
            tmC = tmD;  // never dereferenced
        }
        p.alpha = g.alpha;
        p.beta = g.beta;
        p.out_n_stride = 0;
        p.c_fmt = elem_fmt(g.c_type);
        p.d_fmt = elem_fmt(g.d_type);
    }

    const int units = q.tiles_m * q.tiles_n * (batched ? static_cast<int>(g.batch) : q.split_k);
    int cap = plan.max_ctas > 0 ? plan.max_ctas : sm_count;
    if (cap > sm_count) cap = sm_count;
    int grid;
    if (plan.cta_pair == 2) {
        int clusters = cap / 2;
        if (clusters < 1) clusters = 1;
        if (clusters > units) clusters = units;
        grid = clusters * 2;
    } else {
        grid = cap < units ? cap : units;
        if (grid < 1) grid = 1;
    }

    if (plan.cta_pair == 2) {
        if (plan.tile_n == 256) rc = launch_layout<256, 2>(a_mn, b_mn, tmA, tmB, tmC, tmD, p, grid, stream, plan.pdl != 0);
        else if (plan.tile_n == 128) rc = launch_layout<128, 2>(a_mn, b_mn, tmA, tmB, tmC, tmD, p, grid, stream, plan.pdl != 0);
        else return fail(B200_UNSUPPORTED, "2-CTA tiles exist for tile_n 128 and 256");
    } else {
        if (plan.tile_n == 256) rc = launch_layout<256, 1>(a_mn, b_mn, tmA, tmB, tmC, tmD, p, grid, stream, plan.pdl != 0);
        else if (plan.tile_n == 128) rc = launch_layout<128, 1>(a_mn, b_mn, tmA, tmB, tmC, tmD, p, grid, stream, plan.pdl != 0);
        else if (plan.tile_n == 64) rc = launch_layout<64, 1>(a_mn, b_mn, tmA, tmB, tmC, tmD, p, grid, stream, plan.pdl != 0);
        else return fail(B200_UNSUPPORTED, "tile_n must be 64, 128 or 256");
    }
    if (rc) return rc;

    if (q.split_k > 1) {
        const bool vec_ok = g.c_type == B200_F32 && g.d_type == B200_F32 &&
                            !((reinterpret_cast<uintptr_t>(g.D) & 15u) || (g.ldd % 4) ||
                              (g.beta != 0.0f && ((reinterpret_cast<uintptr_t>(g.C) & 15u) || (g.ldc % 4))));
        const long long quads = (g.M + 3) / 4 * g.N;
        int blocks = static_cast<int>((quads + 255) / 256);
        if (blocks > sm_count * 8) blocks = sm_count * 8;
        if (blocks < 1) blocks = 1;
        gemm_splitk_reduce<<<blocks, 256, 0, stream>>>(scratch, q.ws_ld, q.ws_n_stride, q.split_k, p.M, p.N, g.alpha,
                                                       g.beta, g.C, g.ldc, g.D, g.ldd, vec_ok ? 1 : 0, elem_fmt(g.c_type),
                                                       elem_fmt(g.d_type));
        B200_CUDA_TRY(cudaGetLastError());
    }
    if (info) {
        info->kernel = B200_KERNEL_TCGEN05;
        info->tile_n = plan.tile_n;
        info->split_k = q.split_k;
        info->ctas = grid;
        info->cta_pair = plan.cta_pair;
    }
    return B200_OK;
}

}  // namespace b200
