// Persistent, warp-specialised FP16 x FP16 -> FP32 GEMM for sm_100a.
//
//   D = alpha * op(A) * op(B) + beta * C        (column-major C / D, FP32 epilogue)
//
// This is the many-tile form of the reference's load_a / load_b / load_c -> mma -> store_d
// sequence (src/device/cuda/wmma.jl:507-632 of CUDAnative.jl): "fragments" are shared-memory
// tiles filled by TMA, the multiply-accumulate is tcgen05.mma with the accumulator in tensor
// memory, and the alpha/beta broadcast of wmma.jl:678-716 is fused into the epilogue.
//
// One CTA (or a pair of CTAs on neighbouring SMs, kCtas == 2) owns an output tile of
// (128 * kCtas) x kBN.  Roles, by warp:
//   warp 0    TMA producer: streams 128 x 64 slices of op(A) and (kBN / kCtas) x 64 slices of
//             op(B) into a ring of shared-memory stages (128-byte swizzle)
//   warp 1    MMA issuer: one thread issues tcgen05.mma (K = 16 per instruction, 4 per stage)
//             and commits stage-release / accumulator-ready barriers
//   warp 2    allocates and frees tensor memory (two accumulators of kBN columns)
//   warp 3    idle
//   warps 4-7 epilogue: tcgen05.ld the accumulator (lane = row), combine with C staged in
//             shared memory by TMA, write the result back into the same staging buffer and
//             TMA-store it; double-buffered in chunks of 32 columns
// The two accumulators let the epilogue of tile i overlap the main loop of tile i + 1.
//
// Work units are (tile, k-slice) pairs; with split_k > 1 each unit writes a raw FP32 partial
// product to a scratch matrix and a second kernel reduces them (gemm_splitk_reduce).
//
// Batched problems (kBatch) run the same pipeline over 3-D tensor maps whose outermost coordinate is
// the matrix of the batch; a work unit is then (matrix, tile) and split-K is not used.
//
// Every barrier wait is bounded (ptx_sm100.cuh: mbar_wait); on expiry the CTA records the wait
// in the device status word and every role falls through to the common exit.
//
// The kernel is launched with programmatic stream serialization: its set-up (barriers, tensor
// memory, descriptor prefetch) runs under the tail of the previous kernel of the stream, and
// griddepcontrol.wait orders every global access behind that kernel's completion.
#pragma once

#include "ptx_sm100.cuh"

namespace b200 {

struct GemmParams {
    int M, N, K;
    int tiles_m, tiles_n;  // tile grid; a tile is (128 * kCtas) x kBN
    int split_k;           // k-slices per tile (>= 1)
    int kb_total;          // ceil(K / 64)
    int kb_per_split;      // ceil(kb_total / split_k)
    int raster_group;      // tiles_m per rasterisation group
    int out_n_stride;      // column offset between k-slices in the output map (split_k > 1)
    float alpha, beta;     // epilogue scalars (split_k > 1: 1 and 0)
    // Gated A: when panel_flags != nullptr, k-blocks [j * kb_per_panel, (j + 1) * kb_per_panel) of A
    // may be loaded only once panel_flags[j] != 0 (written by a stream memory operation after the
    // panel has arrived in this GPU's memory).  At most 32 panels.
    const unsigned int* panel_flags;
    int kb_per_panel;
    int c_fmt, d_fmt;      // element types of C and D in memory: 0 = binary32, 1 = binary16, 2 = bfloat16
    int ab_bf16;           // A and B are bfloat16 instead of binary16
    int acc_f16;           // accumulate in binary16 (tensor memory then holds one binary16 value per 32-bit cell)
    int batch;             // matrices per launch (kBatch kernels; the tensor maps are 3-D then)
    int* status;
    unsigned long long wait_budget_ns;
};

template <int kBN, bool kAMn, bool kBMn, int kCtas>
struct GemmCfg {
    static constexpr int BM = 128;                 // rows per CTA
    static constexpr int BK = 64;                  // k per stage: one 128-byte swizzle row
    static constexpr int BN = kBN;                 // columns per tile
    static constexpr int BN_LOCAL = kBN / kCtas;   // B rows this CTA loads
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN_LOCAL * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int EPI_COLS = 32;
    static constexpr int EPI_BYTES = BM * EPI_COLS * 4;
    static constexpr int EPI_BUFS = 2;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 1024 /*alignment slack*/ - 512 /*barriers*/;
    static constexpr int STAGES_RAW = (SMEM_BUDGET - EPI_BUFS * EPI_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int TMEM_COLS = 2 * kBN < 32 ? 32 : 2 * kBN;
    static constexpr int NCHUNK = kBN / EPI_COLS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BUFS * EPI_BYTES + 512 + 1024;
    static constexpr int THREADS = 256;
    static_assert(kBN % 32 == 0 && kBN >= 32 && kBN <= 256, "tile N");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");
    static_assert(STAGES >= 2, "pipeline depth");
    static_assert(kCtas == 1 || kCtas == 2, "CTAs per tile");
    static_assert(!kBMn || (BN_LOCAL % 64 == 0), "MN-major B loads 64 columns per box");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

// Maps a linear tile index to (tile_m, tile_n): tiles walk down M inside groups of
// `raster_group` tile rows so that concurrently running CTAs share A and B panels in L2.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
    const int per_group = p.raster_group * p.tiles_n;
    const int group = tile / per_group;
    const int first_m = group * p.raster_group;
    const int rows = min(p.raster_group, p.tiles_m - first_m);
    const int idx = tile - group * per_group;
    tm = first_m + idx % rows;
    tn = idx / rows;
}

template <int kBN, bool kAMn, bool kBMn, int kCtas, bool kBatch = false>
__global__ void __launch_bounds__(256, 1)
gemm_f16f32_tcgen05(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmD,
                    const GemmParams p) {
    using Cfg = GemmCfg<kBN, kAMn, kBMn, kCtas>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr bool kPair = (kCtas == 2);

    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzling is a function of the shared-memory address: stages start on 1 KiB.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t stages_base = smem_base;
    const uint32_t epi_base = smem_base + STAGES * Cfg::STAGE_BYTES;
    const uint32_t bar_base = epi_base + Cfg::EPI_BUFS * Cfg::EPI_BYTES;
    float* epi_gen = reinterpret_cast<float*>(smem_gen + STAGES * Cfg::STAGE_BYTES);
    uint8_t* bar_gen = smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BUFS * Cfg::EPI_BYTES;

    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    auto cfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 4 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * STAGES + 6));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * STAGES + 6) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
    const int unit_stride = kPair ? (gridDim.x >> 1) : gridDim.x;
    const int unit_first = kPair ? (blockIdx.x >> 1) : blockIdx.x;
    const int tiles_per_matrix = p.tiles_m * p.tiles_n;
    const int num_units = kBatch ? tiles_per_matrix * p.batch : tiles_per_matrix * p.split_k;

    WaitCtx wc{abort_flag, p.status, p.wait_budget_ns};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);       // the leader's arrive; it expects both CTAs' bytes
            mbar_init(empty_bar(s), 1);      // one tcgen05.commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), 4 * kCtas);  // one arrive per epilogue warp
        }
        for (int b = 0; b < Cfg::EPI_BUFS; ++b) mbar_init(cfull_bar(b), 1);
        fence_mbar_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        tma_prefetch_desc(&tmC);
        tma_prefetch_desc(&tmD);
    }
    if (warp == 2) tmem_alloc<kCtas>(smem_u32(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
    tc_fence_before_sync();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();  // peer barriers exist before anyone signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this CTA's own shared and tensor memory, so it may overlap the
    // tail of the previous kernel in the stream (whose last CTAs are still finishing while this CTA
    // already sits on an SM that has become free); global memory is touched only after the wait.
    griddep_launch_dependents();
    griddep_wait();

    // unit -> (tile row, tile col, k-block range, matrix of the batch)
    auto unit_decode = [&](int unit, int& m0, int& n0, int& kb0, int& kb1, int& out_n0, int& bz) {
        int tile, slice;
        if constexpr (kBatch) {
            bz = unit / tiles_per_matrix;
            tile = unit - bz * tiles_per_matrix;
            slice = 0;
        } else {
            bz = 0;
            tile = unit / p.split_k;
            slice = unit - tile * p.split_k;
        }
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        m0 = tm * (Cfg::BM * kCtas) + static_cast<int>(cta_rank) * Cfg::BM;
        n0 = tn * kBN;
        kb0 = slice * p.kb_per_split;
        kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        out_n0 = n0 + slice * p.out_n_stride;
    };
    // TMA copies of C / D chunks (2-D maps, or 3-D with the matrix index when batched)
    auto load_c_chunk = [&](uint32_t dst, int x, int y, int z, uint32_t bar, uint64_t policy) {
        if constexpr (kBatch) tma_load_3d_hint(dst, &tmC, x, y, z, bar, policy);
        else tma_load_2d_hint(dst, &tmC, x, y, bar, policy);
    };
    auto store_d_chunk = [&](int x, int y, int z, uint32_t src, uint64_t policy, bool hinted) {
        if constexpr (kBatch) {
            tma_store_3d_hint(&tmD, x, y, z, src, policy);
        } else {
            if (hinted) tma_store_2d_hint(&tmD, x, y, src, policy);
            else tma_store_2d(&tmD, x, y, src);  // partial products are read back by the reduction right away
        }
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int s = 0;          // stage of the ring
            uint32_t ph = 0;    // its phase bit
            bool ok = true;
            uint32_t panels_seen = p.panel_flags ? 0u : 0xffffffffu;  // bit j: panel j is known to be here
            // One tile column: every tile of A is read by exactly one CTA (the HBM-bound skinny shape).
            // Mark those loads evict-first so that the stream of A does not displace B, which every
            // CTA re-reads from L2.
            const bool a_once = (p.tiles_n == 1);
            const uint64_t once_policy = l2_policy_evict_first();
            int bz = 0;  // matrix of the batch the current unit belongs to
            auto load_a = [&](uint32_t dst, int x, int y, uint32_t bar) {
                if constexpr (kBatch) {
                    if constexpr (kPair) tma_load_3d_pair(dst, &tmA, x, y, bz, bar);
                    else tma_load_3d(dst, &tmA, x, y, bz, bar);
                } else if constexpr (kPair) {
                    if (a_once) tma_load_2d_pair_hint(dst, &tmA, x, y, bar, once_policy);
                    else tma_load_2d_pair(dst, &tmA, x, y, bar);
                } else {
                    if (a_once) tma_load_2d_hint(dst, &tmA, x, y, bar, once_policy);
                    else tma_load_2d(dst, &tmA, x, y, bar);
                }
            };
            auto load_b = [&](uint32_t dst, int x, int y, uint32_t bar) {
                if constexpr (kBatch) {
                    if constexpr (kPair) tma_load_3d_pair(dst, &tmB, x, y, bz, bar);
                    else tma_load_3d(dst, &tmB, x, y, bz, bar);
                } else if constexpr (kPair) {
                    tma_load_2d_pair(dst, &tmB, x, y, bar);
                } else {
                    tma_load_2d(dst, &tmB, x, y, bar);
                }
            };
            for (int unit = unit_first; ok && unit < num_units; unit += unit_stride) {
                int m0, n0, kb0, kb1, out_n0;
                unit_decode(unit, m0, n0, kb0, kb1, out_n0, bz);
                const int nb0 = n0 + static_cast<int>(cta_rank) * Cfg::BN_LOCAL;
                for (int kb = kb0; kb < kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
                    if (panels_seen != 0xffffffffu) {
                        const uint32_t panel = static_cast<uint32_t>(kb / p.kb_per_panel);
                        if (!((panels_seen >> panel) & 1u)) {
                            ok = flag_wait(p.panel_flags + panel, wc, kWaitPanel);
                            if (!ok) break;
                            panels_seen |= 1u << panel;
                        }
                    }
                    ok = mbar_wait(empty_bar(s), ph ^ 1u, wc, kWaitEmptyStage);
                    if (!ok) break;
                    const uint32_t sa = stages_base + s * Cfg::STAGE_BYTES;
                    const uint32_t sb = sa + Cfg::A_BYTES;
                    const int k0 = kb * Cfg::BK;
                    if constexpr (!kPair) {
                        const uint32_t fb = full_bar(s);
                        mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
                        if constexpr (kAMn) {
                            load_a(sa, m0, k0, fb);
                            load_a(sa + 8192, m0 + 64, k0, fb);
                        } else {
                            load_a(sa, k0, m0, fb);
                        }
                        if constexpr (kBMn) {
#pragma unroll
                            for (int i = 0; i < Cfg::BN_LOCAL / 64; ++i)
                                load_b(sb + i * 8192, nb0 + i * 64, k0, fb);
                        } else {
                            load_b(sb, k0, nb0, fb);
                        }
                    } else {
                        // Both CTAs' loads complete on the leader's barrier.  Only the leader
                        // arrives, expecting the bytes of both: a cluster-scope (remote) arrive
                        // per k-block from the peer would cost a memory barrier each time.  The
                        // peer's bytes may land before the leader's expect_tx; the phase cannot
                        // complete before the leader's arrival, so that is harmless.
                        const uint32_t fb = mapa_shared(full_bar(s), 0);
                        if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
                        if constexpr (kAMn) {
                            load_a(sa, m0, k0, fb);
                            load_a(sa + 8192, m0 + 64, k0, fb);
                        } else {
                            load_a(sa, k0, m0, fb);
                        }
                        if constexpr (kBMn) {
#pragma unroll
                            for (int i = 0; i < Cfg::BN_LOCAL / 64; ++i)
                                load_b(sb + i * 8192, nb0 + i * 64, k0, fb);
                        } else {
                            load_b(sb, k0, nb0, fb);
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && cta_rank == 0) {
            const uint32_t idesc = make_idesc_f16_f32(Cfg::BM * kCtas, kBN, kAMn ? 1 : 0, kBMn ? 1 : 0, p.ab_bf16 ? 1 : 0,
                                                      p.acc_f16 ? 1 : 0);
            // Descriptors differ between stages and k-steps only in their start-address field
            // (bits [0,14), in units of 16 bytes): build them once and add offsets.
            // K-major tile: rows of 128 B, 8-row groups 1 KiB apart, k = 16 advances 32 B inside
            // the swizzled row.  MN-major tile: 64 (m or n) x 64 k boxes of 8 KiB, 8-k groups
            // 1 KiB apart, k = 16 advances 2 KiB.
            const uint64_t da0 = kAMn ? make_smem_desc(stages_base, 8192, 1024, kSwizzle128B)
                                      : make_smem_desc(stages_base, 16, 1024, kSwizzle128B);
            const uint64_t db0 = kBMn ? make_smem_desc(stages_base + Cfg::A_BYTES, 8192, 1024, kSwizzle128B)
                                      : make_smem_desc(stages_base + Cfg::A_BYTES, 16, 1024, kSwizzle128B);
            constexpr uint32_t kStepA = (kAMn ? 2048 : 32) >> 4, kStepB = (kBMn ? 2048 : 32) >> 4;
            int s = 0;
            uint32_t ph = 0, ucount = 0;
            bool ok = true;
            for (int unit = unit_first; ok && unit < num_units; unit += unit_stride, ++ucount) {
                int m0, n0, kb0, kb1, out_n0, bz;
                unit_decode(unit, m0, n0, kb0, kb1, out_n0, bz);
                const uint32_t acc = ucount & 1u;
                const uint32_t aph = (ucount >> 1) & 1u;
                ok = mbar_wait(tmem_empty_bar(acc), aph ^ 1u, wc, kWaitTmemEmpty);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                uint32_t accumulate = 0;
                for (int kb = kb0; kb < kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
                    ok = mbar_wait(full_bar(s), ph, wc, kWaitFullStage);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t da = da0 + static_cast<uint64_t>(s * (Cfg::STAGE_BYTES >> 4));
                    const uint64_t db = db0 + static_cast<uint64_t>(s * (Cfg::STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < Cfg::BK / 16; ++k) {
                        umma_f16<kCtas>(d_tmem, da + k * kStepA, db + k * kStepB, idesc, accumulate);
                        accumulate = 1u;
                    }
                    if constexpr (kPair) umma_commit_pair(empty_bar(s));
                    else umma_commit<kCtas>(empty_bar(s));
                }
                if (!ok) break;
                if constexpr (kPair) umma_commit_pair(tmem_full_bar(acc));
                else umma_commit<kCtas>(tmem_full_bar(acc));
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        const int et = threadIdx.x - 128;          // 0..127 = accumulator row inside the CTA
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const bool elected = (et == 0);
        const bool has_c = (p.beta != 0.0f);
        const float alpha = p.alpha, beta = p.beta;
        const bool c_half = p.c_fmt != 0, d_half = p.d_fmt != 0;  // 2-byte elements
        const bool c_bf16 = p.c_fmt == 2, d_bf16 = p.d_fmt == 2;
        const bool acc_f16 = p.acc_f16 != 0;
        const uint32_t c_chunk_bytes = c_half ? Cfg::EPI_BYTES / 2 : Cfg::EPI_BYTES;
        // C is updated in place in the staging buffer only if D has the same element size; otherwise
        // every thread must have read its C values before anybody writes D over them
        const bool two_phase = has_c && (c_half != d_half);

        auto chunks_of = [&](int n0) { return min(Cfg::NCHUNK, (p.N - n0 + Cfg::EPI_COLS - 1) / Cfg::EPI_COLS); };

        // C is read once and D written once: keep them from displacing the shared A / B panels in L2
        const uint64_t stream_policy = l2_policy_evict_first();
        uint32_t g = 0;  // chunk counter: staging buffer g & 1, C-barrier phase (g >> 1) & 1
        if (has_c && elected && unit_first < num_units) {
            int m0, n0, kb0, kb1, out_n0, bz;
            unit_decode(unit_first, m0, n0, kb0, kb1, out_n0, bz);
            mbar_arrive_expect_tx(cfull_bar(0), c_chunk_bytes);
            load_c_chunk(epi_base, m0, n0, bz, cfull_bar(0), stream_policy);
        }
        uint32_t ucount = 0;
        bool fail = false;
        for (int unit = unit_first; unit < num_units; unit += unit_stride, ++ucount) {
            int m0, n0, kb0, kb1, out_n0, bz;
            unit_decode(unit, m0, n0, kb0, kb1, out_n0, bz);
            const int nchunks = chunks_of(n0);
            const uint32_t acc = ucount & 1u;
            const uint32_t aph = (ucount >> 1) & 1u;
            bool ok = mbar_wait(tmem_full_bar(acc), aph, wc, kWaitTmemFull);
            tc_fence_after_sync();
            for (int j = 0; j < nchunks; ++j, ++g) {
                const uint32_t buf = g & 1u;
                if (elected) {
                    if (has_c) {
                        // fetch the next chunk of C into the other buffer once the store that
                        // last used it has finished reading shared memory
                        int nm0 = m0, nn0 = n0 + (j + 1) * Cfg::EPI_COLS, nbz = bz;
                        bool have_next = (j + 1 < nchunks);
                        if (!have_next && unit + unit_stride < num_units) {
                            int a, b, c;
                            unit_decode(unit + unit_stride, nm0, nn0, a, b, c, nbz);
                            have_next = true;
                        }
                        if (have_next) {
                            tma_store_wait_read<0>();
                            mbar_arrive_expect_tx(cfull_bar(buf ^ 1u), c_chunk_bytes);
                            load_c_chunk(epi_base + (buf ^ 1u) * Cfg::EPI_BYTES, nm0, nn0, nbz, cfull_bar(buf ^ 1u),
                                         stream_policy);
                        }
                    } else {
                        tma_store_wait_read<1>();
                    }
                }
                if (has_c) {
                    ok = ok && mbar_wait(cfull_bar(buf), (g >> 1) & 1u, wc, kWaitCTile);
                } else {
                    named_bar_sync(1, 128);
                }
                ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective
                uint32_t r[32];
                float* col = epi_gen + buf * (Cfg::EPI_BYTES / 4) + et;                      // binary32 view
                __half* colh = reinterpret_cast<__half*>(epi_gen + buf * (Cfg::EPI_BYTES / 4)) + et;  // binary16 view
                __nv_bfloat16* colb = reinterpret_cast<__nv_bfloat16*>(colh);                        // bfloat16 view
                if (ok) {
                    tmem_ld_32x32b_x32(tmem_base + lane_base + acc * kBN + j * Cfg::EPI_COLS, r);
                    tmem_wait_ld();
                    if (acc_f16) {  // a binary16 accumulator sits in the low half of its 32-bit cell
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            r[i] = __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(r[i] & 0xffffu))));
                    }
                    if (has_c) {
                        if (c_bf16) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                r[i] = __float_as_uint(fmaf(alpha, __uint_as_float(r[i]), beta * __bfloat162float(colb[i * Cfg::BM])));
                        } else if (c_half) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                r[i] = __float_as_uint(fmaf(alpha, __uint_as_float(r[i]), beta * __half2float(colh[i * Cfg::BM])));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                r[i] = __float_as_uint(fmaf(alpha, __uint_as_float(r[i]), beta * col[i * Cfg::BM]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(alpha * __uint_as_float(r[i]));
                    }
                }
                if (two_phase) named_bar_sync(3, 128);
                if (ok) {
                    if (d_bf16) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) colb[i * Cfg::BM] = __float2bfloat16_rn(__uint_as_float(r[i]));
                    } else if (d_half) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) colh[i * Cfg::BM] = __float2half_rn(__uint_as_float(r[i]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) col[i * Cfg::BM] = __uint_as_float(r[i]);
                    }
                    fence_proxy_async_smem();
                }
                fail = named_bar_or(2, 128, !ok);
                if (fail) break;
                if (elected && m0 < p.M) {  // a pair's second CTA may own no rows of a bottom-edge tile
                    store_d_chunk(m0, out_n0 + j * Cfg::EPI_COLS, bz, epi_base + buf * Cfg::EPI_BYTES, stream_policy,
                                  p.split_k <= 1);
                    tma_store_commit();
                }
            }
            if (fail) break;
            // the accumulator has been read out: hand it back to the MMA issuer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if constexpr (kPair) mbar_arrive_cluster(tmem_empty_bar(acc), 0);
                else mbar_arrive(tmem_empty_bar(acc));
            }
        }
        if (elected) tma_store_wait_all<0>();
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // give bulk copies that may still be in flight towards this CTA time to land
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    if constexpr (kPair) cluster_sync_all();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc<kCtas>(tmem_base, Cfg::TMEM_COLS);
    }
}

// D[m, n] = alpha * sum_s ws[m, n + s * n_stride] + beta * C[m, n]; ws column-major with ldw.
// Four rows per thread (M-contiguous float4 when everything is binary32 and 16-byte aligned).
__global__ void gemm_splitk_reduce(const float* __restrict__ ws, long long ldw, int n_stride,
                                   int split_k, int M, int N, float alpha, float beta,
                                   const void* __restrict__ Cv, long long ldc, void* __restrict__ Dv,
                                   long long ldd, int vec_ok, int c_fmt, int d_fmt) {
    const float* C = static_cast<const float*>(Cv);
    float* D = static_cast<float*>(Dv);
    const __half* Ch = static_cast<const __half*>(Cv);
    __half* Dh = static_cast<__half*>(Dv);
    const __nv_bfloat16* Cb = static_cast<const __nv_bfloat16*>(Cv);
    __nv_bfloat16* Db = static_cast<__nv_bfloat16*>(Dv);
    const long long quads_m = (M + 3) / 4;
    const long long total = quads_m * N;
    for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < total;
         q += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(q / quads_m);
        const int m = static_cast<int>(q - n * quads_m) * 4;
        if (vec_ok && m + 3 < M) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < split_k; ++s) {
                const float4 v = *reinterpret_cast<const float4*>(ws + (n + static_cast<long long>(s) * n_stride) * ldw + m);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            float4 out = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
            if (beta != 0.0f) {
                const float4 c = *reinterpret_cast<const float4*>(C + n * ldc + m);
                out.x = fmaf(beta, c.x, out.x); out.y = fmaf(beta, c.y, out.y);
                out.z = fmaf(beta, c.z, out.z); out.w = fmaf(beta, c.w, out.w);
            }
            *reinterpret_cast<float4*>(D + n * ldd + m) = out;
        } else {
            for (int i = 0; i < 4 && m + i < M; ++i) {
                float acc = 0.f;
                for (int s = 0; s < split_k; ++s) acc += ws[(n + static_cast<long long>(s) * n_stride) * ldw + m + i];
                float out = alpha * acc;
                if (beta != 0.0f) {
                    const long long ci = n * ldc + m + i;
                    out = fmaf(beta, c_fmt == 2 ? __bfloat162float(Cb[ci]) : c_fmt == 1 ? __half2float(Ch[ci]) : C[ci], out);
                }
                const long long di = n * ldd + m + i;
                if (d_fmt == 2) Db[di] = __float2bfloat16_rn(out);
                else if (d_fmt == 1) Dh[di] = __float2half_rn(out);
                else D[di] = out;
            }
        }
    }
}

}  // namespace b200
