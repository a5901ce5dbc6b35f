// Inline-PTX building blocks for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM allocation, MMA, commit, load/store) and the shared-memory / instruction descriptors
// tcgen05.mma consumes.  Everything here is device-only and header-only.
//
// Every wait on an mbarrier is bounded: see mbar_wait().  Every bulk load writes only the
// issuing CTA's own shared memory.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------------------------
// addresses, timers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on the barrier at the same offset in CTA `cta_rank` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank) {
    asm volatile(
        "{\n"
        ".reg .b32 remote;\n"
        "mapa.shared::cluster.u32 remote, %0, %1;\n"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n"
        "}" ::"r"(bar),
        "r"(cta_rank)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Same test, but the thread may stay suspended for up to `hint_ns` while the phase is incomplete; it
// resumes at once when the phase completes.  Without the hint the hardware's own limit is short, and
// the six waiting warps of a GEMM CTA then poll so often that they take issue slots from the one
// thread that feeds the tensor pipe (measured: 4 % of the cycles of an 8192^3 product, 15 % of a
// skinny one).
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// ids written to the status word when a wait runs out
enum : int {
    kWaitEmptyStage = 101,   // producer waiting for the MMA to release a stage
    kWaitFullStage = 102,    // MMA waiting for TMA data
    kWaitTmemEmpty = 103,    // MMA waiting for the epilogue to drain an accumulator
    kWaitTmemFull = 104,     // epilogue waiting for the accumulator
    kWaitCTile = 105,        // epilogue waiting for its C chunk
    kWaitUnit = 106,         // 16x16x16 unit waiting for its MMA
    kWaitSelftest = 107,     // the bounded-wait self test (nothing ever arrives)
    kWaitPanel = 108         // producer waiting for a panel of A to arrive in this GPU's memory
};

// What a kernel needs to give up on a wait cleanly.
struct WaitCtx {
    volatile int* abort_flag;      // in shared memory; set once by whoever gives up first
    int* status;                   // 4 ints in global memory: {code, block, detail, spare}
    unsigned long long budget_ns;  // how long one wait may spin (see mbar_wait)
};

// Records the first failure of the grid in the status word and raises the CTA's abort flag.
static __device__ __noinline__ void report_timeout(const WaitCtx& w, int where, int detail) {
    *w.abort_flag = 1;
    if (atomicCAS(w.status, 0, where) == 0) {
        w.status[1] = static_cast<int>(blockIdx.x);
        w.status[2] = detail;
        __threadfence();
    }
}

// Bounded wait for phase `parity` of an mbarrier.  Returns false when the budget ran out or
// another role of this CTA already gave up; the caller must then fall through to the kernel's
// common exit (which frees TMEM).  Never spins unboundedly.
//
// The budget is counted on the SM's cycle counter (reading %globaltimer costs a large fraction of
// a microsecond, which a producer that is one stage ahead would pay on every k-block) at two
// cycles per nanosecond: with SM clocks between 1 and 2 GHz a wait gives up after one to two
// times budget_ns.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, int where) {
    // Every poll carries the suspend hint, the first one too: a poll without it comes back so soon that the
    // waiting warps of the CTA keep the issue slots busy.  The thread sleeps in hardware until the phase
    // completes, 50 us at most; the abort flag and the budget are looked at that often.
    if (mbar_try_wait_suspend(bar, parity, 50000u)) return true;
    const long long t0 = clock64();
    const long long budget_cycles = static_cast<long long>(w.budget_ns) * 2;
    for (;;) {
        if (mbar_try_wait_suspend(bar, parity, 50000u)) return true;
        if (*w.abort_flag) return false;
        if (clock64() - t0 > budget_cycles) {
            report_timeout(w, where, static_cast<int>(parity));
            return false;
        }
    }
}

// Bounded wait for a 32-bit word in global memory to become non-zero.  The word is written by a
// stream memory operation (not by a kernel) once data that a copy engine moved into this GPU's
// memory is complete; the acquire at system scope plus the proxy fence order the bulk loads that
// follow after the data.
__device__ __forceinline__ bool flag_wait(const unsigned int* flag, const WaitCtx& w, int where) {
    const long long t0 = clock64();
    const long long budget_cycles = static_cast<long long>(w.budget_ns) * 2;
    uint32_t spins = 0;
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v != 0u) {
            asm volatile("fence.proxy.async;" ::: "memory");
            return true;
        }
        __nanosleep(200);
        if ((++spins & 15u) == 0u) {
            if (*w.abort_flag) return false;
            if (clock64() - t0 > budget_cycles) {
                report_timeout(w, where, static_cast<int>(spins));
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// proxies and named barriers
// ---------------------------------------------------------------------------------------------
// Makes this thread's generic-proxy shared-memory writes visible to the async proxy (TMA
// stores, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Barrier + OR-reduction of a predicate over the participating threads.
__device__ __forceinline__ bool named_bar_or(uint32_t id, uint32_t nthreads, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n"
        ".reg .pred pin, pout;\n"
        "setp.ne.u32 pin, %3, 0;\n"
        "barrier.cta.red.or.pred pout, %1, %2, pin;\n"
        "selp.u32 %0, 1, 0, pout;\n"
        "}"
        : "=r"(out)
        : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
        : "memory");
    return out != 0;
}

// ---------------------------------------------------------------------------------------------
// clusters
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while the kernel
// before it in the stream is still running.  griddep_wait() returns once that kernel has completed
// and its memory operations are visible: nothing that reads or writes global memory may come before
// it.  griddep_launch_dependents() tells the scheduler that the NEXT kernel in the stream may be
// brought onto SMs as they free up.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// 2-D tiled load global -> this CTA's shared memory, completion on an mbarrier of this CTA.
// x is the innermost coordinate: x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tm, int x,
                                            int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Same for a CTA of a 2-CTA pair: the mbarrier operand is a shared::cluster address, so the
// transaction bytes may be signalled to the pair leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* tm, int x,
                                                 int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}

// L2 eviction policies for streaming data (read or written once, never reused by another CTA):
// marking it evict-first keeps it from displacing the A / B panels the co-resident CTAs share.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* tm, int x, int y,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* tm, int x, int y, uint32_t src_smem,
                                                  uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;" ::"l"(
            reinterpret_cast<uint64_t>(tm)),
        "r"(x), "r"(y), "r"(src_smem), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst_smem, const CUtensorMap* tm, int x, int y,
                                                      uint32_t bar_cluster_addr, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar_cluster_addr), "l"(policy)
        : "memory");
}

// 2-D tiled store shared -> global, tracked by this thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, int x, int y,
                                             uint32_t src_smem) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                     reinterpret_cast<uint64_t>(tm)),
                 "r"(x), "r"(y), "r"(src_smem)
                 : "memory");
}

// 3-D forms of the copies above for batched problems: z selects the matrix of the batch (box extent 1
// in that dimension, so the shared-memory image of a tile is the same as in the 2-D case).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* tm, int x, int y, int z,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst_smem, const CUtensorMap* tm, int x, int y, int z,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst_smem, const CUtensorMap* tm, int x, int y, int z,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t dst_smem, const CUtensorMap* tm, int x, int y,
                                                      int z, uint32_t bar_cluster_addr, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tm, int x, int y, int z, uint32_t src_smem) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                     reinterpret_cast<uint64_t>(tm)),
                 "r"(x), "r"(y), "r"(z), "r"(src_smem)
                 : "memory");
}

__device__ __forceinline__ void tma_store_3d_hint(const CUtensorMap* tm, int x, int y, int z, uint32_t src_smem,
                                                  uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2, %3}], [%4], %5;" ::"l"(
            reinterpret_cast<uint64_t>(tm)),
        "r"(x), "r"(y), "r"(z), "r"(src_smem), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Wait until at most N of this thread's bulk groups are incomplete (writes globally done).
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM allocation
// ---------------------------------------------------------------------------------------------
// One full warp; ncols a power of two in [32, 512].  The TMEM base address lands in *slot.
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         slot_smem),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         slot_smem),
                     "r"(ncols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (kCtaGroup == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr),
                     "r"(ncols)
                     : "memory");
    }
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------------------------
// Instruction descriptor of tcgen05.mma.kind::f16 with binary16 (or, ab_bf16 = 1, bfloat16) A and
// B and a binary32 (or, d_f16 = 1, binary16) accumulator.  Bit layout (PTX ISA, "Instruction descriptor"): [4,6) D format
// (0 = F16, 1 = F32), [7,10) A format (0 = F16, 1 = BF16), [10,13) B format, [15] A major (0 = K, 1 = MN), [16] B major,
// [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16_f32(int m, int n, int a_mn_major,
                                                          int b_mn_major, int ab_bf16 = 0, int d_f16 = 0) {
    return ((d_f16 ? 0u : 1u) << 4) | (static_cast<uint32_t>(ab_bf16) << 7) | (static_cast<uint32_t>(ab_bf16) << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor (PTX ISA, "Shared memory descriptor"): [0,14) start address
// >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4, [46,48) version
// (1 on sm_100), [61,64) swizzle mode (0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B).
constexpr uint32_t kSwizzleNone = 0;
constexpr uint32_t kSwizzle128B = 2;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swizzle & 7u) << 61;
    return d;
}

// ---------------------------------------------------------------------------------------------
// tcgen05: MMA, commit
// ---------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
template <int kCtaGroup>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    if constexpr (kCtaGroup == 1) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
            "}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Arrive on an mbarrier once every tcgen05 operation this thread issued so far has completed.
// `bar` is a shared::cluster address: a plain shared::cta address names this CTA's own barrier,
// a mapa-translated one names a peer CTA's.
template <int kCtaGroup>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if constexpr (kCtaGroup == 1) {
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                bar)
            : "memory");
    } else {
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                bar)
            : "memory");
    }
}

// 2-CTA form that arrives on the barrier at offset `bar` in BOTH CTAs of the pair (CTA mask 0b11)
// with one instruction.  This qualifier applies to the commit's barrier signal only; no load in
// this library carries it.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(static_cast<uint16_t>(3))
        : "memory");
}

__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}

// ---------------------------------------------------------------------------------------------
// tcgen05: TMEM <-> registers.  Warp w may touch TMEM lanes 32*(w%4) .. 32*(w%4)+31; with the
// 32x32b shape, thread t of the warp gets lane 32*(w%4)+t and register i gets column c+i.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

}  // namespace b200
