// The N-sharded multi-GPU GEMM behind the C ABI (b200_sharded_*), one object per rank.
//
//     D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]          on every rank r
//
// B, C and D are split into contiguous column slabs that never move.  A (M x K column-major,
// lda = M, binary16) starts on rank 0 and reaches every rank's own memory in K panels while the
// GEMM on the panels that have already arrived is running; every TMA load reads local memory.
// There is no output collective: D stays sharded like C.
//
// Transport, per panel: rank 0 copies sub-block g of the panel into rank g's A (scatter), then every
// rank copies its sub-block into every other rank's A (all-gather), so that no GPU sends more than
// the panel's size.  The copies run on the copy engines (cudaMemcpyAsync between peer-mapped
// buffers): no kernel, no SM.  Ordering is by stream memory operations: behind each copy the sending
// stream writes the call's epoch into a flag word in the RECEIVER's flag block, and the receiver's
// streams wait (>=) for those words before they forward the data or launch the GEMM that reads it.
// Every wait therefore looks at this rank's own flag block, which is what lets b200_sharded_wait
// release a rank whose peer never wrote.
//
// The product is a few GEMM launches over growing K ranges, each accumulating into D and ordered
// behind the arrival of its own panels only.
//
// The reference has no multi-GPU code (its only multi-device facility is device!(), src/init.jl:
// 187-209 of CUDAnative.jl); what this file keeps from it is the calling convention: raw device
// pointers owned by the caller (src/array.jl:15), asynchronous enqueue on the caller's stream
// (src/execution.jl:158-166), failures found by polling at a later call (src/exceptions.jl:76-89).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "internal.h"

namespace b200 {

// ---------------------------------------------------------------------------------------------
// layout arithmetic (host only)
// ---------------------------------------------------------------------------------------------
// Range `part` of [0, n) cut into `parts` contiguous pieces whose starts are multiples of `align`,
// as even as whole blocks of `align` allow.
static void even_split(int64_t n, int parts, int part, int64_t align, int64_t* lo, int64_t* hi) {
    const int64_t blocks = (n + align - 1) / align;
    const int64_t per = blocks / parts, extra = blocks % parts;
    const int64_t b0 = part * per + std::min<int64_t>(part, extra);
    const int64_t b1 = b0 + per + (part < extra ? 1 : 0);
    *lo = std::min(b0 * align, n);
    *hi = std::min(b1 * align, n);
}

struct ShardLayout {
    int world = 1;
    std::vector<int64_t> slab;           // world + 1 column bounds of B / C / D
    int64_t panel_k = 0;                 // columns of A per transfer panel (multiple of 64)
    std::vector<int64_t> panel;          // panels + 1 column bounds of A
    std::vector<int> group;              // groups + 1 panel bounds: GEMM launch i covers panels [group[i], group[i+1])
    std::vector<int64_t> sub;            // [(p * world + g) * 2 + {0,1}]: columns of A rank g forwards in panel p
    int panels() const { return static_cast<int>(panel.size()) - 1; }
    int groups() const { return static_cast<int>(group.size()) - 1; }
};

static int make_layout(int world, int64_t N, int64_t K, int panels, int first_group, ShardLayout* out) {
    if (world < 1 || world > B200_SHARDED_MAX_RANKS) return fail(B200_INVALID_ARG, "sharded: world must be in [1, 64]");
    if (N < 0 || K <= 0) return fail(B200_INVALID_ARG, "sharded: N must be >= 0 and K positive");
    ShardLayout L;
    L.world = world;
    L.slab.resize(world + 1);
    for (int r = 0; r < world; ++r) {
        int64_t lo, hi;
        even_split(N, world, r, 256, &lo, &hi);  // whole 256-column tiles per rank
        L.slab[r] = lo;
        L.slab[r + 1] = hi;
    }
    int np = std::max(1, std::min(world > 1 ? panels : 1, B200_SHARDED_MAX_PANELS));
    const int64_t per = (K + np - 1) / np;
    L.panel_k = (per + 63) / 64 * 64;  // a panel starts on a shared-memory stage boundary
    for (int64_t k0 = 0; k0 < K; k0 += L.panel_k) L.panel.push_back(k0);
    L.panel.push_back(K);
    np = L.panels();
    // GEMM launches over growing K ranges: 1, 2, 2, 3, 4, 4 ... panels (ceil(1.4^i), at most a quarter of
    // the panels).  The first launch starts when little of A has arrived; a launch can only start once its
    // last panel is here, so late launches must stay short enough that the wait for that panel does not
    // idle the GPU, and long enough that their fixed cost and their extra pass over D do not matter.
    // Measured on 8 GPUs (32768 x 32768 x 16384, 16 panels arriving 0.19 ms apart against 0.22 ms of GEMM
    // per panel): 1,2,6,7 -> 4.70 ms; 2,2,4,4,4 -> 4.12; 1,2,3,3,3,4 -> 4.11; 1,2,2,3,4,4 -> 4.08;
    // 1,1,2,2,3,3,4 -> 4.16.
    const int cap = std::max({1, first_group, np / 4});
    int p = 0;
    double size = std::max(1, first_group);
    L.group.push_back(0);
    while (p < np) {
        const int q = std::min(np, p + std::min(cap, static_cast<int>(std::ceil(size - 1e-9))));
        L.group.push_back(q);
        size *= 1.4;
        p = q;
    }
    const int ng = L.groups();
    if (ng > 1 && (L.group[ng] - L.group[ng - 1]) * 2 < (L.group[ng - 1] - L.group[ng - 2])) {
        L.group.erase(L.group.end() - 2);  // a short tail joins the launch before it
    }
    // ownership during the transfer: a panel is cut into world - 1 sub-blocks, one per receiving rank,
    // so that rank 0 sends every byte of A exactly once and forwards nothing
    L.sub.assign(static_cast<size_t>(np) * world * 2, 0);
    for (int pp = 0; pp < np; ++pp) {
        const int64_t k0 = L.panel[pp], k1 = L.panel[pp + 1];
        L.sub[(static_cast<size_t>(pp) * world) * 2] = k0;
        L.sub[(static_cast<size_t>(pp) * world) * 2 + 1] = k0;
        for (int g = 1; g < world; ++g) {
            int64_t lo, hi;
            even_split(k1 - k0, world - 1, g - 1, 8, &lo, &hi);
            L.sub[(static_cast<size_t>(pp) * world + g) * 2] = k0 + lo;
            L.sub[(static_cast<size_t>(pp) * world + g) * 2 + 1] = k0 + hi;
        }
    }
    *out = std::move(L);
    return B200_OK;
}

// ---------------------------------------------------------------------------------------------
// stream memory operations
// ---------------------------------------------------------------------------------------------
// flag block layout (32-bit words): done[64] | scattered[32] (+32 spare) | gathered[32][64]
static inline size_t word_done(int g) { return 4u * static_cast<size_t>(g); }
static inline size_t word_scat(int p) { return 4u * (64u + static_cast<size_t>(p)); }
static inline size_t word_gath(int p, int g) { return 4u * (128u + static_cast<size_t>(p) * 64u + static_cast<size_t>(g)); }
static_assert(B200_SHARDED_FLAG_BYTES == 4 * (128 + B200_SHARDED_MAX_PANELS * 64), "flag block layout");
static_assert(B200_SHARDED_MAX_RANKS == 64, "flag block layout");

using BatchFn = CUresult (*)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);

static BatchFn batch_fn() {
    static BatchFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<BatchFn>(p);
    }
    return fn;
}

// One driver call for a list of 32-bit waits (>=) or writes on a stream.
struct MemOps {
    std::vector<CUstreamBatchMemOpParams> ops;
    void wait(void* base, size_t off, uint32_t value) {
        CUstreamBatchMemOpParams o;
        std::memset(&o, 0, sizeof(o));
        o.waitValue.operation = CU_STREAM_MEM_OP_WAIT_VALUE_32;
        o.waitValue.address = reinterpret_cast<CUdeviceptr>(static_cast<char*>(base) + off);
        o.waitValue.value = value;
        o.waitValue.flags = CU_STREAM_WAIT_VALUE_GEQ;
        ops.push_back(o);
    }
    void write(void* base, size_t off, uint32_t value) {
        CUstreamBatchMemOpParams o;
        std::memset(&o, 0, sizeof(o));
        o.writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_32;
        o.writeValue.address = reinterpret_cast<CUdeviceptr>(static_cast<char*>(base) + off);
        o.writeValue.value = value;
        o.writeValue.flags = 0;
        ops.push_back(o);
    }
    int flush(cudaStream_t stream, const char* what) {
        if (ops.empty()) return B200_OK;
        BatchFn fn = batch_fn();
        if (!fn) return fail(B200_CUDA_ERROR, "cuStreamBatchMemOp entry point not found");
        for (size_t i = 0; i < ops.size(); i += 128) {
            const unsigned n = static_cast<unsigned>(std::min<size_t>(128, ops.size() - i));
            CUresult r = fn(static_cast<CUstream>(stream), n, ops.data() + i, 0);
            if (r != CUDA_SUCCESS)
                return fail(B200_CUDA_ERROR, std::string("cuStreamBatchMemOp failed for ") + what + " (CUresult " +
                                                 std::to_string(static_cast<int>(r)) + ")");
        }
        ops.clear();
        return B200_OK;
    }
};

}  // namespace b200

using namespace b200;

struct b200_sharded {
    b200_handle* h = nullptr;
    int rank = 0, world = 1;
    int64_t M = 0, N = 0, K = 0;
    ShardLayout lay;
    // this rank's A and flag block (owned), and everybody's as this rank addresses them
    void* a_local = nullptr;
    void* flags_local = nullptr;
    std::vector<void*> a_peers, flag_peers;
    std::vector<char> ipc_mapped;  // peer g was opened through CUDA IPC (needs closing)
    bool attached = false;
    cudaStream_t scatter = nullptr, gather = nullptr, rescue = nullptr;
    // Copies to different receivers may run side by side on several copy engines: lane 0 of each kind is
    // the stream above, further lanes are created when the option asks for them.
    std::vector<cudaStream_t> scatter_lanes, gather_lanes;
    int first_group = 1;
    int panels_requested = 16;
    cudaEvent_t fork = nullptr;
    uint32_t* gate_words = nullptr;
    uint32_t epoch = 0;
    bool poisoned = false;
    cudaStream_t last_compute = nullptr;
    bool in_flight = false;
};

namespace {

int p2p_begin(b200_sharded* s, cudaStream_t compute) {
    // "I no longer touch my A from the previous product" to every peer; the streams that are about to
    // overwrite the peers' A wait until every peer has said the same for this epoch
    int rc;
    MemOps tell;
    for (int g = 0; g < s->world; ++g)
        if (g != s->rank) tell.write(s->flag_peers[g], word_done(s->rank), s->epoch);
    if ((rc = tell.flush(compute, "done flags"))) return rc;
    auto hear_on = [&](cudaStream_t st) -> int {
        MemOps hear;
        for (int g = 0; g < s->world; ++g)
            if (g != s->rank) hear.wait(s->flags_local, word_done(g), s->epoch);
        return hear.flush(st, "done waits");
    };
    if (s->rank == 0)  // only rank 0 scatters
        for (cudaStream_t st : s->scatter_lanes)
            if ((rc = hear_on(st))) return rc;
    for (cudaStream_t st : s->gather_lanes)
        if ((rc = hear_on(st))) return rc;
    return B200_OK;
}

int p2p_exchange(b200_sharded* s, int p0, int p1, cudaStream_t compute, bool gates) {
    const int rank = s->rank, world = s->world;
    const int64_t M = s->M;
    int rc;
    // Copies of one panel go out back to back on their lane; the words that tell the receivers that they
    // have landed follow as ONE batch of stream writes per lane.  Anything that is not another copy costs
    // the stream about 40 us on this path (measured on 8 GPUs: a write -- or a 4-byte copy carrying the
    // word -- behind every copy makes the 1 GiB of A take 9.9 ms instead of 3.1 ms), so there are as few
    // of them as the pipelining of scatter and all-gather allows.
    auto send_cols = [&](int dst, int64_t c0, int64_t c1, cudaStream_t st) -> int {
        if (c1 <= c0) return B200_OK;
        char* d = static_cast<char*>(s->a_peers[dst]) + 2 * c0 * M;
        const char* src = static_cast<const char*>(s->a_local) + 2 * c0 * M;
        B200_CUDA_TRY(cudaMemcpyAsync(d, src, static_cast<size_t>(2 * (c1 - c0) * M), cudaMemcpyDefault, st));
        return B200_OK;
    };
    const int ns = static_cast<int>(s->scatter_lanes.size()), ng = static_cast<int>(s->gather_lanes.size());
    std::vector<MemOps> landed(std::max(ns, ng));
    MemOps arrived;  // what the compute stream waits for before the launch that reads panels [p0, p1): one batch
    for (int p = p0; p < p1; ++p) {
        const int64_t* sub = s->lay.sub.data() + static_cast<size_t>(p) * world * 2;
        if (rank == 0) {  // scatter: sub-block g goes to rank g
            for (int g = 1; g < world; ++g) {
                const int lane = (g - 1) % ns;
                if ((rc = send_cols(g, sub[2 * g], sub[2 * g + 1], s->scatter_lanes[lane]))) return rc;
                landed[lane].write(s->flag_peers[g], word_scat(p), s->epoch);
            }
            for (int lane = 0; lane < ns; ++lane)
                if ((rc = landed[lane].flush(s->scatter_lanes[lane], "scatter flags"))) return rc;
        } else {
            // all-gather: my sub-block goes to everybody but rank 0, which has all of A.  It must be here
            // before I can pass it on.  Destinations are visited starting after this rank, so that at any
            // moment the senders aim at different receivers instead of all at the same one.
            for (int l = 0; l < std::min(ng, world - 2); ++l) {
                MemOps got;
                got.wait(s->flags_local, word_scat(p), s->epoch);
                if ((rc = got.flush(s->gather_lanes[l], "scatter wait"))) return rc;
            }
            int n_sent = 0;
            for (int i = 1; i < world; ++i) {
                const int dst = (rank + i) % world;
                if (dst == 0) continue;
                const int lane = n_sent % ng;
                if ((rc = send_cols(dst, sub[2 * rank], sub[2 * rank + 1], s->gather_lanes[lane]))) return rc;
                landed[lane].write(s->flag_peers[dst], word_gath(p, rank), s->epoch);
                ++n_sent;
            }
            for (int lane = 0; lane < ng; ++lane)
                if ((rc = landed[lane].flush(s->gather_lanes[lane], "all-gather flags"))) return rc;
            // arrival of panel p on this rank: my own sub-block (scatter) and everybody else's
            MemOps here;
            here.wait(s->flags_local, word_scat(p), s->epoch);
            for (int g = 1; g < world; ++g)
                if (g != rank) here.wait(s->flags_local, word_gath(p, g), s->epoch);
            if (gates) {
                MemOps gate = here;
                gate.write(s->gate_words, 4u * static_cast<size_t>(p), 1u);
                if ((rc = gate.flush(s->gather, "panel gate"))) return rc;
            }
            arrived.ops.insert(arrived.ops.end(), here.ops.begin(), here.ops.end());
        }
    }
    return arrived.flush(compute, "panel waits");
}

int enable_peer(int my_device, const void* ptr) {
    cudaPointerAttributes at;
    B200_CUDA_TRY(cudaPointerGetAttributes(&at, ptr));
    if (at.type != cudaMemoryTypeDevice) return fail(B200_INVALID_ARG, "sharded attach: not a device pointer");
    if (at.device == my_device) return B200_OK;
    int can = 0;
    B200_CUDA_TRY(cudaDeviceCanAccessPeer(&can, my_device, at.device));
    if (!can) return fail(B200_UNSUPPORTED, "sharded attach: no peer access between the two devices");
    cudaError_t e = cudaDeviceEnablePeerAccess(at.device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
    cudaGetLastError();
    return B200_OK;
}

}  // namespace

extern "C" {

int b200_sharded_layout(int world, int64_t N, int64_t K, int panels, int64_t* slab_bounds, int64_t* panel_bounds,
                        int* n_panels, int* group_bounds, int* n_groups, int64_t* sub_cols) {
    ShardLayout L;
    int rc = make_layout(world, N, K, panels, 1, &L);
    if (rc) return rc;
    if (slab_bounds) std::copy(L.slab.begin(), L.slab.end(), slab_bounds);
    if (panel_bounds) std::copy(L.panel.begin(), L.panel.end(), panel_bounds);
    if (n_panels) *n_panels = L.panels();
    if (group_bounds) std::copy(L.group.begin(), L.group.end(), group_bounds);
    if (n_groups) *n_groups = L.groups();
    if (sub_cols) std::copy(L.sub.begin(), L.sub.end(), sub_cols);
    return B200_OK;
}

int b200_sharded_create(b200_sharded** out, b200_handle* h, int rank, int world, int64_t M, int64_t N, int64_t K,
                        int panels) {
    if (!out) return fail(B200_INVALID_ARG, "sharded_create: out is null");
    *out = nullptr;
    if (!h) return fail(B200_INVALID_ARG, "sharded_create: null handle");
    if (world < 1 || world > B200_SHARDED_MAX_RANKS || rank < 0 || rank >= world)
        return fail(B200_INVALID_ARG, "sharded_create: bad rank / world");
    if (M <= 0 || N < 0 || K <= 0) return fail(B200_INVALID_ARG, "sharded_create: M and K must be positive, N >= 0");
    if (M % 8) return fail(B200_INVALID_ARG, "sharded_create: M must be a multiple of 8 (16-byte columns of A)");
    int rc;
    if ((rc = check_current_device(h))) return rc;
    b200_sharded* s = new b200_sharded();
    s->h = h;
    s->rank = rank;
    s->world = world;
    s->M = M;
    s->N = N;
    s->K = K;
    s->panels_requested = panels;
    if ((rc = make_layout(world, N, K, panels, 1, &s->lay))) {
        delete s;
        return rc;
    }
    auto bail = [&](int code) {
        b200_sharded_destroy(s);
        return code;
    };
    // The driver loads a kernel when it is first launched, and loading may wait for everything the
    // context has in flight.  A product enqueues stream-level waits for peers BEFORE its first launch:
    // a first launch that had to load its kernel would then wait for the peers on the host -- for good
    // when the peers are ranks of this very thread.  So every kernel a product can launch is loaded here.
    if ((rc = gemm_tcgen05_preload()) || (rc = gemm_simple_preload())) return bail(rc);
    cudaError_t e;
    if ((e = cudaMalloc(&s->a_local, static_cast<size_t>(2) * M * K)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: A"));
    s->a_peers.assign(world, nullptr);
    s->flag_peers.assign(world, nullptr);
    s->ipc_mapped.assign(world, 0);
    s->a_peers[rank] = s->a_local;
    if (world > 1) {
        if ((e = cudaMalloc(&s->flags_local, B200_SHARDED_FLAG_BYTES)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: flags"));
        if ((e = cudaMalloc(reinterpret_cast<void**>(&s->gate_words), 4 * B200_SHARDED_MAX_PANELS)) != cudaSuccess)
            return bail(cuda_fail(e, "sharded_create: gate words"));
        // cleared and complete before this call returns, i.e. before any peer can learn the address
        if ((e = cudaMemset(s->flags_local, 0, B200_SHARDED_FLAG_BYTES)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: clear flags"));
        if ((e = cudaMemset(s->gate_words, 0, 4 * B200_SHARDED_MAX_PANELS)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: clear gates"));

        if ((e = cudaDeviceSynchronize()) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: sync"));
        s->flag_peers[rank] = s->flags_local;
        if ((e = cudaStreamCreateWithFlags(&s->scatter, cudaStreamNonBlocking)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: stream"));
        if ((e = cudaStreamCreateWithFlags(&s->gather, cudaStreamNonBlocking)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: stream"));
        s->scatter_lanes.assign(1, s->scatter);
        s->gather_lanes.assign(1, s->gather);
        if ((e = cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming)) != cudaSuccess) return bail(cuda_fail(e, "sharded_create: event"));
    } else {
        s->attached = true;
    }
    *out = s;
    return B200_OK;
}

int b200_sharded_destroy(b200_sharded* s) {
    if (!s) return B200_OK;
    cudaSetDevice(s->h->device);
    for (int g = 0; g < static_cast<int>(s->ipc_mapped.size()); ++g) {
        if (!s->ipc_mapped[g]) continue;
        if (s->a_peers[g]) cudaIpcCloseMemHandle(s->a_peers[g]);
        if (s->flag_peers[g]) cudaIpcCloseMemHandle(s->flag_peers[g]);
    }
    for (size_t i = 1; i < s->scatter_lanes.size(); ++i) cudaStreamDestroy(s->scatter_lanes[i]);
    for (size_t i = 1; i < s->gather_lanes.size(); ++i) cudaStreamDestroy(s->gather_lanes[i]);
    if (s->scatter) cudaStreamDestroy(s->scatter);
    if (s->gather) cudaStreamDestroy(s->gather);
    if (s->rescue) cudaStreamDestroy(s->rescue);
    if (s->fork) cudaEventDestroy(s->fork);
    if (s->a_local) cudaFree(s->a_local);
    if (s->flags_local) cudaFree(s->flags_local);
    if (s->gate_words) cudaFree(s->gate_words);
    cudaGetLastError();
    delete s;
    return B200_OK;
}

int b200_sharded_info(b200_sharded* s, int64_t* n0, int64_t* n1, void** a, void** flags, int* n_panels, int* n_groups) {
    if (!s) return fail(B200_INVALID_ARG, "sharded_info: null object");
    if (n0) *n0 = s->lay.slab[s->rank];
    if (n1) *n1 = s->lay.slab[s->rank + 1];
    if (a) *a = s->a_local;
    if (flags) *flags = s->flags_local;
    if (n_panels) *n_panels = s->lay.panels();
    if (n_groups) *n_groups = s->lay.groups();
    return B200_OK;
}

int b200_sharded_ipc_blob(b200_sharded* s, void* blob128) {
    if (!s || !blob128) return fail(B200_INVALID_ARG, "sharded_ipc_blob: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64 && B200_SHARDED_BLOB_BYTES == 128, "two CUDA IPC handles");
    std::memset(blob128, 0, B200_SHARDED_BLOB_BYTES);
    if (s->world == 1) return B200_OK;
    cudaIpcMemHandle_t ha, hf;
    B200_CUDA_TRY(cudaIpcGetMemHandle(&ha, s->a_local));
    B200_CUDA_TRY(cudaIpcGetMemHandle(&hf, s->flags_local));
    std::memcpy(blob128, &ha, 64);
    std::memcpy(static_cast<char*>(blob128) + 64, &hf, 64);
    return B200_OK;
}

int b200_sharded_attach(b200_sharded* s, const void* blobs) {
    if (!s || !blobs) return fail(B200_INVALID_ARG, "sharded_attach: null argument");
    if (s->attached) return fail(B200_INVALID_ARG, "sharded_attach: peers are attached already");
    int rc;
    if ((rc = check_current_device(s->h))) return rc;
    for (int g = 0; g < s->world; ++g) {
        if (g == s->rank) continue;
        cudaIpcMemHandle_t ha, hf;
        std::memcpy(&ha, static_cast<const char*>(blobs) + static_cast<size_t>(g) * B200_SHARDED_BLOB_BYTES, 64);
        std::memcpy(&hf, static_cast<const char*>(blobs) + static_cast<size_t>(g) * B200_SHARDED_BLOB_BYTES + 64, 64);
        s->ipc_mapped[g] = 1;
        B200_CUDA_TRY(cudaIpcOpenMemHandle(&s->a_peers[g], ha, cudaIpcMemLazyEnablePeerAccess));
        B200_CUDA_TRY(cudaIpcOpenMemHandle(&s->flag_peers[g], hf, cudaIpcMemLazyEnablePeerAccess));
    }
    s->attached = true;
    return B200_OK;
}

int b200_sharded_attach_local(b200_sharded* s, void* const* a_ptrs, void* const* flag_ptrs) {
    if (!s || !a_ptrs || !flag_ptrs) return fail(B200_INVALID_ARG, "sharded_attach_local: null argument");
    if (s->attached) return fail(B200_INVALID_ARG, "sharded_attach_local: peers are attached already");
    int rc;
    if ((rc = check_current_device(s->h))) return rc;
    for (int g = 0; g < s->world; ++g) {
        if (g == s->rank) continue;
        if (!a_ptrs[g] || !flag_ptrs[g]) return fail(B200_INVALID_ARG, "sharded_attach_local: null peer pointer");
        if ((rc = enable_peer(s->h->device, a_ptrs[g]))) return rc;
        s->a_peers[g] = a_ptrs[g];
        s->flag_peers[g] = flag_ptrs[g];
    }
    s->attached = true;
    return B200_OK;
}

int b200_sharded_run(b200_sharded* s, b200_stream stream, float alpha, const void* B_slab, int64_t ldb, float beta,
                     const float* C_slab, int64_t ldc, float* D_slab, int64_t ldd, int flags) {
    if (!s) return fail(B200_INVALID_ARG, "sharded_run: null object");
    if (!s->attached) return fail(B200_INVALID_ARG, "sharded_run: peers are not attached yet (b200_sharded_attach)");
    if (s->poisoned)
        return fail(B200_PEER_TIMEOUT, "sharded_run: an earlier product timed out waiting for a peer; destroy the object on every rank");
    if (flags & ~(B200_SHARDED_GATED | B200_SHARDED_NO_TRANSFER | B200_SHARDED_NO_COMPUTE)) return fail(B200_INVALID_ARG, "sharded_run: unknown flag");
    int rc;
    if ((rc = check_current_device(s->h))) return rc;
    b200_handle* h = s->h;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    // transfer only: the slab is treated as empty, the copies, flags and waits are all there
    const int64_t ns = (flags & B200_SHARDED_NO_COMPUTE) ? 0 : s->lay.slab[s->rank + 1] - s->lay.slab[s->rank];
    const int64_t M = s->M, K = s->K;
    const bool transfer = s->world > 1 && !(flags & B200_SHARDED_NO_TRANSFER);
    const bool gated = transfer && (flags & B200_SHARDED_GATED);
    // everything that could make a launch fail is looked at BEFORE the first copy or flag is enqueued: a rank
    // that gave up half-way would leave its peers waiting for words it never writes
    if (ns > 0 && (!B_slab || !D_slab || (beta != 0.0f && !C_slab))) return fail(B200_INVALID_ARG, "sharded_run: null slab pointer");
    if (ns > 0 && (ldb < K || ldd < M || (beta != 0.0f && ldc < M)))
        return fail(B200_INVALID_ARG, "sharded_run: leading dimension smaller than the rows of the slab (ldb >= K, ldc and ldd >= M)");
    const __half* a = static_cast<const __half*>(s->a_local);
    const __half* b = static_cast<const __half*>(B_slab);
    if (transfer) {
        // the transfer streams start behind whatever the caller enqueued before this call (rank 0's A)
        ++s->epoch;
        B200_CUDA_TRY(cudaEventRecord(s->fork, cs));
        for (cudaStream_t st : s->scatter_lanes) B200_CUDA_TRY(cudaStreamWaitEvent(st, s->fork, 0));
        for (cudaStream_t st : s->gather_lanes) B200_CUDA_TRY(cudaStreamWaitEvent(st, s->fork, 0));
        if ((rc = p2p_begin(s, cs))) return rc;
        s->last_compute = cs;
        s->in_flight = true;
    }
    // the caller's options stay untouched: launches made here always take the TMA kernel's own plan
    const int saved_split = h->split_k;
    h->split_k = 1;
    struct Restore {
        b200_handle* h;
        int split;
        ~Restore() { h->split_k = split; }
    } restore{h, saved_split};
    if (gated) {
        // ONE launch whose TMA producer waits for per-panel gate words itself; the transfers are enqueued
        // behind the launch so that the waits they put on this stream follow it
        B200_CUDA_TRY(cudaMemsetAsync(s->gate_words, s->rank == 0 ? 1 : 0, 4 * B200_SHARDED_MAX_PANELS, cs));
        B200_CUDA_TRY(cudaEventRecord(s->fork, cs));
        B200_CUDA_TRY(cudaStreamWaitEvent(s->gather, s->fork, 0));
        if (ns > 0) {
            if ((rc = b200_gemm_f16f32_gated(h, cs, 0, 0, M, ns, K, alpha, a, M, b, ldb, beta, C_slab, ldc, D_slab, ldd,
                                             s->gate_words, s->lay.panel_k)))
                return rc;
        }
        return p2p_exchange(s, 0, s->lay.panels(), cs, true);
    }
    for (int i = 0; i < s->lay.groups(); ++i) {
        const int p0 = s->lay.group[i], p1 = s->lay.group[i + 1];
        if (transfer && (rc = p2p_exchange(s, p0, p1, cs, false))) return rc;  // this group's copies, then the waits for them
        if (ns <= 0) continue;
        const int64_t k0 = s->lay.panel[p0], k1 = s->lay.panel[p1];
        GemmProblem g{0, 0, M, ns, k1 - k0, alpha, i == 0 ? beta : 1.0f, a + k0 * M, M, b + k0, ldb,
                      i == 0 ? C_slab : D_slab, i == 0 ? ldc : ldd, D_slab, ldd};
        if ((rc = gemm_dispatch(h, cs, g))) return rc;
    }
    return B200_OK;
}

int b200_sharded_set_option(b200_sharded* s, int option, int64_t value) {
    if (!s) return fail(B200_INVALID_ARG, "sharded_set_option: null object");
    if (s->in_flight) return fail(B200_INVALID_ARG, "sharded_set_option: a product is in flight (b200_sharded_wait first)");
    int rc;
    if ((rc = check_current_device(s->h))) return rc;
    auto grow = [&](std::vector<cudaStream_t>& lanes, int64_t n) -> int {
        if (s->world == 1) return B200_OK;
        while (static_cast<int64_t>(lanes.size()) < n) {
            cudaStream_t st = nullptr;
            B200_CUDA_TRY(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
            lanes.push_back(st);
        }
        while (static_cast<int64_t>(lanes.size()) > n) {
            B200_CUDA_TRY(cudaStreamDestroy(lanes.back()));
            lanes.pop_back();
        }
        return B200_OK;
    };
    switch (option) {
        case B200_SHARDED_OPT_SCATTER_LANES:
            if (value < 1 || value > 8) return fail(B200_INVALID_ARG, "scatter lanes must be in [1, 8]");
            return grow(s->scatter_lanes, value);
        case B200_SHARDED_OPT_GATHER_LANES:
            if (value < 1 || value > 8) return fail(B200_INVALID_ARG, "gather lanes must be in [1, 8]");
            return grow(s->gather_lanes, value);
        case B200_SHARDED_OPT_FIRST_GROUP: {
            if (value < 1 || value > B200_SHARDED_MAX_PANELS) return fail(B200_INVALID_ARG, "first group must be in [1, 32] panels");
            ShardLayout L;
            if ((rc = make_layout(s->world, s->N, s->K, s->panels_requested, static_cast<int>(value), &L))) return rc;
            if (L.panels() != s->lay.panels()) return fail(B200_INVALID_ARG, "sharded_set_option: layout changed");
            s->lay.group = L.group;
            s->first_group = static_cast<int>(value);
            return B200_OK;
        }
        default:
            return fail(B200_INVALID_ARG, "sharded_set_option: unknown option");
    }
}

int b200_sharded_set_groups(b200_sharded* s, const int* sizes, int n) {
    if (!s || !sizes) return fail(B200_INVALID_ARG, "sharded_set_groups: null argument");
    if (s->in_flight) return fail(B200_INVALID_ARG, "sharded_set_groups: a product is in flight (b200_sharded_wait first)");
    if (n < 1 || n > B200_SHARDED_MAX_PANELS) return fail(B200_INVALID_ARG, "sharded_set_groups: between 1 and 32 launches");
    std::vector<int> bounds(1, 0);
    for (int i = 0; i < n; ++i) {
        if (sizes[i] < 1) return fail(B200_INVALID_ARG, "sharded_set_groups: every launch needs at least one panel");
        bounds.push_back(bounds.back() + sizes[i]);
    }
    if (bounds.back() != s->lay.panels())
        return fail(B200_INVALID_ARG, "sharded_set_groups: the sizes must add up to the " + std::to_string(s->lay.panels()) +
                                          " panels of this object");
    s->lay.group = bounds;
    return B200_OK;
}

int b200_sharded_wait(b200_sharded* s, int64_t timeout_ms) {
    if (!s) return fail(B200_INVALID_ARG, "sharded_wait: null object");
    if (timeout_ms < 1) return fail(B200_INVALID_ARG, "sharded_wait: the timeout must be at least 1 ms");
    int rc;
    if ((rc = check_current_device(s->h))) return rc;
    if (s->poisoned) return fail(B200_PEER_TIMEOUT, "sharded_wait: an earlier product timed out waiting for a peer");
    // (stream, kind): kind 0 = the caller's stream of the last product, 1 = scatter lane, 2 = gather lane
    std::vector<std::pair<cudaStream_t, int>> streams;
    streams.emplace_back(s->last_compute, 0);
    for (cudaStream_t st : s->scatter_lanes) streams.emplace_back(st, 1);
    for (cudaStream_t st : s->gather_lanes) streams.emplace_back(st, 2);
    const auto t0 = std::chrono::steady_clock::now();
    // host-side poll, bounded by the caller's deadline
    bool expired = false, busy = true;
    unsigned busy_mask = 0;
    while (busy && !expired) {
        busy = false;
        busy_mask = 0;
        for (const auto& sk : streams) {
            cudaError_t e = cudaStreamQuery(sk.first);
            if (e == cudaErrorNotReady) {
                busy = true;
                busy_mask |= 1u << sk.second;
            } else if (e != cudaSuccess) {
                return cuda_fail(e, "sharded_wait: cudaStreamQuery");
            }
        }
        if (!busy) break;
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) expired = true;
        else std::this_thread::sleep_for(std::chrono::microseconds(ms < 5 ? 50 : 500));
    }
    if (expired && s->world > 1) {
        // Every wait of this object's streams looks at a word of this rank's own flag block and passes once
        // that word is >= the epoch: raising all of them from here releases the streams.  What they then
        // compute is garbage (A is incomplete); the object is unusable from now on.
        s->poisoned = true;
        using SetFn = CUresult (*)(CUdeviceptr, unsigned int, size_t, CUstream);
        static SetFn set32 = nullptr;
        if (!set32) {
            void* p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuMemsetD32Async", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
                set32 = reinterpret_cast<SetFn>(p);
        }
        if (!set32) return fail(B200_CUDA_ERROR, "cuMemsetD32Async entry point not found");
        if (!s->rescue) B200_CUDA_TRY(cudaStreamCreateWithFlags(&s->rescue, cudaStreamNonBlocking));
        // what this rank has heard so far, for the error text: which peers said "done", how many panels arrived
        std::vector<uint32_t> seen(B200_SHARDED_FLAG_BYTES / 4, 0);
        std::string heard;
        if (cudaMemcpyAsync(seen.data(), s->flags_local, B200_SHARDED_FLAG_BYTES, cudaMemcpyDeviceToHost, s->rescue) == cudaSuccess &&
            cudaStreamSynchronize(s->rescue) == cudaSuccess) {
            heard = "; silent peers:";
            for (int g = 0; g < s->world; ++g)
                if (g != s->rank && seen[word_done(g) / 4] < s->epoch) heard += " " + std::to_string(g);
            int scat = 0;
            for (int p = 0; p < s->lay.panels(); ++p) scat += seen[word_scat(p) / 4] >= s->epoch;
            heard += "; panels scattered to this rank: " + std::to_string(scat) + " of " + std::to_string(s->lay.panels());
        }
        cudaGetLastError();
        heard += std::string("; streams still busy:") + ((busy_mask & 1u) ? " compute" : "") + ((busy_mask & 2u) ? " scatter" : "") +
                 ((busy_mask & 4u) ? " gather" : "");
        CUresult r = set32(reinterpret_cast<CUdeviceptr>(s->flags_local), s->epoch, B200_SHARDED_FLAG_BYTES / 4, s->rescue);
        if (r != CUDA_SUCCESS) return fail(B200_CUDA_ERROR, "cuMemsetD32Async failed (CUresult " + std::to_string(static_cast<int>(r)) + ")");
        // the gated form also polls gate words from inside the kernel (bounded there); open them too
        B200_CUDA_TRY(cudaMemsetAsync(s->gate_words, 1, 4 * B200_SHARDED_MAX_PANELS, s->rescue));
        B200_CUDA_TRY(cudaStreamSynchronize(s->rescue));
        // the released work is finite (copies and GEMM launches with bounded waits): let it drain
        for (const auto& sk : streams) B200_CUDA_TRY(cudaStreamSynchronize(sk.first));
        int word[4];
        read_status(s->h, word);
        s->in_flight = false;
        return fail(B200_PEER_TIMEOUT, "sharded_wait: no word from a peer within " + std::to_string(timeout_ms) +
                                           " ms (epoch " + std::to_string(s->epoch) + ")" + heard + "; the waits were released, D is not valid");
    }
    s->in_flight = false;
    int word[4] = {0, 0, 0, 0};
    if ((rc = read_status(s->h, word))) return rc;
    if (word[0] != 0)
        return fail(B200_DEVICE_TIMEOUT, "sharded gemm: a bounded wait ran out on the device (wait id " + std::to_string(word[0]) +
                                             ", block " + std::to_string(word[1]) + ")");
    return B200_OK;
}

}  // extern "C"
