/*
 * b200wmma.h -- C ABI of libb200wmma.so: the FP16 x FP16 -> FP32 tensor-core GEMM path of
 * CUDAnative.jl's WMMA module, rebuilt for NVIDIA B200 (sm_100a).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int status
 * (0 = B200_OK) and never throws.  Device work is enqueued on the caller's stream and the call
 * returns immediately unless its comment says otherwise; buffers stay owned by the caller.
 * Matrices follow the reference's CuArray convention: dense column-major with a leading
 * dimension in ELEMENTS (src/device/array.jl:104 of the reference, linear column-major
 * indexing); a "row-major" operand is the same memory read as its transpose.
 *
 * Reference citations below are paths inside the CUDAnative.jl source tree.
 */
#ifndef B200WMMA_H
#define B200WMMA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------ */
/* status codes                                                                                */
/* ------------------------------------------------------------------------------------------ */
enum {
    B200_OK = 0,
    B200_INVALID_ARG = 1,    /* bad dims / leading dimension / null or misaligned pointer        */
    B200_UNSUPPORTED = 2,    /* legal request this build has no kernel for                       */
    B200_CUDA_ERROR = 3,     /* a CUDA runtime / driver call failed; text in b200_last_error()   */
    B200_DEVICE_TIMEOUT = 4, /* a bounded wait inside a kernel ran out; see b200_device_status() */
    B200_NO_DEVICE = 5,      /* no CUDA device, or the device is not compute capability 10.x     */
    B200_PEER_TIMEOUT = 6    /* sharded GEMM: a peer's flag write did not arrive within the deadline */
};

/* Layout tags: the reference's WMMA.ColMajor / WMMA.RowMajor (src/device/cuda/wmma.jl:313-338). */
enum { B200_COL_MAJOR = 0, B200_ROW_MAJOR = 1 };

/* Element tags: Float16 / Float32, the two WMMA element types (src/device/cuda/wmma.jl:11-37).
 * B200_BF16 (bfloat16) has no counterpart in the reference; only b200_gemm_ex and
 * b200_gemm_strided_batched accept it. */
enum { B200_F16 = 0, B200_F32 = 1, B200_BF16 = 2 };

/* Fragment use: WMMA.MatrixA / MatrixB / Accumulator (src/device/cuda/wmma.jl:343-346). */
enum { B200_MATRIX_A = 0, B200_MATRIX_B = 1, B200_ACCUMULATOR = 2 };

/* Which instruction family backs the 16x16x16 unit. */
enum {
    B200_LOWER_WARP = 0,   /* warp-level mma.sync.m16n8k16 x2, register fragments               */
    B200_LOWER_TCGEN05 = 1 /* CTA-level tcgen05.mma (M padded to 128), accumulator in TMEM      */
};

/* Kernel selector for b200_set_option(B200_OPT_FORCE_KERNEL). */
enum {
    B200_KERNEL_AUTO = 0,
    B200_KERNEL_TCGEN05 = 1, /* TMA + tcgen05 pipeline; fails with UNSUPPORTED if not eligible   */
    B200_KERNEL_SIMPLE = 2   /* plain shared-memory FP32-FMA kernel (any alignment, any shape)   */
};

enum {
    B200_OPT_FORCE_KERNEL = 0,   /* one of B200_KERNEL_*                                          */
    B200_OPT_MAX_CTAS = 1,       /* cap on the persistent grid (0 = one CTA per SM)               */
    B200_OPT_WAIT_BUDGET_NS = 2, /* budget of every in-kernel barrier wait (default 2e9 ns)       */
    B200_OPT_TILE_N = 3,         /* 0 = auto, else 64 / 128 / 256                                 */
    B200_OPT_SPLIT_K = 4,        /* 0 = auto, 1 = off, n>1 = split the K loop n ways              */
    B200_OPT_CTA_PAIR = 5,       /* 0 = auto, 1 = one-CTA tiles only, 2 = force 2-CTA tiles       */
    B200_OPT_RASTER_GROUP = 6,   /* tile rows per rasterisation group (0 = default)               */
    B200_OPT_F16_ACCUMULATE = 9, /* 1 = b200_gemm_f16_typed with Float16 C AND Float16 D accumulates in     */
                                 /* binary16 on the tensor cores, as WMMA.mma does for Config{16,16,16,    */
                                 /* Float16} with a Float16 accumulator fragment (the .f16.f16 variants,   */
                                 /* src/device/cuda/wmma.jl:222-257).  Default 0: binary32 accumulation,  */
                                 /* Float16 only as the storage type.  tcgen05 kernel only (UNSUPPORTED    */
                                 /* for shapes it cannot take); the split-K option is ignored.            */
    B200_OPT_PDL = 8,            /* 1 (default) = tcgen05 GEMM kernels are launched with programmatic   */
                                 /* stream serialization: their set-up overlaps the tail of the kernel  */
                                 /* before them in the stream; 0 = ordinary launches                    */
    B200_OPT_CHECK_ON_CALL = 7   /* 1 = every GEMM entry point first looks at the status word of the  */
                                 /* handle's previous launch, if that launch has finished, and returns */
                                 /* B200_DEVICE_TIMEOUT when a wait ran out in it: the reference polls */
                                 /* its device exception flag the same way at every API call          */
                                 /* (src/init.jl:37, src/exceptions.jl:76-89).  Default 0.            */
};

typedef struct b200_handle b200_handle;
typedef void* b200_stream; /* a cudaStream_t; NULL = the legacy default stream */

/* ------------------------------------------------------------------------------------------ */
/* library, handle, errors                                                                     */
/* ------------------------------------------------------------------------------------------ */

/* Text of the calling thread's most recent failure ("" if none).  Replaces the CuError /
 * KernelException text the reference surfaces at its next API call (src/exceptions.jl:76-89). */
const char* b200_last_error(void);
const char* b200_status_string(int status);

/* ABI version of this header (major*100 + minor). */
int b200_version(void);

/* Number of CUDA devices with compute capability 10.x; negative status on CUDA failure.
 * Replaces CUDAnative.functional() (src/CUDAnative.jl:29-52) for this path. */
int b200_device_count(void);

/* Create / destroy the per-device handle: device status word, workspace for the host-buffer
 * entry point, split-K scratch.  Binds to the device's primary context and makes `device` the
 * calling thread's current device, as CUDAnative's device!() does (src/init.jl:187-209).  One
 * handle per host thread (or lock externally).  The entry points that take a handle and a stream
 * launch on the calling thread's current device; they return B200_INVALID_ARG when that is not
 * the handle's device. */
int b200_create(b200_handle** out, int device);
int b200_destroy(b200_handle* h);

int b200_set_option(b200_handle* h, int option, int64_t value);
int b200_get_option(b200_handle* h, int option, int64_t* value);

/* After the stream has been synchronised: what the kernels of this handle last wrote into the
 * device status word.  code 0 = nothing; otherwise the id of the wait that ran out, the block
 * it was in and a detail word.  Clears the word.  Plays the role of the reference's polled
 * device exception flag (src/exceptions.jl:55-89, src/device/runtime.jl:18-31). */
int b200_device_status(b200_handle* h, int* code, int* block, int* detail);

/* Launches one warp that waits, with the given budget (1 us .. 1 s), on a barrier nothing ever
 * signals.  After synchronising, b200_device_status() must report wait id 107: the check that a
 * stuck pipeline ends in an error code and a usable context rather than a hang.  The reference's
 * counterpart is its device exception flag test path (src/exceptions.jl:76-89). */
int b200_selftest_bounded_wait(b200_handle* h, b200_stream stream, int64_t budget_ns);

/* Properties of the last GEMM launched through this handle: kernel id (B200_KERNEL_*), tile_n,
 * split_k, CTAs launched, CTAs per tile (1 or 2).  Any out pointer may be NULL. */
int b200_last_launch(b200_handle* h, int* kernel, int* tile_n, int* split_k, int* ctas,
                     int* cta_pair);

/* ------------------------------------------------------------------------------------------ */
/* tiled GEMM: D = alpha * op(A) * op(B) + beta * C                                            */
/* ------------------------------------------------------------------------------------------ */

/* The multi-tile form of WMMA.load_a/load_b/load_c -> WMMA.mma -> WMMA.store_d
 * (src/device/cuda/wmma.jl:507-530, :558-583, :613-632) with the alpha/beta scaling the
 * reference applies by broadcasting over fragments (src/device/cuda/wmma.jl:678-716).
 *
 *   op(A) is M x K, op(B) is K x N, C and D are M x N, all column-major, all DEVICE pointers.
 *   transA = 0: A stored M x K column-major, lda >= M   (WMMA.ColMajor A)
 *   transA = 1: A stored K x M column-major (= M x K row-major), lda >= K (WMMA.RowMajor A)
 *   transB likewise for the K x N operand.
 *   A, B: IEEE binary16.  C, D: binary32.  Products exact, accumulation in binary32,
 *   alpha and beta applied in binary32 in the epilogue.
 *   beta == 0: C is never read and may be NULL (WMMA.fill_c(0) case, wmma.jl:654-667).
 *   D may alias C exactly (same pointer, same ld).  M, N >= 0; K >= 0 (K == 0: D = beta*C).
 *
 * The tcgen05 kernel needs 16-byte aligned pointers and leading dimensions (lda, ldb
 * multiples of 8 elements; ldc, ldd multiples of 4) and M a multiple of 4; with any other M the
 * last M % 4 rows run on the simple kernel, and anything else runs on the simple kernel whole. */
int b200_gemm_f16f32(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M,
                     int64_t N, int64_t K, float alpha, const void* A, int64_t lda, const void* B,
                     int64_t ldb, float beta, const float* C, int64_t ldc, float* D, int64_t ldd);

/* b200_gemm_f16f32 with the element types of C and D chosen per call (B200_F16 or B200_F32): the
 * four accumulator / result type combinations WMMA.Config{16,16,16,d_type} and load_c offer
 * (src/device/cuda/wmma.jl:23-30, :394; all four are swept by test/device/wmma.jl:188-248).
 * Accumulation is binary32 in every case unless B200_OPT_F16_ACCUMULATE is set (then binary16
 * for Float16 C with Float16 D); a binary16 C is widened when it is read and a binary16
 * D is rounded once (to nearest even) when it is written.  ldc / ldd count elements of the
 * respective type.  TMA path: ldc / ldd multiples of 16 bytes, and whole 16-byte chunks of rows
 * (M % 8 for a binary16 D); the remaining rows run on the simple kernel. */
int b200_gemm_f16_typed(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M,
                        int64_t N, int64_t K, float alpha, const void* A, int64_t lda,
                        const void* B, int64_t ldb, float beta, const void* C, int64_t ldc,
                        int c_type, void* D, int64_t ldd, int d_type);

/* The general form of the two entry points above: A and B are both binary16 (ab_type = B200_F16) or
 * both bfloat16 (B200_BF16); C and D are binary32, binary16 or bfloat16 independently.  Products
 * of two bfloat16 values are exact in binary32 as well, accumulation stays binary32, a 16-bit D
 * is rounded once to nearest even.  Leading dimensions count elements of the respective type.
 * No counterpart in the reference beyond the Float16 / Float32 combinations of
 * b200_gemm_f16_typed: bfloat16 is what callers of a tensor-core product expect next to them. */
int b200_gemm_ex(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M, int64_t N,
                 int64_t K, float alpha, const void* A, int64_t lda, const void* B, int64_t ldb,
                 int ab_type, float beta, const void* C, int64_t ldc, int c_type, void* D,
                 int64_t ldd, int d_type);

/* `batch` independent products of one shape in one call:
 *     D_i = alpha * op(A_i) * op(B_i) + beta * C_i,   X_i = X + i * stride_x elements,  i < batch
 * (no counterpart in the reference, which stops at one 16x16x16 tile per warp).  A stride of 0
 * repeats A, B or C for every i; D_i must not overlap (stride_d >= ldd * N).  batch == 0 is a
 * no-op.  One launch runs every tile of every matrix when the strides are multiples of 16 bytes
 * and at least one matrix long (the matrix index is a third TMA coordinate); otherwise the
 * matrices are multiplied one launch each, or all on the simple kernel.  Types as in
 * b200_gemm_ex.  The split-K option is ignored for batches. */
int b200_gemm_strided_batched(b200_handle* h, b200_stream stream, int transA, int transB,
                              int64_t M, int64_t N, int64_t K, float alpha, const void* A,
                              int64_t lda, int64_t stride_a, const void* B, int64_t ldb,
                              int64_t stride_b, int ab_type, float beta, const void* C,
                              int64_t ldc, int64_t stride_c, int c_type, void* D, int64_t ldd,
                              int64_t stride_d, int d_type, int64_t batch);

/* b200_gemm_f16f32 whose main loop may start before all of A is in this GPU's memory: columns
 * [j*panel_k, (j+1)*panel_k) of op(A) are read only once the 32-bit word panel_flags[j] (device
 * memory) is non-zero.  panel_k is a multiple of 64; at most 32 panels.  The words are meant to
 * be written with b200_stream_write_u32 on the stream that moves A (behind the copy of that
 * panel), so that one GEMM launch overlaps the arrival of A over NVLink.  A wait for a panel is
 * bounded like every other wait (wait id 108).  No counterpart in the reference (single GPU
 * only, src/init.jl:187-209). */
int b200_gemm_f16f32_gated(b200_handle* h, b200_stream stream, int transA, int transB, int64_t M,
                           int64_t N, int64_t K, float alpha, const void* A, int64_t lda,
                           const void* B, int64_t ldb, float beta, const float* C, int64_t ldc,
                           float* D, int64_t ldd, const uint32_t* panel_flags, int64_t panel_k);

/* Stream-ordered 32-bit store to device memory (cuStreamWriteValue32): runs without an SM, so it
 * can signal a kernel that already occupies the whole GPU. */
int b200_stream_write_u32(b200_stream stream, void* dptr, uint32_t value);

/* Stream-ordered wait (cuStreamWaitValue32, compare >=): work enqueued on `stream` after this
 * call starts only once the 32-bit word at dptr is >= value.  Together with
 * b200_stream_write_u32 on a peer-mapped address this orders two GPUs' streams without any
 * kernel.  The wait has no timeout: only wait for words whose writer is already enqueued. */
int b200_stream_wait_u32(b200_stream stream, void* dptr, uint32_t value);

/* Same operation with HOST pointers (ideally page-locked): copies A, B and (beta != 0) C to the
 * handle's device workspace, runs the GEMM, copies D back and synchronises before returning.
 * This is the Array -> CuArray -> kernel -> Array(d_dev) round trip of the reference's examples
 * (examples/wmma/high-level.jl:21-47) as one call.  Allocates workspace on first use. */
int b200_gemm_f16f32_host(b200_handle* h, int transA, int transB, int64_t M, int64_t N, int64_t K,
                          float alpha, const void* A, int64_t lda, const void* B, int64_t ldb,
                          float beta, const float* C, int64_t ldc, float* D, int64_t ldd);

/* The same product for callers that cannot allocate device memory when they need it (inside an
 * allocator callback, in a loop that promised "no driver allocations after start-up", in a host
 * that owns every byte of device memory).  No counterpart in the reference, which allocates
 * freely through CUDAdrv.  Needs no handle and calls no cudaMalloc / cudaFree: the K loop is cut
 * into `split_k` slices (2..64) whose FP32 partial products, and the device status word, live in
 * a 16 MiB + 256 B array that is part of the library image on every GPU that loads it.
 *   - The partials take roundup(M,4) * roundup(N, tile width) * slices * 4 bytes; a problem that
 *     needs more than 16 MiB is refused with B200_INVALID_ARG (text in b200_last_error()).
 *   - Same alignment rules as the TMA path of b200_gemm_f16f32; there is no fallback kernel.
 *   - The first call on a device looks the array's address up; make it outside stream capture.
 *   - All calls on a device share the array: calls that overlap on the GPU race.  Serialise them.
 *   - sync_and_check != 0: synchronise the stream and return B200_DEVICE_TIMEOUT if a bounded
 *     wait ran out; 0: return as soon as the work is enqueued (then ask b200_static_status).
 *   - The first launch of each kernel variant makes the driver load it, which allocates: call
 *     b200_static_warmup at start-up if even that must not happen later. */
int b200_gemm_f16f32_splitk_static(b200_stream stream, int transA, int transB, int64_t M,
                                   int64_t N, int64_t K, float alpha, const void* A, int64_t lda,
                                   const void* B, int64_t ldb, float beta, const float* C,
                                   int64_t ldc, float* D, int64_t ldd, int split_k,
                                   int sync_and_check);

/* Companions of b200_gemm_f16f32_splitk_static; like it they have no counterpart in the reference
 * and call no cudaMalloc / cudaFree.
 *
 * b200_static_warmup: once per device at start-up, outside stream capture.  Looks the static
 *   array's address up and makes the driver load every kernel variant the static entry point can
 *   pick (loading a kernel for its first launch is the one thing that would still allocate later).
 * b200_static_status: the device status word of the static entry point on the current device:
 *   code 0 = nothing, else the id of the wait that ran out, its block and a detail word; clears
 *   the word.  A caller that passes sync_and_check = 0 calls this after it has synchronised, and
 *   before results are used; the word keeps the first failure until somebody reads it.
 * b200_static_selftest_bounded_wait: one warp waits with the given budget (1 us .. 1 s) on a
 *   barrier nothing signals and reports into the static status word (wait id 107). */
int b200_static_warmup(void);
int b200_static_status(int* code, int* block, int* detail);
int b200_static_selftest_bounded_wait(b200_stream stream, int64_t budget_ns);

/* ------------------------------------------------------------------------------------------ */
/* the 16x16x16 unit: one WMMA multiply-accumulate                                             */
/* ------------------------------------------------------------------------------------------ */

/* The whole body of the reference's example kernels (examples/wmma/high-level.jl:30-44,
 * examples/wmma/low-level.jl:33-42) and of its high-level API test
 * (test/device/wmma.jl:188-248) as one launch:
 *     a = load_a(A); b = load_b(B); c = mac ? load_c(C) : fill_c(0)
 *     a = alpha .* a   (rounded to Float16, as the fragment is Float16)
 *     c = beta  .* c   (in C's element type)
 *     d = mma(a, b, c); store_d(D, d)
 * A, B: 16x16 binary16 with the given layouts and leading dimensions; C / D: binary16 or
 * binary32.  `lowering` is B200_LOWER_WARP or B200_LOWER_TCGEN05.  use_alpha / use_beta = 0
 * skip the corresponding broadcast entirely.  The tcgen05 lowering synchronises the stream
 * before it returns, so that a bounded wait that ran out comes back as B200_DEVICE_TIMEOUT. */
int b200_wmma_16x16x16(b200_stream stream, int lowering, int a_layout, int b_layout, int c_layout,
                       int d_layout, int c_type, int d_type, int mac, int use_alpha, float alpha,
                       int use_beta, float beta, const void* A, int64_t lda, const void* B,
                       int64_t ldb, const void* C, int64_t ldc, void* D, int64_t ldd);

/* Fragment-granular forms.  A fragment is the per-lane register image of one warp, kept in
 * device memory as 32 lanes x FS elements (FS = 16 for A/B, 8 for C/D: src/device/cuda/wmma.jl:
 * 413-420).  Which matrix element sits in which lane slot is private to this library, as the
 * reference leaves it unspecified (docs/src/device/wmma.md:47-49).
 *
 * b200_wmma_load  : WMMA.load_a / load_b / load_c   (wmma.jl:507-530); use = B200_MATRIX_*.
 * b200_wmma_fill_c: WMMA.fill_c                      (wmma.jl:654-667)
 * b200_wmma_bcast : `s .* frag` / `s .+ frag`        (wmma.jl:678-716); op 0 = mul, 1 = add;
 *                   computed in the fragment's element type.
 * b200_wmma_mma   : WMMA.mma                         (wmma.jl:558-583)
 * b200_wmma_store_d: WMMA.store_d                    (wmma.jl:613-632) */
int b200_wmma_load(b200_stream stream, int use, int layout, int elem_type, const void* addr,
                   int64_t stride, void* frag);
int b200_wmma_fill_c(b200_stream stream, int elem_type, float value, void* frag);
int b200_wmma_bcast(b200_stream stream, int op, int elem_type, int frag_size, float scalar,
                    const void* frag_in, void* frag_out);
int b200_wmma_mma(b200_stream stream, int c_type, int d_type, const void* a_frag,
                  const void* b_frag, const void* c_frag, void* d_frag);
int b200_wmma_store_d(b200_stream stream, int layout, int elem_type, void* addr, const void* frag,
                      int64_t stride);

/* ------------------------------------------------------------------------------------------ */
/* device memory and synthetic inputs                                                          */
/* ------------------------------------------------------------------------------------------ */

/* What CUDAnative.CuHostArray does around a kernel (src/array.jl:20-60): allocate, upload,
 * download, free.  b200_host_alloc returns page-locked host memory. */
int b200_malloc(void** dptr, size_t bytes);
int b200_free(void* dptr);
int b200_host_alloc(void** hptr, size_t bytes);
int b200_host_free(void* hptr);
int b200_memcpy_h2d(void* dst, const void* src, size_t bytes, b200_stream stream);
int b200_memcpy_d2h(void* dst, const void* src, size_t bytes, b200_stream stream);
int b200_memset(void* dst, int byte, size_t bytes, b200_stream stream);
int b200_stream_sync(b200_stream stream);
/* A new stream that does not synchronise with the legacy default stream (CUDAdrv's CuStream(),
 * which the reference's `stream` launch keyword takes: src/execution.jl:158-166). */
int b200_stream_create(b200_stream* out);
int b200_stream_destroy(b200_stream stream);

/* Peer access for the N-sharded multi-GPU GEMM, one process per GPU (no counterpart in the
 * reference, whose only multi-device facility is picking a device per task: src/init.jl:187-209).
 * b200_ipc_get_handle writes the 64-byte CUDA IPC handle of a b200_malloc'ed buffer;
 * b200_ipc_open_handle maps another process's buffer into this one (peer access is enabled on
 * demand) and b200_ipc_close_handle unmaps it.  b200_memcpy_d2d copies between any two device
 * addresses, local or mapped, on a stream; between GPUs it runs on the copy engines over NVLink
 * and takes no SM away from a GEMM that is running. */
int b200_ipc_get_handle(void* dptr, void* handle64);
int b200_ipc_open_handle(const void* handle64, void** dptr);
int b200_ipc_close_handle(void* dptr);
int b200_memcpy_d2d(void* dst, const void* src, size_t bytes, b200_stream stream);

/* ------------------------------------------------------------------------------------------ */
/* N-sharded multi-GPU GEMM, one object per rank                                               */
/* ------------------------------------------------------------------------------------------ */

/*     D[:, slab_r] = alpha * A * B[:, slab_r] + beta * C[:, slab_r]        on every rank r
 *
 * No counterpart in the reference, which computes on one device per task (src/init.jl:187-209).
 * What is kept from it: raw device pointers that the caller owns, the way a CuArray converts for
 * ccall (src/array.jl:15); asynchronous enqueue on the caller's stream (src/execution.jl:158-166);
 * one process (or task) per device.
 *
 * B, C and D are split into contiguous column slabs (whole 256-column tiles per rank) that never
 * move.  A (M x K, column-major, lda = M, binary16) lives in a buffer the object owns on every
 * rank; before a product its contents are valid on rank 0 only, afterwards everywhere.  It
 * travels in K panels over NVLink on the copy engines (scatter from rank 0, then all-gather
 * among the receivers), ordered by stream memory operations on flag words; the GEMM runs as a
 * few launches over growing K ranges, each behind the arrival of its own panels only.
 *
 * Life cycle, on every rank, in this order:
 *   b200_sharded_create     allocates A and the flag block on the handle's device
 *   b200_sharded_ipc_blob   128 bytes that let another process map both
 *   (the caller moves every rank's blob to every rank: MPI, files, sockets, torch.distributed)
 *   b200_sharded_attach     maps the peers' buffers; `blobs` = world x 128 bytes, entry r from rank r
 *     or b200_sharded_attach_local for peers that live in THIS process (one process driving
 *     several devices): entry r = rank r's A and flag block as b200_sharded_info returns them
 *   b200_sharded_run        once per product; every rank must make the same sequence of calls
 *   b200_sharded_wait       host-side wait with a deadline (optional; see below)
 *   b200_sharded_destroy    after every rank has synchronised its last product
 */
typedef struct b200_sharded b200_sharded;

#define B200_SHARDED_MAX_RANKS 64
#define B200_SHARDED_MAX_PANELS 32
#define B200_SHARDED_BLOB_BYTES 128
#define B200_SHARDED_FLAG_BYTES (4 * (128 + 32 * 64))

/* flags of b200_sharded_run */
enum {
    B200_SHARDED_GATED = 1,       /* ONE launch of the gated GEMM (b200_gemm_f16f32_gated) instead of a
                                     few launches: overlaps transfer and main loop inside the kernel  */
    B200_SHARDED_NO_TRANSFER = 2, /* A is already valid on this rank: the same launches without any copy
                                     or wait (the compute-only time of a product)                     */
    B200_SHARDED_NO_COMPUTE = 4   /* the transfer alone: every copy, flag and wait, no GEMM launch (the
                                     transfer-only time of a product; D is not touched)               */
};

/* options of b200_sharded_set_option; set them on every rank alike, between products */
enum {
    B200_SHARDED_OPT_SCATTER_LANES = 0, /* streams rank 0 spreads its copies to different receivers over   */
    B200_SHARDED_OPT_GATHER_LANES = 1,  /* streams every other rank spreads its forwarding copies over     */
    B200_SHARDED_OPT_FIRST_GROUP = 2    /* panels in the first GEMM launch (later launches grow by 1.4x up  */
                                        /* to a quarter of the panels; see b200_sharded_set_groups)         */
};

int b200_sharded_create(b200_sharded** out, b200_handle* h, int rank, int world, int64_t M, int64_t N,
                        int64_t K, int panels);
int b200_sharded_destroy(b200_sharded* s);
int b200_sharded_set_option(b200_sharded* s, int option, int64_t value);
/* The GEMM launches of a product as panel counts: launch i multiplies the next sizes[i] panels of A and
 * starts once they have arrived.  The sizes must add up to the object's panel count (b200_sharded_info).
 * Same on every rank, between products. */
int b200_sharded_set_groups(b200_sharded* s, const int* sizes, int n);

/* This rank's column slab [n0, n1) of B / C / D, its A buffer (M * K binary16) and flag block, and
 * how many transfer panels and GEMM launches a product takes.  Any out pointer may be NULL. */
int b200_sharded_info(b200_sharded* s, int64_t* n0, int64_t* n1, void** a, void** flags, int* n_panels,
                      int* n_groups);
int b200_sharded_ipc_blob(b200_sharded* s, void* blob128);
int b200_sharded_attach(b200_sharded* s, const void* blobs);
int b200_sharded_attach_local(b200_sharded* s, void* const* a_ptrs, void* const* flag_ptrs);

/* Enqueue one product on `stream`.  B_slab: K x (n1-n0), C_slab / D_slab: M x (n1-n0), column-major
 * device pointers with their leading dimensions; D_slab may alias C_slab.  A rank whose slab is
 * empty still makes the call (it takes part in the transfer).  Returns as soon as the work is
 * enqueued; a wait that ran out inside a kernel shows in b200_device_status / b200_sharded_wait. */
int b200_sharded_run(b200_sharded* s, b200_stream stream, float alpha, const void* B_slab, int64_t ldb,
                     float beta, const float* C_slab, int64_t ldc, float* D_slab, int64_t ldd, int flags);

/* Wait on the host until the last product's work on this rank has finished, for at most
 * timeout_ms.  The stream-level waits of the transfer have no timeout of their own: a peer that
 * skipped the call or died would leave this rank's streams blocked for good.  On expiry this call
 * therefore raises every flag word of this rank's own flag block itself (all stream waits look
 * only at that block), lets the released work drain, marks the object unusable and returns
 * B200_PEER_TIMEOUT; D is not valid then.  Otherwise B200_OK, or B200_DEVICE_TIMEOUT when a
 * bounded wait ran out inside a kernel.  Plays the role of the reference's synchronize() plus its
 * exception poll (src/exceptions.jl:76-89). */
int b200_sharded_wait(b200_sharded* s, int64_t timeout_ms);

/* The layout arithmetic of the above as a pure host function (no CUDA call): slab bounds
 * (world + 1), panel bounds (*n_panels + 1), GEMM launch groups as panel bounds (*n_groups + 1) and,
 * for every panel p and rank g, the columns [c0, c1) of A that rank g forwards:
 * sub_cols[(p * world + g) * 2 + {0, 1}].  Arrays must hold B200_SHARDED_MAX_RANKS + 1,
 * B200_SHARDED_MAX_PANELS + 1, B200_SHARDED_MAX_PANELS + 1 and 2 * world * B200_SHARDED_MAX_PANELS
 * entries; any may be NULL. */
int b200_sharded_layout(int world, int64_t N, int64_t K, int panels, int64_t* slab_bounds,
                        int64_t* panel_bounds, int* n_panels, int* group_bounds, int* n_groups,
                        int64_t* sub_cols);

/* Counter-based synthetic matrices (no counterpart in the reference, whose tests draw from
 * Julia's unseeded rand; test/device/wmma.jl:196-199).  Element (i, j) of a rows x cols
 * column-major matrix gets
 *     u = splitmix64(seed * 0x9E3779B97F4A7C15 + matrix_id * 0xD1B54A32D192ED03 + index0 + (j*rows + i))
 * (index0 = linear index of this window's first element inside a larger synthetic matrix of the
 * same height: col0 * rows for a slab that starts at column col0, 0 for a whole matrix)
 * dist 0: uniform[-1,1) = (u >> 40) * 2^-23 - 1
 * dist 1: normal(0,1) by Box-Muller on the two 24-bit halves of u's top 48 bits
 * dist 2: zeros
 * times `scale`, then (f16 / bf16 variants) rounded to nearest-even binary16 / bfloat16. */
int b200_fill_f16(b200_stream stream, void* dptr, int64_t rows, int64_t cols, int64_t ld,
                  uint64_t seed, uint64_t matrix_id, uint64_t index0, int dist, float scale);
int b200_fill_bf16(b200_stream stream, void* dptr, int64_t rows, int64_t cols, int64_t ld,
                   uint64_t seed, uint64_t matrix_id, uint64_t index0, int dist, float scale);
int b200_fill_f32(b200_stream stream, float* dptr, int64_t rows, int64_t cols, int64_t ld,
                  uint64_t seed, uint64_t matrix_id, uint64_t index0, int dist, float scale);

#ifdef __cplusplus
}
#endif
#endif /* B200WMMA_H */
