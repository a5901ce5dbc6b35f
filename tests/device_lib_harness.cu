// Test harness for the linkable device-side fragment library (csrc/wmma_device_lib.cu): a one-warp
// kernel with the body of the reference's low-level example (examples/wmma/low-level.jl:33-42 of
// CUDAnative.jl) -- load a, b, c; mma; store d -- calling the library's `extern "C" __device__`
// functions by name through the same relocatable-device-code link a Julia kernel would use.
// Every one of the 52 functions is reachable through the selectors.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" {
struct b200_frag_ab { uint32_t x[8]; };
struct b200_frag_h { uint32_t x[4]; };
struct b200_frag_f { float x[8]; };

#define DECL_LOAD_AB(mat, lay, sfx) __device__ b200_frag_ab b200_wmma_load_##mat##_##lay##_m16n16k16##sfx##_stride_f16(const void*, int);
#define DECL_LOAD_C(lay, sfx)                                                                         \
    __device__ b200_frag_h b200_wmma_load_c_##lay##_m16n16k16##sfx##_stride_f16(const void*, int);    \
    __device__ b200_frag_f b200_wmma_load_c_##lay##_m16n16k16##sfx##_stride_f32(const void*, int);
#define DECL_STORE(lay, sfx)                                                                          \
    __device__ void b200_wmma_store_d_##lay##_m16n16k16##sfx##_stride_f16(void*, b200_frag_h, int);   \
    __device__ void b200_wmma_store_d_##lay##_m16n16k16##sfx##_stride_f32(void*, b200_frag_f, int);
#define DECL_MMA(al, bl)                                                                                              \
    __device__ b200_frag_h b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f16(b200_frag_ab, b200_frag_ab, b200_frag_h);    \
    __device__ b200_frag_h b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f32(b200_frag_ab, b200_frag_ab, b200_frag_f);    \
    __device__ b200_frag_f b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f16(b200_frag_ab, b200_frag_ab, b200_frag_h);    \
    __device__ b200_frag_f b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f32(b200_frag_ab, b200_frag_ab, b200_frag_f);
#define FOR_AS(M, ...) M(__VA_ARGS__, ) M(__VA_ARGS__, _global) M(__VA_ARGS__, _shared)
FOR_AS(DECL_LOAD_AB, a, col) FOR_AS(DECL_LOAD_AB, a, row) FOR_AS(DECL_LOAD_AB, b, col) FOR_AS(DECL_LOAD_AB, b, row)
FOR_AS(DECL_LOAD_C, col) FOR_AS(DECL_LOAD_C, row) FOR_AS(DECL_STORE, col) FOR_AS(DECL_STORE, row)
DECL_MMA(col, col) DECL_MMA(col, row) DECL_MMA(row, col) DECL_MMA(row, row)
}

struct Sel { int a_row, b_row, c_row, d_row, c_f16, d_f16, as; };

// address of `p` in the state space the selected variant expects
__device__ const void* in_space(const void* p, int as) {
    if (as == 1) return reinterpret_cast<const void*>(__cvta_generic_to_global(p));
    if (as == 3) return reinterpret_cast<const void*>(__cvta_generic_to_shared(p));
    return p;
}

#define PICK_AS(call_generic, call_global, call_shared) (s.as == 0 ? call_generic : (s.as == 1 ? call_global : call_shared))

__global__ void harness_kernel(Sel s, const void* a, const void* b, const void* c, void* d) {
    __shared__ __align__(32) unsigned char sa[512], sb[512], sc[1024], sd[1024];
    const void *pa = a, *pb = b, *pc = c;
    void* pd = d;
    if (s.as == 3) {  // stage everything through shared memory, like the reference's shared-memory tests
        for (int i = threadIdx.x; i < 512; i += 32) { sa[i] = static_cast<const unsigned char*>(a)[i]; sb[i] = static_cast<const unsigned char*>(b)[i]; }
        for (int i = threadIdx.x; i < (s.c_f16 ? 512 : 1024); i += 32) sc[i] = static_cast<const unsigned char*>(c)[i];
        __syncwarp();
        pa = sa; pb = sb; pc = sc; pd = sd;
    }
    pa = in_space(pa, s.as); pb = in_space(pb, s.as); pc = in_space(pc, s.as);
    void* pd_sp = const_cast<void*>(in_space(pd, s.as));

    b200_frag_ab fa = s.a_row ? PICK_AS(b200_wmma_load_a_row_m16n16k16_stride_f16(pa, 16), b200_wmma_load_a_row_m16n16k16_global_stride_f16(pa, 16), b200_wmma_load_a_row_m16n16k16_shared_stride_f16(pa, 16))
                              : PICK_AS(b200_wmma_load_a_col_m16n16k16_stride_f16(pa, 16), b200_wmma_load_a_col_m16n16k16_global_stride_f16(pa, 16), b200_wmma_load_a_col_m16n16k16_shared_stride_f16(pa, 16));
    b200_frag_ab fb = s.b_row ? PICK_AS(b200_wmma_load_b_row_m16n16k16_stride_f16(pb, 16), b200_wmma_load_b_row_m16n16k16_global_stride_f16(pb, 16), b200_wmma_load_b_row_m16n16k16_shared_stride_f16(pb, 16))
                              : PICK_AS(b200_wmma_load_b_col_m16n16k16_stride_f16(pb, 16), b200_wmma_load_b_col_m16n16k16_global_stride_f16(pb, 16), b200_wmma_load_b_col_m16n16k16_shared_stride_f16(pb, 16));
    b200_frag_h ch = {}, dh = {};
    b200_frag_f cf = {}, df = {};
    if (s.c_f16)
        ch = s.c_row ? PICK_AS(b200_wmma_load_c_row_m16n16k16_stride_f16(pc, 16), b200_wmma_load_c_row_m16n16k16_global_stride_f16(pc, 16), b200_wmma_load_c_row_m16n16k16_shared_stride_f16(pc, 16))
                     : PICK_AS(b200_wmma_load_c_col_m16n16k16_stride_f16(pc, 16), b200_wmma_load_c_col_m16n16k16_global_stride_f16(pc, 16), b200_wmma_load_c_col_m16n16k16_shared_stride_f16(pc, 16));
    else
        cf = s.c_row ? PICK_AS(b200_wmma_load_c_row_m16n16k16_stride_f32(pc, 16), b200_wmma_load_c_row_m16n16k16_global_stride_f32(pc, 16), b200_wmma_load_c_row_m16n16k16_shared_stride_f32(pc, 16))
                     : PICK_AS(b200_wmma_load_c_col_m16n16k16_stride_f32(pc, 16), b200_wmma_load_c_col_m16n16k16_global_stride_f32(pc, 16), b200_wmma_load_c_col_m16n16k16_shared_stride_f32(pc, 16));

#define MMA4(al, bl)                                                                             \
    if (s.d_f16) dh = s.c_f16 ? b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f16(fa, fb, ch)        \
                              : b200_wmma_mma_##al##_##bl##_m16n16k16_f16_f32(fa, fb, cf);       \
    else df = s.c_f16 ? b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f16(fa, fb, ch)                \
                      : b200_wmma_mma_##al##_##bl##_m16n16k16_f32_f32(fa, fb, cf);
    if (s.a_row) { if (s.b_row) { MMA4(row, row) } else { MMA4(row, col) } }
    else         { if (s.b_row) { MMA4(col, row) } else { MMA4(col, col) } }

    if (s.d_f16) {
        if (s.d_row) PICK_AS(b200_wmma_store_d_row_m16n16k16_stride_f16(pd_sp, dh, 16), b200_wmma_store_d_row_m16n16k16_global_stride_f16(pd_sp, dh, 16), b200_wmma_store_d_row_m16n16k16_shared_stride_f16(pd_sp, dh, 16));
        else PICK_AS(b200_wmma_store_d_col_m16n16k16_stride_f16(pd_sp, dh, 16), b200_wmma_store_d_col_m16n16k16_global_stride_f16(pd_sp, dh, 16), b200_wmma_store_d_col_m16n16k16_shared_stride_f16(pd_sp, dh, 16));
    } else {
        if (s.d_row) PICK_AS(b200_wmma_store_d_row_m16n16k16_stride_f32(pd_sp, df, 16), b200_wmma_store_d_row_m16n16k16_global_stride_f32(pd_sp, df, 16), b200_wmma_store_d_row_m16n16k16_shared_stride_f32(pd_sp, df, 16));
        else PICK_AS(b200_wmma_store_d_col_m16n16k16_stride_f32(pd_sp, df, 16), b200_wmma_store_d_col_m16n16k16_global_stride_f32(pd_sp, df, 16), b200_wmma_store_d_col_m16n16k16_shared_stride_f32(pd_sp, df, 16));
    }
    if (s.as == 3) {
        __syncwarp();
        for (int i = threadIdx.x; i < (s.d_f16 ? 512 : 1024); i += 32) static_cast<unsigned char*>(d)[i] = sd[i];
    }
}

// Launch on the default stream and wait.  Returns the cudaError_t of the launch / sync.
extern "C" int harness_run(int a_row, int b_row, int c_row, int d_row, int c_f16, int d_f16, int as, const void* a,
                           const void* b, const void* c, void* d) {
    Sel s{a_row, b_row, c_row, d_row, c_f16, d_f16, as};
    harness_kernel<<<1, 32>>>(s, a, b, c, d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaDeviceSynchronize());
}

// The same one-warp kernel launched as a 16 x 2 block: the warp's lanes are then NOT threadIdx.x & 31.
// Generic and global address spaces only (the shared-memory staging above strides by threadIdx.x).
extern "C" int harness_run_block16x2(int a_row, int b_row, int c_row, int d_row, int c_f16, int d_f16, int as, const void* a,
                                     const void* b, const void* c, void* d) {
    if (as == 3) return static_cast<int>(cudaErrorInvalidValue);
    Sel s{a_row, b_row, c_row, d_row, c_f16, d_f16, as};
    harness_kernel<<<1, dim3(16, 2, 1)>>>(s, a, b, c, d);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    return static_cast<int>(cudaDeviceSynchronize());
}
