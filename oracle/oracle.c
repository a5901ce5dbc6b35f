/*
 * oracle.c -- CPU restatement of the arithmetic behind CUDAnative.jl's WMMA path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing under the product package may include, link or call this
 * file; it exists so that tests, the smoke check and the benchmark's CPU-baseline leg have an
 * independent answer to compare the CUDA kernels with.
 *
 * PARITY UNPINNED for the arithmetic: the reference defines D = A*B + C only by delegating to
 * the wmma.mma hardware instruction (src/device/cuda/wmma.jl:222-257 emits
 * llvm.nvvm.wmma.m16n16k16.mma.*), ships no golden vectors, and its own tests compare against a
 * CPU product recomputed from unseeded rand() with rtol = sqrt(eps(Float16))
 * (test/device/wmma.jl:102-151, :188-248).  Julia is not available in this environment, so no
 * output of the reference could be recorded either.  What IS pinned: the exact host-side
 * equalities of test/device/wmma.jl:156-184 (flatten / unflatten / broadcasting), restated in
 * tests/test_wmma_host.py.
 *
 * The restatement follows the CPU side of the reference's own tests:
 *   - oracle_wmma_unit : alpha * new_a * new_b + beta * new_c with alpha folded into the Float16
 *     A operand and beta into C in C's element type (test/device/wmma.jl:223-224, :238-246) and
 *     "row major" meaning the transpose of the stored matrix (test/device/wmma.jl:233-236)
 *   - oracle_gemm      : D = alpha * (A*B) + beta * C in binary32 on binary16-rounded inputs,
 *     the product the examples check (examples/wmma/high-level.jl:49: a*b + 0.5*c)
 * plus the binary16 rounding and the counter-based input generator shared with the library.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* ---- binary16 <-> binary32, round to nearest even (IEEE 754) ---------------------------- */
uint16_t oracle_f32_to_f16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x200u : 0)); /* inf / nan */
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to >= 65520: overflow to inf */
    if (absx < 0x33000001u) return (uint16_t)sign;              /* below half the smallest subnormal */
    int exp = (int)(absx >> 23) - 127;
    uint32_t mant = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t half_exp;
    if (exp < -14) { /* subnormal result */
        shift = 13 + (-14 - exp);
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t kept = mant >> shift;
    const uint32_t rem = mant & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (kept & 1u))) kept++;
    uint32_t out;
    if (half_exp == 0) out = kept; /* a carry into bit 10 correctly becomes the smallest normal */
    else out = ((half_exp - 1) << 10) + kept; /* kept carries the implicit bit: adds 1 to the exponent */
    return (uint16_t)(sign | out);
}

float oracle_f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t mant = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (mant == 0) x = sign;
        else {
            int e = -1;
            do { mant <<= 1; e++; } while (!(mant & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((mant & 0x3ffu) << 13);
        }
    } else if (exp == 31) x = sign | 0x7f800000u | (mant << 13);
    else x = sign | ((exp + 112) << 23) | (mant << 13);
    float f;
    memcpy(&f, &x, 4);
    return f;
}

float oracle_round_f16(float f) { return oracle_f16_bits_to_f32(oracle_f32_to_f16_bits(f)); }

/* ---- bfloat16 <-> binary32 ---------------------------------------------------------------
 * bfloat16 is the upper half of a binary32 (1 sign, 8 exponent, 7 fraction bits); the reference has no
 * such type (its WMMA element types are Float16 and Float32, src/device/cuda/wmma.jl:11-37), so this
 * follows IEEE 754 round-to-nearest-even on the dropped 16 bits.  Written with a comparison of the
 * remainder against the half-way point instead of the add-and-shift trick the library's host helper
 * uses, so that the two check each other. */
uint16_t oracle_f32_to_bf16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x0040u); /* NaN stays NaN (quiet) */
    uint32_t kept = x >> 16;
    const uint32_t rem = x & 0xffffu;
    if (rem > 0x8000u || (rem == 0x8000u && (kept & 1u))) kept++; /* may carry into the exponent: up to infinity */
    return (uint16_t)kept;
}

float oracle_bf16_bits_to_f32(uint16_t b) {
    const uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

void oracle_round_bf16_array(const float* in, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = oracle_f32_to_bf16_bits(in[i]);
}

void oracle_widen_bf16_array(const uint16_t* in, float* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = oracle_bf16_bits_to_f32(in[i]);
}

/* ---- counter-based inputs (same definition as the library's fill kernels) ---------------- */
static uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

float oracle_synth_value(uint64_t seed, uint64_t matrix_id, uint64_t index, int dist) {
    const uint64_t u = splitmix64(seed * 0x9E3779B97F4A7C15ull + matrix_id * 0xD1B54A32D192ED03ull + index);
    if (dist == 0) return (float)((double)(u >> 40) * (1.0 / 8388608.0) - 1.0);
    if (dist == 1) {
        const double u1 = ((double)(u >> 40) + 1.0) * (1.0 / 16777216.0);
        const double u2 = (double)((u >> 16) & 0xFFFFFFull) * (1.0 / 16777216.0);
        return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
    }
    return 0.0f;
}

/* rows x cols column-major window starting at column col0 of a `rows`-tall synthetic matrix */
void oracle_fill(float* out, int64_t rows, int64_t cols, int64_t ld, uint64_t seed, uint64_t matrix_id,
                 int64_t col0, int dist, float scale, int round_to_f16) {
    for (int64_t j = 0; j < cols; ++j)
        for (int64_t i = 0; i < rows; ++i) {
            float v = oracle_synth_value(seed, matrix_id, (uint64_t)((j + col0) * rows + i), dist) * scale;
            out[i + j * ld] = round_to_f16 ? oracle_round_f16(v) : v;
        }
}

/* ---- D = alpha * op(A) * op(B) + beta * C ------------------------------------------------ */
/* A, B hold binary16-representable values as float.  acc64 != 0 accumulates in double (the
 * yardstick for checking the binary32 answers themselves); otherwise in float, k ascending.
 * Column-major; transX = 1 reads the stored matrix transposed. */
void oracle_gemm(int transA, int transB, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda,
                 const float* B, int64_t ldb, float beta, const float* C, int64_t ldc, float* D, int64_t ldd,
                 int acc64) {
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            double accd = 0.0;
            float accf = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                const float a = transA ? A[k + m * lda] : A[m + k * lda];
                const float b = transB ? B[n + k * ldb] : B[k + n * ldb];
                if (acc64) accd += (double)a * (double)b;
                else accf += a * b;
            }
            if (acc64) {
                double v = (double)alpha * accd;
                if (beta != 0.0f) v += (double)beta * (double)C[m + n * ldc];
                D[m + n * ldd] = (float)v;
            } else {
                float v = alpha * accf;
                if (beta != 0.0f) v += beta * C[m + n * ldc];
                D[m + n * ldd] = v;
            }
        }
}

/* ---- the same product with a binary16 accumulator ------------------------------------------- */
/* What a caller of the reference gets who loops WMMA.mma over K with Config{16, 16, 16, Float16} and a
 * Float16 accumulator fragment (the .f16.f16 variants, src/device/cuda/wmma.jl:222-257): the running
 * sum is rounded to binary16 after every `block` products (16 = the instruction's K).  Inside a block
 * the products are summed in double and rounded once -- the hardware's order inside one instruction is
 * not specified, the reference's own test allows rtol = sqrt(eps(Float16)) (test/device/wmma.jl:243-246).
 * alpha and beta are applied in binary32 and D is rounded to binary16 once. */
void oracle_gemm_f16acc(int transA, int transB, int64_t M, int64_t N, int64_t K, float alpha, const float* A, int64_t lda,
                        const float* B, int64_t ldb, float beta, const float* C, int64_t ldc, float* D, int64_t ldd,
                        int block) {
    if (block < 1) block = 16;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t m = 0; m < M; ++m) {
            float acc = 0.0f; /* always a binary16 value */
            for (int64_t k0 = 0; k0 < K; k0 += block) {
                double part = 0.0;
                for (int64_t k = k0; k < K && k < k0 + block; ++k) {
                    const float a = transA ? A[k + m * lda] : A[m + k * lda];
                    const float b = transB ? B[n + k * ldb] : B[k + n * ldb];
                    part += (double)a * (double)b;
                }
                acc = oracle_round_f16((float)((double)acc + part));
            }
            float v = alpha * acc;
            if (beta != 0.0f) v += beta * C[m + n * ldc];
            D[m + n * ldd] = oracle_round_f16(v);
        }
}

/* ---- the 16x16x16 unit as the reference's test states it ----------------------------------- */
/* a, b: 16x16 binary16 values as float in their STORED order with leading dimension 16;
 * layouts 0 = ColMajor, 1 = RowMajor (stored matrix is the transpose).  c_is_f16 / d_is_f16
 * select the element types of C and D.  use_alpha: a := Float16(alpha) * a rounded to binary16;
 * use_beta: c := beta * c in C's type.  mac = 0 is the fill_c(0) case.  The product itself is
 * evaluated in double and rounded once to D's type, so that the hardware's accumulation order
 * stays inside the tolerance the reference's test allows. */
void oracle_wmma_unit(int a_layout, int b_layout, int c_layout, int d_layout, int c_is_f16, int d_is_f16, int mac,
                      int use_alpha, float alpha, int use_beta, float beta, const float* a, const float* b,
                      const float* c, float* d) {
    float as[256], bs[256], cs[256];
    const float alpha_t = oracle_round_f16(alpha);
    const float beta_t = c_is_f16 ? oracle_round_f16(beta) : beta;
    for (int i = 0; i < 16; ++i)
        for (int j = 0; j < 16; ++j) {
            float av = a_layout ? a[i * 16 + j] : a[i + j * 16];
            if (use_alpha) av = oracle_round_f16(alpha_t * av);
            as[i + j * 16] = av;
            bs[i + j * 16] = b_layout ? b[i * 16 + j] : b[i + j * 16];
            float cv = 0.0f;
            if (mac) {
                cv = c_layout ? c[i * 16 + j] : c[i + j * 16];
                if (use_beta) cv = c_is_f16 ? oracle_round_f16(beta_t * cv) : beta_t * cv;
            }
            cs[i + j * 16] = cv;
        }
    for (int i = 0; i < 16; ++i)
        for (int j = 0; j < 16; ++j) {
            double acc = (double)cs[i + j * 16];
            for (int k = 0; k < 16; ++k) acc += (double)as[i + k * 16] * (double)bs[k + j * 16];
            const float v = d_is_f16 ? oracle_round_f16((float)acc) : (float)acc;
            if (d_layout) d[i * 16 + j] = v;
            else d[i + j * 16] = v;
        }
}
