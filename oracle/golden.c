/*
 * CPU oracle for the block-scaled GEMM path.  TEST INFRASTRUCTURE ONLY: nothing
 * in the shipped library links, loads or calls this file; it is the checker the
 * tests, the smoke run and the benchmark's cpu_baseline leg compare against.
 *
 * It restates, in plain C, the arithmetic of the reference's CPU golden model
 * (deepgemm/src/golden.rs:56-510).  Each function names the lines it follows.
 * Parity pin: the known-answer tests of the reference's own test-suite
 * (deepgemm/tests/golden_tests.rs, deepgemm/tests/cpu_tests.rs) are re-run
 * against this file by tests/test_oracle_kat.py.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC -o liboracle.so golden.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DG_FP8 0
#define DG_FP4 1

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* golden.rs:56-73 */
uint32_t dgo_ceil_div(uint32_t a, uint32_t b) { return (a + b - 1) / b; }
uint32_t dgo_align_up(uint32_t x, uint32_t to) { return dgo_ceil_div(x, to) * to; }
uint32_t dgo_tma_aligned(uint32_t mn, uint32_t elem_size) {
    uint32_t per = 16 / elem_size;
    if (per < 1) per = 1;
    return dgo_align_up(mn, per);
}

/* golden.rs:80-92 : 0x7f / 0xff are NaN; exponent field 0 is subnormal m*2^-9. */
float dgo_e4m3_decode(uint8_t b) {
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int exp = (b >> 3) & 0xf;
    float mant = (float)(b & 0x7);
    if (exp == 0) return sign * mant * ldexpf(1.0f, -9);
    if ((b & 0x7f) == 0x7f) return NAN;
    return sign * (1.0f + mant / 8.0f) * ldexpf(1.0f, exp - 7);
}

/* golden.rs:95-103 */
float dgo_e2m1_decode(uint8_t n) {
    static const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = grid[n & 7];
    return (n & 8) ? -v : v;
}

/* golden.rs:107-109 */
float dgo_ue8m0_decode(uint8_t code) { return ldexpf(1.0f, (int)code - 127); }

/* golden.rs:115-117 */
uint8_t dgo_f32_to_ue8m0(float v) { return (uint8_t)((f2u(v) >> 23) & 0xff); }

/* golden.rs:120-135 : the E4M3 grid has 8 subnormals + 15 binades x 8 = 128 entries,
 * so its last entry is 480 (the byte 0x7f), not 448. */
static double g_e4m3_grid[128];
static const double g_e2m1_grid[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
static int g_grid_ready = 0;
static void grids_init(void) {
    if (g_grid_ready) return;
    int n = 0;
    for (int m = 0; m < 8; ++m) g_e4m3_grid[n++] = (double)m * ldexp(1.0, -9);
    for (int e = 1; e <= 15; ++e)
        for (int m = 0; m < 8; ++m) g_e4m3_grid[n++] = (1.0 + (double)m / 8.0) * ldexp(1.0, e - 7);
    g_grid_ready = 1;
}

/* golden.rs:142-176 : nearest grid entry, ties to the even index, clamp at both ends.
 * A NaN input fails every comparison and lands on index 0, as in the reference. */
static int rne_on_grid(double a, const double* grid, int len) {
    if (a <= grid[0]) return 0;
    if (a >= grid[len - 1]) return len - 1;
    int lo = 0, hi = len - 1;
    while (hi - lo > 1) {
        int mid = (lo + hi) / 2;
        if (grid[mid] <= a) lo = mid; else hi = mid;
    }
    double gl = grid[lo], gh = grid[hi];
    double mid = (gl + gh) / 2.0;
    if (a < mid) return lo;
    if (a > mid) return hi;
    return (lo % 2 == 0) ? lo : hi;
}

/* golden.rs:180-189 : sign comes from the sign bit, so -0.0 encodes as 0x80. */
uint8_t dgo_quant_e4m3(float v) {
    grids_init();
    int code = rne_on_grid((double)fabsf(v), g_e4m3_grid, 128);
    return (uint8_t)((signbit(v) ? 0x80 : 0) | code);
}

/* quant_e4m3 over an array (input generator for raw-E4M3 tensors such as the MQA query). */
void dgo_quant_e4m3_vec(const float* x, size_t n, uint8_t* out) {
    grids_init();
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = dgo_quant_e4m3(x[i]);
}

/* golden.rs:193-202 */
uint8_t dgo_quant_e2m1(float v) {
    int code = rne_on_grid((double)fabsf(v), g_e2m1_grid, 8);
    return (uint8_t)((signbit(v) ? 0x8 : 0) | code);
}

/* golden.rs:211-224 : 448 = 1.75 * 2^8; floor exponent 105. */
uint8_t dgo_ue8m0_exp_fp8(float amax) {
    uint32_t bits = f2u(amax);
    uint32_t rounded = (bits + 0x7fffffu - (0x60u << 16)) >> 23;
    uint32_t lo = 105u + 8u;
    if (rounded < lo) rounded = lo;
    return (uint8_t)(rounded - 8u);
}

/* golden.rs:228-241 : 6 = 1.5 * 2^2; floor exponent 1. */
uint8_t dgo_ue8m0_exp_fp4(float amax) {
    uint32_t bits = f2u(amax);
    uint32_t rounded = (bits + 0x7fffffu - (0x40u << 16)) >> 23;
    uint32_t lo = 1u + 2u;
    if (rounded < lo) rounded = lo;
    return (uint8_t)(rounded - 2u);
}

/* golden.rs:261-281 : f32 [mn, sf_k] -> u32 [ceil(sf_k/4), align4(mn)], byte k%4 of
 * word [k/4][m] is the exponent byte of sf[m][k]; padding stays zero.
 * `out` must hold ceil(sf_k/4) * align4(mn) words. */
void dgo_transform_sf_host(const float* sf, uint32_t mn, uint32_t sf_k, uint32_t* out) {
    uint32_t cols = dgo_tma_aligned(mn, 4), rows = dgo_ceil_div(sf_k, 4);
    memset(out, 0, (size_t)rows * cols * 4);
    for (uint32_t m = 0; m < mn; ++m)
        for (uint32_t k = 0; k < sf_k; ++k) {
            uint32_t byte = dgo_f32_to_ue8m0(sf[(size_t)m * sf_k + k]);
            out[(size_t)(k / 4) * cols + m] |= byte << (8 * (k % 4));
        }
}

/* golden.rs:299-363 : per (row, group of g) amax -> exponent -> codes.
 * data: m*k bytes (FP8) or m*k/2 bytes (FP4, even k in the low nibble);
 * sf: ceil(k/g/4) * align4(m) words, zero-initialised here. */
void dgo_quant_mx_host(const float* x, uint32_t m, uint32_t k, int dtype, uint32_t g,
                       uint8_t* data, uint32_t* sf) {
    grids_init();
    uint32_t num_groups = k / g;
    uint32_t sf_cols = dgo_tma_aligned(m, 4), sf_rows = dgo_ceil_div(num_groups, 4);
    int is_fp4 = dtype == DG_FP4;
    memset(data, 0, is_fp4 ? (size_t)m * k / 2 : (size_t)m * k);
    memset(sf, 0, (size_t)sf_rows * sf_cols * 4);
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < m; ++row) {
        for (uint32_t gi = 0; gi < num_groups; ++gi) {
            const float* px = x + (size_t)row * k + (size_t)gi * g;
            float amax = 0.0f;
            for (uint32_t i = 0; i < g; ++i) {
                float v = fabsf(px[i]);
                if (v > amax) amax = v;
            }
            if (amax < 1e-30f) amax = 1e-30f;
            uint8_t e = is_fp4 ? dgo_ue8m0_exp_fp4(amax) : dgo_ue8m0_exp_fp8(amax);
            float inv_sf = u2f((254u - (uint32_t)e) << 23);
            for (uint32_t i = 0; i < g; ++i) {
                float v = px[i] * inv_sf;
                uint32_t kk = gi * g + i;
                if (is_fp4) {
                    size_t bi = ((size_t)row * k) / 2 + kk / 2;
                    uint8_t nib = dgo_quant_e2m1(v);
                    if ((kk & 1) == 0) data[bi] = (uint8_t)((data[bi] & 0xf0) | (nib & 0x0f));
                    else data[bi] = (uint8_t)((data[bi] & 0x0f) | (nib << 4));
                } else {
                    data[(size_t)row * k + kk] = dgo_quant_e4m3(v);
                }
            }
            /* Rows of one word are touched by one thread only: the word index depends
             * on (gi/4, row) and rows are partitioned across threads. */
            sf[(size_t)(gi / 4) * sf_cols + row] |= (uint32_t)e << (8 * (gi % 4));
        }
    }
}

/* golden.rs:366-396 */
void dgo_dequant_mx_host(const uint8_t* data, const uint32_t* sf, uint32_t sf_cols,
                         uint32_t m, uint32_t k, int dtype, uint32_t g, float* out) {
    int is_fp4 = dtype == DG_FP4;
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < m; ++row)
        for (uint32_t col = 0; col < k; ++col) {
            uint32_t slot = col / g;
            uint32_t word = sf[(size_t)(slot / 4) * sf_cols + row];
            float scale = dgo_ue8m0_decode((uint8_t)((word >> (8 * (slot % 4))) & 0xff));
            float v;
            if (is_fp4) {
                uint8_t b = data[((size_t)row * k) / 2 + col / 2];
                v = dgo_e2m1_decode((col & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf)) * scale;
            } else {
                v = dgo_e4m3_decode(data[(size_t)row * k + col]) * scale;
            }
            out[(size_t)row * k + col] = v;
        }
}

/* GoldenOperand::scaled, golden.rs:418-439 : decoded code (as f64) times the f32 scale
 * widened to f64.  Hoisted out of the MAC loop: one row is decoded once into a f64
 * buffer; the products and the k-ordered f64 sum are the reference's (golden.rs:444-458). */
static void decode_row(const uint8_t* data, const uint32_t* sf, uint32_t sf_cols, int dtype,
                       uint32_t g, uint32_t r, uint32_t k, double* out) {
    for (uint32_t kk = 0; kk < k; ++kk) {
        double raw;
        if (dtype == DG_FP4) {
            uint8_t b = data[((size_t)r * k) / 2 + kk / 2];
            raw = (double)dgo_e2m1_decode((kk & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf));
        } else {
            raw = (double)dgo_e4m3_decode(data[(size_t)r * k + kk]);
        }
        uint32_t slot = kk / g;
        uint32_t word = sf[(size_t)(slot / 4) * sf_cols + r];
        out[kk] = raw * (double)dgo_ue8m0_decode((uint8_t)((word >> (8 * (slot % 4))) & 0xff));
    }
}

/*
 * gemm_ref, golden.rs:444-458, on a sub-rectangle so that large shapes can be sampled:
 * out[i*ldo + j] = (f32) sum_k a.scaled(rows[i], k) * b.scaled(b_row0 + cols[j], k),
 * f64 products and f64 accumulation in k order.  `rows`/`cols` may be NULL for 0..n-1.
 * `b_row0` offsets B rows (expert e of a stacked [G*N, K] weight: b_row0 = e*N).
 */
void dgo_gemm_ref_sub(const uint8_t* a_data, const uint32_t* a_sf, uint32_t a_sf_cols, int a_dtype, uint32_t a_g,
                      const uint8_t* b_data, const uint32_t* b_sf, uint32_t b_sf_cols, int b_dtype, uint32_t b_g,
                      uint32_t k, const uint32_t* rows, uint32_t n_rows,
                      const uint32_t* cols, uint32_t n_cols, uint32_t b_row0,
                      float* out, uint32_t ldo) {
    double* bdec = (double*)malloc((size_t)n_cols * k * sizeof(double));
#pragma omp parallel for schedule(static)
    for (uint32_t j = 0; j < n_cols; ++j)
        decode_row(b_data, b_sf, b_sf_cols, b_dtype, b_g, b_row0 + (cols ? cols[j] : j), k, bdec + (size_t)j * k);
#pragma omp parallel
    {
        double* adec = (double*)malloc((size_t)k * sizeof(double));
#pragma omp for schedule(dynamic, 1)
        for (uint32_t i = 0; i < n_rows; ++i) {
            decode_row(a_data, a_sf, a_sf_cols, a_dtype, a_g, rows ? rows[i] : i, k, adec);
            for (uint32_t j = 0; j < n_cols; ++j) {
                const double* bj = bdec + (size_t)j * k;
                double acc = 0.0;
                for (uint32_t kk = 0; kk < k; ++kk) acc += adec[kk] * bj[kk];
                out[(size_t)i * ldo + j] = (float)acc;
            }
        }
        free(adec);
    }
    free(bdec);
}

/* GoldenOperand::scaled for one element, golden.rs:418-439. */
static double scaled_one(const uint8_t* data, const uint32_t* sf, uint32_t sf_cols, int dtype,
                         uint32_t g, uint32_t r, uint32_t k, uint32_t kk) {
    uint8_t code;
    if (dtype == DG_FP4) {
        uint8_t b = data[((size_t)r * k) / 2 + kk / 2];
        code = (kk & 1) ? (uint8_t)(b >> 4) : (uint8_t)(b & 0xf);
    } else {
        code = data[(size_t)r * k + kk];
    }
    double raw = dtype == DG_FP4 ? (double)dgo_e2m1_decode(code) : (double)dgo_e4m3_decode(code);
    uint32_t slot = kk / g;
    uint32_t w = sf[(size_t)(slot / 4) * sf_cols + r];
    return raw * (double)dgo_ue8m0_decode((uint8_t)((w >> (8 * (slot % 4))) & 0xff));
}

/* gemm_ref exactly in the shape golden.rs:444-458 writes it (two decodes per MAC); used
 * to check that the hoisted form above is bit-identical. */
void dgo_gemm_ref_naive(const uint8_t* a_data, const uint32_t* a_sf, uint32_t a_sf_cols, int a_dtype, uint32_t a_g,
                        const uint8_t* b_data, const uint32_t* b_sf, uint32_t b_sf_cols, int b_dtype, uint32_t b_g,
                        uint32_t m, uint32_t n, uint32_t k, float* out) {
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (uint32_t kk = 0; kk < k; ++kk)
                acc += scaled_one(a_data, a_sf, a_sf_cols, a_dtype, a_g, i, k, kk) *
                       scaled_one(b_data, b_sf, b_sf_cols, b_dtype, b_g, j, k, kk);
            out[(size_t)i * n + j] = (float)acc;
        }
}

/* A plain f64-accumulated NT product of f32 (or widened bf16) operands: the shape of
 * gemm_ref with no codes to decode, used for the BF16 GEMM and as the "direct matmul of
 * dequantised operands" of golden_tests.rs:285-295. */
void dgo_gemm_f32_ref(const float* a, const float* b, uint32_t m, uint32_t n, uint32_t k, float* out) {
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (uint32_t kk = 0; kk < k; ++kk) acc += (double)a[(size_t)i * k + kk] * (double)b[(size_t)j * k + kk];
            out[(size_t)i * n + j] = (float)acc;
        }
}

/* mqa_logits_ref, golden.rs:469-501 : f64 dot, `dot > 0` gate, f64 head sum, f32 output at
 * the ABSOLUTE column, zero outside [k_start, min(k_end, num_kv)).  `tokens` (may be NULL)
 * selects the query rows to evaluate; `out` is [n_tokens, num_kv]. */
void dgo_mqa_logits_ref(const float* q, const float* kv, const float* weights,
                        uint32_t num_heads, uint32_t head_dim, uint32_t num_kv,
                        const uint32_t* k_start, const uint32_t* k_end,
                        const uint32_t* tokens, uint32_t n_tokens, float* out) {
    memset(out, 0, (size_t)n_tokens * num_kv * sizeof(float));
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t ti = 0; ti < n_tokens; ++ti) {
        uint32_t t = tokens ? tokens[ti] : ti;
        uint32_t lo = k_start[t], hi = k_end[t] < num_kv ? k_end[t] : num_kv;
        for (uint32_t kvv = lo; kvv < hi; ++kvv) {
            double acc = 0.0;
            for (uint32_t h = 0; h < num_heads; ++h) {
                const float* qp = q + ((size_t)t * num_heads + h) * head_dim;
                const float* kp = kv + (size_t)kvv * head_dim;
                double dot = 0.0;
                for (uint32_t d = 0; d < head_dim; ++d) dot += (double)qp[d] * (double)kp[d];
                if (dot > 0.0) acc += (double)weights[(size_t)t * num_heads + h] * dot;
            }
            out[(size_t)ti * num_kv + kvv] = (float)acc;
        }
    }
}

/* golden.rs:505-510 */
uint16_t dgo_f32_to_bf16_bits(float v) {
    uint32_t bits = f2u(v);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t rounding = 0x7fffu + lsb;
    return (uint16_t)((((bits + rounding) >> 16) & 0x7fffu) | ((bits >> 31) << 15));
}

/* calc_diff = 1 - 2*sum(xy) / sum(x^2 + y^2), deepgemm/tests/parity_tests.rs:553-568 and
 * deepgemm-bench/src/main.rs:2191-2200; 0 when both are all-zero. */
double dgo_calc_diff(const float* x, const float* y, size_t n) {
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < n; ++i) {
        double a = x[i], b = y[i];
        num += 2.0 * a * b;
        den += a * a + b * b;
    }
    return den == 0.0 ? 0.0 : 1.0 - num / den;
}

/*
 * Input generator for the "128x128 block of B" recipe.  The reference has no such
 * quantiser (its quant_mx_host is per row); the operator API carries a block scale as
 * the same exponent byte replicated over the block's 128 rows in the ordinary per-row
 * packed layout.  amax is taken over each 128-row x 128-column block, then the per-row
 * arithmetic of golden.rs:327-351 is applied with that shared exponent.
 */
void dgo_quant_fp8_block128_host(const float* x, uint32_t n, uint32_t k, uint8_t* data, uint32_t* sf) {
    grids_init();
    uint32_t num_groups = k / 128;
    uint32_t sf_cols = dgo_tma_aligned(n, 4), sf_rows = dgo_ceil_div(num_groups, 4);
    memset(sf, 0, (size_t)sf_rows * sf_cols * 4);
    uint32_t n_blocks = dgo_ceil_div(n, 128);
#pragma omp parallel for schedule(static)
    for (uint32_t rb = 0; rb < n_blocks; ++rb) {
        uint32_t r0 = rb * 128, r1 = r0 + 128 < n ? r0 + 128 : n;
        for (uint32_t gi = 0; gi < num_groups; ++gi) {
            float amax = 0.0f;
            for (uint32_t r = r0; r < r1; ++r)
                for (uint32_t i = 0; i < 128; ++i) {
                    float v = fabsf(x[(size_t)r * k + (size_t)gi * 128 + i]);
                    if (v > amax) amax = v;
                }
            if (amax < 1e-30f) amax = 1e-30f;
            uint8_t e = dgo_ue8m0_exp_fp8(amax);
            float inv_sf = u2f((254u - (uint32_t)e) << 23);
            for (uint32_t r = r0; r < r1; ++r) {
                for (uint32_t i = 0; i < 128; ++i) {
                    size_t idx = (size_t)r * k + (size_t)gi * 128 + i;
                    data[idx] = dgo_quant_e4m3(x[idx] * inv_sf);
                }
                sf[(size_t)(gi / 4) * sf_cols + r] |= (uint32_t)e << (8 * (gi % 4));
            }
        }
    }
}

/* SwiGLU between the two grouped GEMMs of an MoE layer, on the BF16 output [m, 2 * inter] of the
 * gate/up projection (row pitch ld elements): gate = columns [0, inter), up = columns
 * [inter, 2 * inter) ("the two halves", deepgemm/src/api_serving.rs:371-373).  As in the golden model of
 * the fused path (golden.rs:569-577) both factors are the bf16-rounded GEMM outputs and the product
 * silu(g) * u, silu(g) = g * (1 / (1 + exp(-g))) (a reciprocal, then a product), is formed in f32; there is no clamp and the routing weight is
 * applied later, when the copies of a token are combined.  out: f32 [m, inter], the input of the
 * re-quantisation (dgo_quant_mx_host).
 * The golden model calls the platform's exp; platforms differ in its last bit, which would make the
 * E4M3 codes after re-quantisation platform dependent.  The function is therefore spelled out here as a
 * sequence of correctly rounded f32 operations, and the device code evaluates the same sequence:
 *   x = -g clamped to [-87, 87];  t = fma(x, log2 e, 1.5 * 2^23), whose low mantissa bits hold
 *   n = round(x * log2 e);  f = x - n * ln 2 in two steps;  p = degree-6 Taylor polynomial of exp(f), Horner,
 *   fused multiply-adds;  2^n from the bits of t;  p * 2^n is within about 1 ulp of expf (asserted by the tests);
 *   d = fma(p, 2^n, 1);  r = 1 / d by three Newton steps from the seed bits 0x7ef311c7 - bits(d);
 *   silu(g) * u = (g * r) * u. */
static float exp_parts(float x, float* scale) {
    if (x < -87.0f) x = -87.0f;
    if (x > 87.0f) x = 87.0f;
    float t = fmaf(x, 1.44269502162933349609375f, 12582912.0f);
    float n = t - 12582912.0f;
    float f = fmaf(n, -0.693145751953125f, x);
    f = fmaf(n, -1.428606765330187045037746429443359375e-06f, f);
    float p = fmaf(f, 1.0f / 720.0f, 1.0f / 120.0f);
    p = fmaf(p, f, 1.0f / 24.0f);
    p = fmaf(p, f, 1.0f / 6.0f);
    p = fmaf(p, f, 0.5f);
    p = fmaf(p, f, 1.0f);
    p = fmaf(p, f, 1.0f);
    *scale = u2f((f2u(t) << 23) + 0x3f800000u);
    return p;
}
static float exp_taylor6(float x) {
    float s;
    float p = exp_parts(x, &s);
    return p * s;
}
float dgo_exp_taylor6(float x) { return exp_taylor6(x); }

static float recip_newton3(float d) {
    float r = u2f(0x7ef311c7u - f2u(d));
    for (int i = 0; i < 3; ++i) r = fmaf(r, fmaf(-d, r, 1.0f), r);
    return r;
}
float dgo_recip_newton3(float d) { return recip_newton3(d); }

void dgo_swiglu_f32(const uint16_t* inter_bf16, uint32_t m, uint32_t inter, uint32_t ld, float* out) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < m; ++r) {
        const uint16_t* row = inter_bf16 + (size_t)r * ld;
        for (uint32_t c = 0; c < inter; ++c) {
            float g = u2f((uint32_t)row[c] << 16), u = u2f((uint32_t)row[inter + c] << 16);
            float s;
            float p = exp_parts(-g, &s);
            float sig = g * recip_newton3(fmaf(p, s, 1.0f));
            out[(size_t)r * inter + c] = sig * u;
        }
    }
}

/* api::quantize_output_fp8 (deepgemm/src/api.rs:1951-2011): f32 [m, n] with row pitch in_stride -> E4M3
 * codes [m, n] + packed UE8M0 words [ceil(n/32/4), align4(m)], one scale per (row, 32 columns).
 * Round-to-nearest mode: the exponent rule and cast of the golden model (golden.rs:211-224, 299-363),
 * i.e. quant_mx at granularity 32 on a pitched input.  (The reference's device kernel shifts the 8-bit
 * exponent field where the golden model shifts the float's bits, deepgemm/kernels/layout_quant.cu:339-341;
 * the golden model is the contract.)
 * Stochastic mode (no golden model exists for it; the reference's device code draws from an xorshift
 * stream per group, layout_quant.cu:343-353): defined here as a pure function of (x, seed) -- a scaled
 * value v between neighbouring grid values lo < hi becomes hi when the top 24 bits of
 * hash(element index, seed), read as a fraction in [0, 1), lie below (|v| - lo) / (hi - lo). */
static uint32_t hash_u32(uint64_t idx, uint32_t seed) {
    uint32_t x = (uint32_t)idx * 0x9E3779B9u + (uint32_t)(idx >> 32) * 0x7F4A7C15u + seed;
    x ^= x >> 16; x *= 0x85EBCA6Bu;
    x ^= x >> 13; x *= 0xC2B2AE35u;
    x ^= x >> 16;
    return x;
}
uint32_t dgo_hash_u32(uint64_t idx, uint32_t seed) { return hash_u32(idx, seed); }

static float stochastic_e4m3_value(float v, uint32_t rnd) {
    uint32_t bits = f2u(v), sign = bits & 0x80000000u, mag = bits & 0x7fffffffu;
    if (mag > 0x7f800000u) return v;
    float a = u2f(mag);
    if (a >= 448.0f) return u2f(sign | f2u(448.0f));
    uint32_t e = mag >> 23;
    if (e < 121u) e = 121u;
    float step = u2f((e - 3u) << 23), inv_step = u2f((257u - e) << 23);
    float units = a * inv_step;
    float fl = floorf(units);
    float frac = units - fl;
    float u = (float)(rnd >> 8) * (1.0f / 16777216.0f);
    float r = (u < frac ? fl + 1.0f : fl) * step;
    return u2f(f2u(r) | sign);
}

void dgo_quantize_output_fp8(const float* in, uint32_t m, uint32_t n, uint32_t in_stride, int stochastic, uint32_t seed,
                             uint8_t* data, uint32_t* sf) {
    grids_init();
    uint32_t num_groups = n / 32;
    uint32_t sf_cols = dgo_tma_aligned(m, 4), sf_rows = dgo_ceil_div(num_groups, 4);
    memset(sf, 0, (size_t)sf_rows * sf_cols * 4);
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < m; ++row) {
        for (uint32_t gi = 0; gi < num_groups; ++gi) {
            const float* px = in + (size_t)row * in_stride + (size_t)gi * 32;
            float amax = 0.0f;
            for (uint32_t i = 0; i < 32; ++i) {
                float v = fabsf(px[i]);
                if (v > amax) amax = v;
            }
            if (amax < 1e-30f) amax = 1e-30f;
            uint8_t e = dgo_ue8m0_exp_fp8(amax);
            float inv_sf = u2f((254u - (uint32_t)e) << 23);
            for (uint32_t i = 0; i < 32; ++i) {
                float v = px[i] * inv_sf;
                uint64_t idx = (uint64_t)row * n + gi * 32 + i;
                if (stochastic) v = stochastic_e4m3_value(v, hash_u32(idx, seed));
                data[idx] = dgo_quant_e4m3(v);
            }
            sf[(size_t)(gi / 4) * sf_cols + row] |= (uint32_t)e << (8 * (gi % 4));
        }
    }
}

/* api::transform_sf_batched (deepgemm/src/api.rs:1263-1311): [batch, mn, sf_k] scales -> one arena
 * [batch * ceil(sf_k/4), align4(mn)]; batch b's rows start at b * ceil(sf_k/4), each batch packed as by
 * transform_sf_host. */
void dgo_transform_sf_batched_host(const float* sf, uint32_t batch, uint32_t mn, uint32_t sf_k, uint32_t* out) {
    uint32_t cols = dgo_tma_aligned(mn, 4), rows = dgo_ceil_div(sf_k, 4);
    for (uint32_t b = 0; b < batch; ++b)
        dgo_transform_sf_host(sf + (size_t)b * mn * sf_k, mn, sf_k, out + (size_t)b * rows * cols);
}

/* Thread count of the OpenMP loops above (the benchmark's CPU arm sets it to the host's cores explicitly:
 * launchers such as torch.distributed.run export OMP_NUM_THREADS=1). */
#ifdef _OPENMP
#include <omp.h>
void dgo_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
int dgo_get_threads(void) { return omp_get_max_threads(); }
#else
void dgo_set_threads(int n) { (void)n; }
int dgo_get_threads(void) { return 1; }
#endif
