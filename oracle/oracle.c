/*
 * CPU oracle for the quantised-inference GEMM path (see oracle.h for the
 * role and the pinning status). TEST INFRASTRUCTURE ONLY.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared (see Makefile).
 * -ffp-contract=off matters: the quantisers are specified as separate IEEE
 * f32 operations (multiply, then convert), never fused.
 *
 * Reference files are cited by their path inside the reference project.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------
 * Scalar conversions
 * ---------------------------------------------------------------------- */

/* binary16 -> f32. The reference decodes normals only
 * (src/cuda_runtime.rs:648-655: sign<<31 | (exp+112)<<23 | mant<<13); this
 * is the same mapping extended to zero, subnormals, inf and NaN. */
float orc_f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u;
    uint32_t exp = (uint32_t)(h >> 10) & 0x1fu;
    uint32_t mant = (uint32_t)h & 0x3ffu;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign << 31);
        float v = (float)mant * (1.0f / 16777216.0f); /* mant * 2^-24, exact */
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32((sign << 31) | 0x7f800000u | (mant << 13));
    return bits_f32((sign << 31) | ((exp + 112u) << 23) | (mant << 13));
}

/* f32 -> binary16, round to nearest even; overflow goes to infinity. */
uint16_t orc_f32_to_f16_bits(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t absu = u & 0x7fffffffu;
    if (absu >= 0x7f800000u) /* inf / NaN */
        return (uint16_t)(sign | 0x7c00u | ((absu > 0x7f800000u) ? 0x200u : 0u));
    if (absu >= 0x477ff000u) /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    if (absu < 0x38800000u) { /* below the smallest normal 2^-14 */
        if (absu < 0x33000000u) return (uint16_t)sign; /* < 2^-25 -> 0 */
        /* Subnormal: value = m * 2^-24 with m rounded to nearest even. */
        float scaled = bits_f32(absu) * 16777216.0f; /* exact: * 2^24 */
        float r = nearbyintf(scaled);               /* ties to even    */
        return (uint16_t)(sign | (uint32_t)r);
    }
    uint32_t exp = (absu >> 23) - 112u;
    uint32_t mant = absu & 0x7fffffu;
    uint32_t half = (exp << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}

/* f32 -> bf16, round to nearest even by adding 0x7FFF + bit 16 and taking
 * the high half (src/quantization_pass.rs:353-370). NaN is quieted. */
uint16_t orc_f32_to_bf16_bits(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t bit16 = (u >> 16) & 1u;
    u += 0x7fffu + bit16;
    return (uint16_t)(u >> 16);
}

float orc_bf16_bits_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* e4m3 (4 exponent bits, bias 7, 3 mantissa bits, no infinity; S.1111.111 is
 * NaN; max finite 448 = 0x7E). */
float orc_e4m3_decode(uint8_t code) {
    uint32_t sign = code >> 7;
    uint32_t exp = (code >> 3) & 0xfu;
    uint32_t mant = code & 7u;
    float v;
    if (exp == 0xf && mant == 7) return bits_f32(0x7fc00000u | (sign << 31));
    if (exp == 0) v = (float)mant * (1.0f / 512.0f);          /* m * 2^-9 */
    else v = ldexpf((float)(8 + mant), (int)exp - 10);        /* (1+m/8)*2^(e-7) */
    return sign ? -v : v;
}

/* f32 -> e4m3, round to nearest even, saturate to +-448, NaN -> 0x7F|sign.
 * This is what `cvt.rn.satfinite.e4m3x2.f32` does per element
 * (src/ptx_emitter.rs:2595-2658). */
uint8_t orc_e4m3_encode(float x) {
    uint32_t u = f32_bits(x);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t absu = u & 0x7fffffffu;
    if (absu > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
    float a = bits_f32(absu);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7eu); /* includes inf */
    if (a < 0.015625f) { /* below 2^-6: subnormal grid, step 2^-9 */
        float r = nearbyintf(a * 512.0f); /* exact scaling, ties to even */
        return (uint8_t)(sign | (uint8_t)r); /* r == 8 is code 0x08 = 2^-6 */
    }
    /* Normal: keep 3 mantissa bits. */
    uint32_t exp = (absu >> 23);           /* biased f32 exponent, >= 121 */
    uint32_t mant = absu & 0x7fffffu;
    uint32_t code = ((exp - 120u) << 3) | (mant >> 20);
    uint32_t rem = mant & 0xfffffu;
    if (rem > 0x80000u || (rem == 0x80000u && (code & 1u))) code++;
    if (code > 0x7eu) code = 0x7eu; /* 464..480 would round up past 448 */
    return (uint8_t)(sign | code);
}

/* ------------------------------------------------------------------------
 * Deterministic inputs
 * ---------------------------------------------------------------------- */

/* splitmix64 keyed by (index, seed) (src/cuda_runtime.rs:668-676). */
uint64_t orc_splitmix64(uint64_t index, uint64_t seed) {
    uint64_t z = index * 0x9E3779B97F4A7C15ull + seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

/* Normal binary16 with exponent in 12..14, i.e. |v| in [2^-3, 1)
 * (src/cuda_runtime.rs:677-682). */
uint16_t orc_random_f16_bits(uint64_t index, uint64_t seed) {
    uint64_t z = orc_splitmix64(index, seed);
    uint16_t sign = (uint16_t)((z >> 63) & 1u);
    uint16_t exp = (uint16_t)(12u + (uint16_t)((z >> 40) & 0x3u) % 3u);
    uint16_t mant = (uint16_t)(z & 0x3ffu);
    return (uint16_t)((sign << 15) | (exp << 10) | mant);
}

void orc_fill_random_f16(uint16_t* out, size_t n, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = orc_random_f16_bits((uint64_t)i, seed);
}

/* Box-Muller on the two 32-bit halves of splitmix64(index, seed), evaluated
 * in double so the f16 result does not depend on the libm's last bit. */
void orc_fill_normal_f16(uint16_t* out, size_t n, uint64_t index0, uint64_t seed, float std) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint64_t z = orc_splitmix64(index0 + (uint64_t)i, seed);
        double u1 = ((double)(uint32_t)(z >> 32) + 1.0) * (1.0 / 4294967296.0); /* (0,1] */
        double u2 = (double)(uint32_t)z * (1.0 / 4294967296.0);                 /* [0,1) */
        double g = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
        out[i] = orc_f32_to_f16_bits((float)(g * (double)std));
    }
}

void orc_fill_uniform_f16(uint16_t* out, size_t n, uint64_t index0, uint64_t seed, float lo, float hi) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint64_t z = orc_splitmix64(index0 + (uint64_t)i, seed);
        double u = (double)(z >> 11) * (1.0 / 9007199254740992.0);
        out[i] = orc_f32_to_f16_bits((float)((double)lo + u * ((double)hi - (double)lo)));
    }
}

/* ------------------------------------------------------------------------
 * Integer helpers
 * ---------------------------------------------------------------------- */

/* src/c_api.rs:196-201. */
uint32_t orc_block_cdiv(uint32_t a, uint32_t b) { return b == 0 ? 0 : (a + b - 1) / b; }

/* Grouped raster: `group` consecutive M tiles are walked column-first; the
 * last group is clamped to the rows that remain (src/ptx_emitter.rs:2222-2284;
 * model at :7449-7461). */
void orc_grid_swizzle(uint32_t bid_x, uint32_t bid_y, uint32_t gdim_x, uint32_t gdim_y,
                      uint32_t group, uint32_t* out_n, uint32_t* out_m) {
    uint32_t tile = bid_y * gdim_x + bid_x;
    uint32_t per_group = gdim_x * group;
    uint32_t gid = tile / per_group;
    uint32_t off = tile % per_group;
    uint32_t first_m = gid * group;
    uint32_t rows = gdim_y - first_m;
    uint32_t gsz = rows < group ? rows : group;
    *out_m = first_m + off % gsz;
    *out_n = off / gsz;
}

/* ------------------------------------------------------------------------
 * FP8 quantisation
 * ---------------------------------------------------------------------- */

float orc_amax_f16(const uint16_t* x, size_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = fabsf(orc_f16_bits_to_f32(x[i]));
        if (v > m) m = v;
    }
    return m;
}

float orc_amax_f32(const float* x, size_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = fabsf(x[i]);
        if (v > m) m = v;
    }
    return m;
}

/* scale = max(amax / 448, 1e-12) in f32
 * (tests/test_fp8_gemm_correctness.py:99-100). */
float orc_scale_from_amax(float amax) {
    float s = amax / 448.0f;
    return s > 1e-12f ? s : 1e-12f;
}

/* q = e4m3_rn_satfinite(x * inv), inv = 1/scale rounded once to f32: the
 * emitted kernel takes rcp.rn.f32 of the scale and multiplies
 * (src/ptx_emitter.rs:3405-3408, 2613-2616). */
void orc_quantize_fp8_f16(const uint16_t* x, size_t n, float scale, uint8_t* q) {
    const float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) q[i] = orc_e4m3_encode(orc_f16_bits_to_f32(x[i]) * inv);
}

void orc_quantize_fp8_f32(const float* x, size_t n, float scale, uint8_t* q) {
    const float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) q[i] = orc_e4m3_encode(x[i] * inv);
}

void orc_quantize_fp8_f16_transpose(const uint16_t* x, size_t rows, size_t cols, float scale,
                                    uint8_t* q) {
    const float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (size_t c = 0; c < cols; ++c)
        for (size_t r = 0; r < rows; ++r)
            q[c * rows + r] = orc_e4m3_encode(orc_f16_bits_to_f32(x[r * cols + c]) * inv);
}

/* ------------------------------------------------------------------------
 * RMSNorm -> FP8 prologue
 *
 * Follows the reference's fused add+RMSNorm math without the residual
 * (src/ptx_emitter.rs:5932-5997): y = h * rsqrt(mean(h^2) + eps) * w in f32.
 * To make the e4m3 codes reproducible bit for bit, the sum of squares has a
 * FIXED order, and rsqrt is the correctly rounded 1/sqrt:
 *   - the row is cut into 8-element vectors; worker t of 256 takes vectors
 *     t, t+256, ... in increasing order and folds each element with
 *     acc = fma(x, x, acc);
 *   - workers are grouped in 8 blocks of 32; inside a block five butterfly
 *     steps (partner = lane ^ 16, 8, 4, 2, 1) add the partials;
 *   - the eight block totals are added in block order;
 *   - mean = total / hidden; rstd = 1 / sqrt(mean + eps) (two IEEE ops).
 * ---------------------------------------------------------------------- */
static float rms_row_sumsq(const uint16_t* x, size_t hidden) {
    float part[256];
    size_t nvec = hidden / 8;
    for (int t = 0; t < 256; ++t) {
        float acc = 0.0f;
        for (size_t v = (size_t)t; v < nvec; v += 256)
            for (int j = 0; j < 8; ++j) {
                float f = orc_f16_bits_to_f32(x[v * 8 + (size_t)j]);
                acc = fmaf(f, f, acc);
            }
        part[t] = acc;
    }
    float total = 0.0f;
    for (int w = 0; w < 8; ++w) {
        float lane[32], next[32];
        memcpy(lane, part + 32 * w, sizeof lane);
        for (int off = 16; off >= 1; off >>= 1) {
            for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ off];
            memcpy(lane, next, sizeof lane);
        }
        total = (w == 0) ? lane[0] : total + lane[0];
    }
    return total;
}

float orc_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, size_t rows, size_t hidden,
                      float eps, float* y_out, float* rstd_out) {
    float amax = 0.0f;
#pragma omp parallel for reduction(max : amax) schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * hidden;
        float total = rms_row_sumsq(xr, hidden);
        float mean = total / (float)hidden;
        float rstd = 1.0f / sqrtf(mean + eps);
        if (rstd_out) rstd_out[r] = rstd;
        for (size_t c = 0; c < hidden; ++c) {
            float y = (orc_f16_bits_to_f32(xr[c]) * rstd) * orc_f16_bits_to_f32(gamma[c]);
            if (y_out) y_out[r * hidden + c] = y;
            float a = fabsf(y);
            if (a > amax) amax = a;
        }
    }
    return amax;
}

void orc_rmsnorm_quantize_fp8(const uint16_t* x, const uint16_t* gamma, size_t rows,
                              size_t hidden, float eps, uint8_t* q, float* scale_out) {
    float* rstd = (float*)malloc(rows * sizeof(float));
    float amax = orc_rmsnorm_f16(x, gamma, rows, hidden, eps, NULL, rstd);
    float scale = orc_scale_from_amax(amax);
    float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < hidden; ++c) {
            float y = (orc_f16_bits_to_f32(x[r * hidden + c]) * rstd[r]) *
                      orc_f16_bits_to_f32(gamma[c]);
            q[r * hidden + c] = orc_e4m3_encode(y * inv);
        }
    if (scale_out) *scale_out = scale;
    free(rstd);
}

/* ------------------------------------------------------------------------
 * Fused add + RMSNorm with the residual stream, f16 in and out
 *
 * Follows emit_rmsnorm_residual_kernel (src/ptx_emitter.rs:5773-6015):
 *   h = f32(x) + f32(residual)                (:5877, h stays f32 for the norm)
 *   total = sum(h^2) over the row
 *   mean = total * f32(1 / hidden)            (:5910, a multiply by the reciprocal)
 *   inv_rms = rsqrt(mean + eps)               (:5914; the reference uses
 *             rsqrt.approx.f32 and fixes eps = 1e-5; here rsqrt is the correctly
 *             rounded 1/sqrt and eps is a parameter, so that results can be pinned)
 *   out = f16_rn((h * inv_rms) * w)           (:5957-5959, two multiplies)
 *   new_residual = f16_rn(h)                  (:6003)
 * The sum of squares uses the same fixed order as the prologue above (worker t of
 * 256 folds vectors t, t+256, ... with fma; butterfly inside blocks of 32; the
 * eight block totals in order); the reference's own order is the same up to
 * whether ptxas fuses its mul+add.
 * ---------------------------------------------------------------------- */
void orc_rmsnorm_residual_f16(const uint16_t* x, const uint16_t* residual, const uint16_t* weight,
                              size_t rows, size_t hidden, float eps, uint16_t* out,
                              uint16_t* new_residual) {
    const float inv_hidden = 1.0f / (float)hidden;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        float* h = (float*)malloc(hidden * sizeof(float));
        for (size_t c = 0; c < hidden; ++c)
            h[c] = orc_f16_bits_to_f32(x[r * hidden + c]) + orc_f16_bits_to_f32(residual[r * hidden + c]);
        float part[256];
        size_t nvec = hidden / 8;
        for (int t = 0; t < 256; ++t) {
            float acc = 0.0f;
            for (size_t v = (size_t)t; v < nvec; v += 256)
                for (int j = 0; j < 8; ++j) acc = fmaf(h[v * 8 + (size_t)j], h[v * 8 + (size_t)j], acc);
            part[t] = acc;
        }
        float total = 0.0f;
        for (int w = 0; w < 8; ++w) {
            float lane[32], next[32];
            memcpy(lane, part + 32 * w, sizeof lane);
            for (int off = 16; off >= 1; off >>= 1) {
                for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ off];
                memcpy(lane, next, sizeof lane);
            }
            total = (w == 0) ? lane[0] : total + lane[0];
        }
        float mean = total * inv_hidden;
        float rstd = 1.0f / sqrtf(mean + eps);
        for (size_t c = 0; c < hidden; ++c) {
            float y = (h[c] * rstd) * orc_f16_bits_to_f32(weight[c]);
            out[r * hidden + c] = orc_f32_to_f16_bits(y);
            new_residual[r * hidden + c] = orc_f32_to_f16_bits(h[c]);
        }
        free(h);
    }
}

/* ------------------------------------------------------------------------
 * Rotary position embedding, interleaved pairs (2i, 2i+1), f16 in and out
 *
 * Follows emit_rope_kernel (src/ptx_emitter.rs:6046-6260):
 *   theta_i = f32(pos) * inv_freq_i in f32,  inv_freq_i = base^(-2i/head_dim)
 *   out[2i]   = fl(fl(x0*cos) - fl(x1*sin)),  out[2i+1] = fl(fl(x0*sin) + fl(x1*cos))
 * one position per row (Positions[row], i32). The reference gets inv_freq from
 * ex2.approx and the trig from sin.approx / cos.approx; here inv_freq_i is the f32
 * rounding of the double-precision power (the library passes the same table to its
 * kernel) and sin/cos are those of the f32 theta evaluated in double precision, so the
 * only device-side freedom left is the last bit of sin/cos.
 * ---------------------------------------------------------------------- */
void orc_rope_inv_freq(int head_dim, float base, float* inv_freq) {
    for (int i = 0; i < head_dim / 2; ++i)
        inv_freq[i] = (float)pow((double)base, -2.0 * (double)i / (double)head_dim);
}

void orc_rope_f16(const uint16_t* x, const int32_t* positions, size_t rows, int head_dim, float base,
                  uint16_t* out) {
    float inv_freq[1024];
    orc_rope_inv_freq(head_dim, base, inv_freq);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const float pos = (float)positions[r];
        for (int i = 0; i < head_dim / 2; ++i) {
            const float theta = pos * inv_freq[i];
            const float s = (float)sin((double)theta), c = (float)cos((double)theta);
            const float x0 = orc_f16_bits_to_f32(x[r * (size_t)head_dim + 2 * (size_t)i]);
            const float x1 = orc_f16_bits_to_f32(x[r * (size_t)head_dim + 2 * (size_t)i + 1]);
            const float a = x0 * c, b = x1 * s, d = x0 * s, e = x1 * c;
            out[r * (size_t)head_dim + 2 * (size_t)i] = orc_f32_to_f16_bits(a - b);
            out[r * (size_t)head_dim + 2 * (size_t)i + 1] = orc_f32_to_f16_bits(d + e);
        }
    }
}

/* ------------------------------------------------------------------------
 * Paged decode attention
 *
 * The definition the reference kernel implements and its benchmark checks against
 * (src/ptx_emitter.rs:6303-6345, tests/benchmark_y_paged_decode_attention.py:159-185):
 * for sequence s and query head h, with kv head h / (q_heads / kv_heads) and tokens
 * t < seq_lens[s] found at KCache[PageTable[s][t / page], t % page, kv head, :]:
 *   score_t = (q . k_t) / sqrt(head_dim);  p = softmax(score);  out = sum_t p_t v_t.
 * Evaluated in double precision and rounded once to f16; length 0 gives zeros. The
 * device kernel accumulates in f32 with online softmax and f16 probabilities, so the
 * comparison is by tolerance.
 * ---------------------------------------------------------------------- */
void orc_paged_decode_attention(const uint16_t* q, const uint16_t* kcache, const uint16_t* vcache,
                                const int32_t* page_table, const int32_t* seq_lens, int num_seqs,
                                int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                                int max_pages, uint16_t* out) {
    const int group = num_q_heads / num_kv_heads;
    const double scale = 1.0 / sqrt((double)head_dim);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int s = 0; s < num_seqs; ++s)
        for (int h = 0; h < num_q_heads; ++h) {
            /* lengths are clamped to what the page table can address, as the device kernel does */
            int len = seq_lens[s] < 0 ? 0 : seq_lens[s];
            if ((long long)len > (long long)max_pages * page_size) len = max_pages * page_size;
            const int kvh = h / group;
            uint16_t* o = out + ((size_t)s * num_q_heads + h) * head_dim;
            if (len <= 0) {
                for (int d = 0; d < head_dim; ++d) o[d] = 0;
                continue;
            }
            const uint16_t* qv = q + ((size_t)s * num_q_heads + h) * head_dim;
            double* score = (double*)malloc((size_t)len * sizeof(double));
            double* acc = (double*)calloc((size_t)head_dim, sizeof(double));
            double mx = -1e300;
            for (int t = 0; t < len; ++t) {
                const size_t row = (((size_t)page_table[(size_t)s * max_pages + t / page_size] * page_size +
                                     (size_t)(t % page_size)) * num_kv_heads + kvh) * head_dim;
                double dot = 0.0;
                for (int d = 0; d < head_dim; ++d)
                    dot += (double)orc_f16_bits_to_f32(qv[d]) * (double)orc_f16_bits_to_f32(kcache[row + d]);
                score[t] = dot * scale;
                if (score[t] > mx) mx = score[t];
            }
            double denom = 0.0;
            for (int t = 0; t < len; ++t) {
                const size_t row = (((size_t)page_table[(size_t)s * max_pages + t / page_size] * page_size +
                                     (size_t)(t % page_size)) * num_kv_heads + kvh) * head_dim;
                const double pexp = exp(score[t] - mx);
                denom += pexp;
                for (int d = 0; d < head_dim; ++d) acc[d] += pexp * (double)orc_f16_bits_to_f32(vcache[row + d]);
            }
            for (int d = 0; d < head_dim; ++d) o[d] = orc_f32_to_f16_bits((float)(acc[d] / denom));
            free(score);
            free(acc);
        }
}

/* ------------------------------------------------------------------------
 * GEMM + epilogues
 * ---------------------------------------------------------------------- */

/* Dot product with f32 accumulation in 16 independent lanes, folded in lane
 * order at the end. Products of two e4m3 (or two f16) values are exact in
 * f32, so only the summation order separates this from any other f32
 * accumulator; the 16-lane order lets the compiler vectorise it. */
static float dot_f32(const float* a, const float* b, size_t k) {
    float acc[16] = {0};
    size_t i = 0;
    for (; i + 16 <= k; i += 16)
        for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
    for (; i < k; ++i) acc[i & 15] += a[i] * b[i];
    float s = 0.0f;
    for (int j = 0; j < 16; ++j) s += acc[j];
    return s;
}

static float bias_at(const void* bias, int kind, size_t col) {
    if (kind == ORC_BIAS_F16) return orc_f16_bits_to_f32(((const uint16_t*)bias)[col]);
    if (kind == ORC_BIAS_F32) return ((const float*)bias)[col];
    return 0.0f;
}

static void store_out(void* out, int kind, size_t idx, float v) {
    if (kind == ORC_OUT_F32) ((float*)out)[idx] = v;
    else if (kind == ORC_OUT_F16) ((uint16_t*)out)[idx] = orc_f32_to_f16_bits(v);
    else ((uint16_t*)out)[idx] = orc_f32_to_bf16_bits(v);
}

/* silu(g) * u with silu(g) = g * 1/(1 + exp(-g)), all f32
 * (src/ptx_emitter.rs:5537-5552; the emitted kernel uses ex2.approx and
 * rcp.approx, this uses the libm exp and a true division). */
static float swiglu(float g, float u) {
    float sig = 1.0f / (1.0f + expf(-g));
    return (g * sig) * u;
}

/* The reference's fused GELU (src/quantization_pass.rs:748-796): 0.5 x (1 + tanh(x * p)) with
 * p = fma(x^2, 0.044715, 0.79788456) exactly as its emitter writes it (the cubic coefficient
 * is not multiplied by sqrt(2/pi) there), all f32; the emitted code uses tanh.approx. */
static float gelu_ref(float x) {
    float p = fmaf(x * x, 0.044715f, 0.79788456f);
    return (0.5f * x) * (1.0f + tanhf(x * p));
}

/* silu(x) = x * 1/(1 + exp(-x)) (src/quantization_pass.rs:716-747). */
static float silu_ref(float x) { return x * (1.0f / (1.0f + expf(-x))); }

static void epilogue_row(const float* acc, size_t N, float scale, const void* bias,
                         int bias_kind, int epilogue, int out_kind, void* out, size_t out_row) {
    if (epilogue == ORC_EPI_SWIGLU) {
        size_t half = N / 2;
        for (size_t j = 0; j < half; ++j) {
            float g = acc[2 * j] * scale, u = acc[2 * j + 1] * scale;
            store_out(out, out_kind, out_row * half + j, swiglu(g, u));
        }
        return;
    }
    for (size_t c = 0; c < N; ++c) {
        /* C = acc * (sa*sb): the scale product is formed once and applied
         * after the sum (src/ptx_emitter.rs:3532-3566). */
        float v = acc[c] * scale;
        if (epilogue == ORC_EPI_BIAS || epilogue == ORC_EPI_BIAS_RELU ||
            ((epilogue == ORC_EPI_BIAS_GELU || epilogue == ORC_EPI_BIAS_SILU) && bias != NULL))
            v = v + bias_at(bias, bias_kind, c);                 /* :4804-4806 */
        if (epilogue == ORC_EPI_BIAS_RELU) v = v > 0.0f ? v : 0.0f; /* :4807-4808 */
        if (epilogue == ORC_EPI_BIAS_GELU) v = gelu_ref(v);
        if (epilogue == ORC_EPI_BIAS_SILU) v = silu_ref(v);
        store_out(out, out_kind, out_row * N + c, v);
    }
}

void orc_decode_e4m3(const uint8_t* q, size_t n, float* out) {
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_decode((uint8_t)i);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) out[i] = lut[q[i]];
}

/* Same as orc_gemm_fp8 with the weight operand already decoded to f32
 * (Bf = orc_decode_e4m3(BqT)): lets a caller that reuses one weight matrix
 * for many calls pay for the decode once. */
void orc_gemm_fp8_decoded(const uint8_t* Aq, const float* Bf, size_t M, size_t N, size_t K,
                          float scale_a, float scale_b, const void* bias, int bias_kind,
                          int epilogue, int out_kind, void* out, size_t row_begin,
                          size_t row_count) {
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_decode((uint8_t)i);
    if (row_begin + row_count > M) row_count = M > row_begin ? M - row_begin : 0;
    const float scale = scale_a * scale_b;
    /* Blocks of 32 rows: the decoded A block stays in cache while each weight
     * row is streamed once per block instead of once per output row. Every
     * output is still the same dot_f32 of the same two vectors. */
    enum { RB = 32 };
    float* ablk = (float*)malloc((size_t)RB * K * sizeof(float));
    float* acc = (float*)malloc((size_t)RB * N * sizeof(float));
    for (size_t r0 = 0; r0 < row_count; r0 += RB) {
        const size_t nr = row_count - r0 < RB ? row_count - r0 : RB;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < nr * K; ++i) ablk[i] = lut[Aq[(row_begin + r0) * K + i]];
#pragma omp parallel for schedule(static)
        for (size_t c = 0; c < N; ++c)
            for (size_t r = 0; r < nr; ++r) acc[r * N + c] = dot_f32(ablk + r * K, Bf + c * K, K);
#pragma omp parallel for schedule(static)
        for (size_t r = 0; r < nr; ++r)
            epilogue_row(acc + r * N, N, scale, bias, bias_kind, epilogue, out_kind, out, r0 + r);
    }
    free(ablk);
    free(acc);
}

void orc_gemm_fp8(const uint8_t* Aq, const uint8_t* BqT, size_t M, size_t N, size_t K,
                  float scale_a, float scale_b, const void* bias, int bias_kind, int epilogue,
                  int out_kind, void* out, size_t row_begin, size_t row_count) {
    float* Bf = (float*)malloc(N * K * sizeof(float));
    orc_decode_e4m3(BqT, N * K, Bf);
    orc_gemm_fp8_decoded(Aq, Bf, M, N, K, scale_a, scale_b, bias, bias_kind, epilogue, out_kind,
                         out, row_begin, row_count);
    free(Bf);
}

void orc_gemm_f16(const uint16_t* A, const uint16_t* Bt, size_t M, size_t N, size_t K,
                  const void* bias, int bias_kind, int epilogue, int out_kind, void* out,
                  size_t row_begin, size_t row_count) {
    if (row_begin + row_count > M) row_count = M > row_begin ? M - row_begin : 0;
    float* Bf = (float*)malloc(N * K * sizeof(float));
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < N * K; ++i) Bf[i] = orc_f16_bits_to_f32(Bt[i]);
#pragma omp parallel
    {
        float* arow = (float*)malloc(K * sizeof(float));
        float* acc = (float*)malloc(N * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (size_t r = 0; r < row_count; ++r) {
            const uint16_t* a = A + (row_begin + r) * K;
            for (size_t k = 0; k < K; ++k) arow[k] = orc_f16_bits_to_f32(a[k]);
            for (size_t c = 0; c < N; ++c) acc[c] = dot_f32(arow, Bf + c * K, K);
            epilogue_row(acc, N, 1.0f, bias, bias_kind, epilogue, out_kind, out, r);
        }
        free(arow);
        free(acc);
    }
    free(Bf);
}

/* amax over a bf16 tensor is order independent, so the fresh scale is exact;
 * q = e4m3(h * (1/scale)). */
void orc_requant_bf16_fp8(const uint16_t* h, size_t n, uint8_t* q, float* scale_out) {
    float amax = 0.0f;
#pragma omp parallel for reduction(max : amax) schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = fabsf(orc_bf16_bits_to_f32(h[i]));
        if (v > amax) amax = v;
    }
    float scale = orc_scale_from_amax(amax);
    float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) q[i] = orc_e4m3_encode(orc_bf16_bits_to_f32(h[i]) * inv);
    if (scale_out) *scale_out = scale;
}

/* ------------------------------------------------------------------------
 * INT4 weight-only path. The reference has no INT4 implementation
 * (src/ptx_emitter.rs:7321-7330 is a dead stub), so this file DEFINES the
 * format: symmetric, groups of `group` along K, s = f16_rn(amax_g / 7),
 * q = clamp(rne(w / float(s)), -8, 7) (0 when s == 0), two's-complement
 * nibbles, element k = 8*kw + j in nibble j of word [kw, n] (low to high,
 * the same order the reference packs e4m3 bytes, src/ptx_emitter.rs:2622-2657).
 * ---------------------------------------------------------------------- */
void orc_int4_quantize(const uint16_t* w, size_t K, size_t N, size_t group, uint32_t* qweight,
                       uint16_t* scales) {
    size_t ngroups = K / group;
#pragma omp parallel for schedule(static)
    for (size_t n = 0; n < N; ++n) {
        for (size_t g = 0; g < ngroups; ++g) {
            float amax = 0.0f;
            for (size_t k = g * group; k < (g + 1) * group; ++k) {
                float v = fabsf(orc_f16_bits_to_f32(w[k * N + n]));
                if (v > amax) amax = v;
            }
            uint16_t sbits = orc_f32_to_f16_bits(amax / 7.0f);
            scales[g * N + n] = sbits;
            float s = orc_f16_bits_to_f32(sbits);
            for (size_t kw = g * group / 8; kw < (g + 1) * group / 8; ++kw) {
                uint32_t word = 0;
                for (int j = 0; j < 8; ++j) {
                    float v = orc_f16_bits_to_f32(w[(kw * 8 + (size_t)j) * N + n]);
                    int q = 0;
                    if (s > 0.0f) {
                        float r = nearbyintf(v / s);
                        if (r > 7.0f) r = 7.0f;
                        if (r < -8.0f) r = -8.0f;
                        q = (int)r;
                    }
                    word |= ((uint32_t)q & 0xfu) << (4 * j);
                }
                qweight[kw * N + n] = word;
            }
        }
    }
}

/* Streaming layout consumed by the decode kernel. One 1056-byte block per
 * (16-column tile, 128-row group), tiles outermost:
 *   bytes [0,1024): for half h in {0,1}, lane in 0..31, a 16-byte unit of
 *     four words. With gq = lane/4, c = lane%4, unit word i holds the eight
 *     K-consecutive weights k = 128*g + 32*(2h + i/2) + 8c + (0..7) of column
 *     16*tile + gq + 8*(i%2), stored offset-binary (q + 8) with logical
 *     element j at nibble position {0,4,1,5,2,6,3,7}[j];
 *   bytes [1024,1056): the 16 f16 group scales of the tile's columns.
 * Requires K % 128 == 0 and N % 16 == 0. */
size_t orc_int4_stream_bytes(size_t K, size_t N) { return (N / 16) * (K / 128) * 1056; }

void orc_int4_repack(const uint32_t* qweight, const uint16_t* scales, size_t K, size_t N,
                     uint8_t* stream) {
    static const int pos[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    size_t ngroups = K / 128, ntiles = N / 16;
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < ntiles; ++t)
        for (size_t g = 0; g < ngroups; ++g) {
            uint8_t* blk = stream + (t * ngroups + g) * 1056;
            for (int h = 0; h < 2; ++h)
                for (int lane = 0; lane < 32; ++lane) {
                    int gq = lane / 4, c = lane % 4;
                    uint32_t unit[4];
                    for (int i = 0; i < 4; ++i) {
                        size_t kw = g * 16 + (size_t)(4 * (2 * h + i / 2) + c);
                        size_t col = t * 16 + (size_t)(gq + 8 * (i % 2));
                        uint32_t src = qweight[kw * N + col] ^ 0x88888888u;
                        uint32_t dst = 0;
                        for (int j = 0; j < 8; ++j) dst |= ((src >> (4 * j)) & 0xfu) << (4 * pos[j]);
                        unit[i] = dst;
                    }
                    memcpy(blk + h * 512 + lane * 16, unit, 16);
                }
            memcpy(blk + 1024, scales + g * N + t * 16, 32);
        }
}

/* out[m, n] = f16_rn( sum_g float(s[g, n]) * (sum_{k in g} q[k, n] * x[m, k]) ),
 * f32 accumulation; the group scale is applied to the group's partial sum. */
void orc_gemm_int4_decode(const uint16_t* x, const uint32_t* qweight, const uint16_t* scales,
                          size_t M, size_t N, size_t K, size_t group, uint16_t* out) {
    float* xf = (float*)malloc(M * K * sizeof(float));
    for (size_t i = 0; i < M * K; ++i) xf[i] = orc_f16_bits_to_f32(x[i]);
    size_t ngroups = K / group;
#pragma omp parallel for schedule(static)
    for (size_t n = 0; n < N; ++n) {
        float* wq = (float*)malloc(K * sizeof(float));
        for (size_t kw = 0; kw < K / 8; ++kw) {
            uint32_t word = qweight[kw * N + n];
            for (int j = 0; j < 8; ++j) {
                int q = (int)((word >> (4 * j)) & 0xfu);
                if (q >= 8) q -= 16;
                wq[kw * 8 + (size_t)j] = (float)q;
            }
        }
        for (size_t m = 0; m < M; ++m) {
            float acc = 0.0f;
            for (size_t g = 0; g < ngroups; ++g) {
                float part = dot_f32(xf + m * K + g * group, wq + g * group, group);
                acc += orc_f16_bits_to_f32(scales[g * N + n]) * part;
            }
            out[m * N + n] = orc_f32_to_f16_bits(acc);
        }
        free(wq);
    }
    free(xf);
}
