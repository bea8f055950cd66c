/*
 * CPU oracle for the quantised-inference GEMM path. TEST INFRASTRUCTURE ONLY:
 * this library is the checker for the CUDA kernels and the timed CPU baseline;
 * nothing in the shipped package links, imports or calls it.
 *
 * It restates, in plain C, the arithmetic the reference compiler's emitted
 * kernels perform. Each function names the reference file:line it follows.
 *
 * Pinning status (what fixes the results independently of this file):
 *   - f16 decode, input generator, y_block_cdiv, grouped-raster swizzle:
 *     pinned by the reference's own known-answer tests.
 *   - e4m3 encode/decode, the FP8 and F16 GEMMs with their scale, bias+ReLU and
 *     SwiGLU epilogues, fused add+RMSNorm, RoPE and paged decode attention:
 *     pinned against the reference's own emitted kernels (its PTX fixtures,
 *     assembled unchanged for sm_100a by make_ref.py into _ref/) run on a B200
 *     on the same inputs - bit for bit where the arithmetic is exact (every
 *     e4m3 code, exact-integer GEMMs, the residual stream), by the reference's
 *     own gates elsewhere. Outputs of those kernels recorded on a B200 are
 *     committed with the tests, so the pin also holds without a GPU.
 *     The e4m3 codec is additionally pinned against torch CPU float8_e4m3fn
 *     and the host conversion in cuda_fp8.h over every code and midpoint.
 *   - INT4 group quantise/pack/decode: parity unpinned (the reference has no
 *     INT4 implementation; the format is defined by this file).
 */
#ifndef Y_B200_ORACLE_H
#define Y_B200_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar conversions ------------------------------------------------ */
float    orc_f16_bits_to_f32(uint16_t h);        /* all classes, exact      */
uint16_t orc_f32_to_f16_bits(float f);           /* RNE, overflow -> inf    */
uint16_t orc_f32_to_bf16_bits(float f);          /* RNE (+0x7FFF + bit16)   */
float    orc_bf16_bits_to_f32(uint16_t b);
uint8_t  orc_e4m3_encode(float x);               /* RNE, satfinite          */
float    orc_e4m3_decode(uint8_t code);

/* ---- deterministic inputs ---------------------------------------------- */
uint64_t orc_splitmix64(uint64_t index, uint64_t seed);
uint16_t orc_random_f16_bits(uint64_t index, uint64_t seed);
void     orc_fill_random_f16(uint16_t* out, size_t n, uint64_t seed);
/* N(0, std) rounded to f16; element i depends only on (i + index0, seed).  */
void     orc_fill_normal_f16(uint16_t* out, size_t n, uint64_t index0,
                             uint64_t seed, float std);
/* U(lo, hi) rounded to f16. */
void     orc_fill_uniform_f16(uint16_t* out, size_t n, uint64_t index0,
                              uint64_t seed, float lo, float hi);

/* ---- integer helpers ---------------------------------------------------- */
uint32_t orc_block_cdiv(uint32_t a, uint32_t b);
/* Grouped-raster remap of a raw CTA id; writes (n_tile, m_tile).           */
void     orc_grid_swizzle(uint32_t bid_x, uint32_t bid_y, uint32_t gdim_x,
                          uint32_t gdim_y, uint32_t group,
                          uint32_t* out_n, uint32_t* out_m);

/* ---- FP8 quantisation --------------------------------------------------- */
float orc_amax_f16(const uint16_t* x, size_t n);
float orc_amax_f32(const float* x, size_t n);
float orc_scale_from_amax(float amax);            /* max(amax/448, 1e-12)    */
void  orc_quantize_fp8_f16(const uint16_t* x, size_t n, float scale, uint8_t* q);
void  orc_quantize_fp8_f32(const float* x, size_t n, float scale, uint8_t* q);
/* x is [rows, cols] row-major; q is [cols, rows] row-major.                */
void  orc_quantize_fp8_f16_transpose(const uint16_t* x, size_t rows, size_t cols,
                                     float scale, uint8_t* q);

/* ---- RMSNorm -> FP8 prologue ------------------------------------------- */
/* y = (x * rstd) * gamma, rstd = 1/sqrt(mean(x^2) + eps); sum of squares is
 * taken in the fixed order documented in oracle.c so it is reproducible.
 * y_out (optional) receives the f32 normalised rows; returns amax(|y|).    */
float orc_rmsnorm_f16(const uint16_t* x, const uint16_t* gamma, size_t rows,
                      size_t hidden, float eps, float* y_out, float* rstd_out);
void  orc_rmsnorm_residual_f16(const uint16_t* x, const uint16_t* residual, const uint16_t* weight,
                                size_t rows, size_t hidden, float eps, uint16_t* out,
                                uint16_t* new_residual);
void  orc_rope_inv_freq(int head_dim, float base, float* inv_freq);
void  orc_rope_f16(const uint16_t* x, const int32_t* positions, size_t rows, int head_dim, float base,
                   uint16_t* out);
void  orc_paged_decode_attention(const uint16_t* q, const uint16_t* kcache, const uint16_t* vcache,
                                 const int32_t* page_table, const int32_t* seq_lens, int num_seqs,
                                 int num_q_heads, int num_kv_heads, int head_dim, int page_size,
                                 int max_pages, uint16_t* out);
void  orc_rmsnorm_quantize_fp8(const uint16_t* x, const uint16_t* gamma,
                               size_t rows, size_t hidden, float eps,
                               uint8_t* q, float* scale_out);

/* ---- FP8 GEMM + epilogues ---------------------------------------------- */
enum { ORC_EPI_NONE = 0, ORC_EPI_BIAS = 1, ORC_EPI_BIAS_RELU = 2, ORC_EPI_SWIGLU = 3,
       ORC_EPI_BIAS_GELU = 4, ORC_EPI_BIAS_SILU = 5 };  /* bias may be absent for 4 and 5 */
enum { ORC_OUT_F32 = 0, ORC_OUT_F16 = 1, ORC_OUT_BF16 = 2 };
enum { ORC_BIAS_NONE = 0, ORC_BIAS_F16 = 1, ORC_BIAS_F32 = 2 };

/* C[r, :] for r in [row_begin, row_begin + row_count): Aq is [M, K] e4m3,
 * BqT is [N, K] e4m3 (B stored K-major). out has row_count rows.
 * For ORC_EPI_SWIGLU the N columns are gate|up interleaved (2j = gate,
 * 2j+1 = up) and out has N/2 columns.                                      */
void orc_gemm_fp8(const uint8_t* Aq, const uint8_t* BqT, size_t M, size_t N,
                  size_t K, float scale_a, float scale_b, const void* bias,
                  int bias_kind, int epilogue, int out_kind, void* out,
                  size_t row_begin, size_t row_count);

void orc_decode_e4m3(const uint8_t* q, size_t n, float* out);
void orc_gemm_fp8_decoded(const uint8_t* Aq, const float* Bf, size_t M, size_t N, size_t K,
                          float scale_a, float scale_b, const void* bias, int bias_kind,
                          int epilogue, int out_kind, void* out, size_t row_begin,
                          size_t row_count);

/* Requantise a bf16 tensor to e4m3 with a fresh per-tensor scale.          */
void orc_requant_bf16_fp8(const uint16_t* h_bf16, size_t n, uint8_t* q,
                          float* scale_out);

/* ---- INT4 weight-only path --------------------------------------------- */
/* w is [K, N] f16 row-major. qweight is [K/8, N] u32 (nibble j of word
 * [kw, n] holds element k = 8*kw + j, two's complement). scales is
 * [K/group, N] f16.                                                         */
void orc_int4_quantize(const uint16_t* w, size_t K, size_t N, size_t group,
                       uint32_t* qweight, uint16_t* scales);
size_t orc_int4_stream_bytes(size_t K, size_t N);
void orc_int4_repack(const uint32_t* qweight, const uint16_t* scales, size_t K,
                     size_t N, uint8_t* stream);
void orc_gemm_int4_decode(const uint16_t* x, const uint32_t* qweight,
                          const uint16_t* scales, size_t M, size_t N, size_t K,
                          size_t group, uint16_t* out_f16);

/* ---- F16-operand GEMM (the reference's gemm_f16_* family) --------------- */
/* A [M,K] f16, Bt [N,K] f16 (K-major), f32 accumulate.                      */
void orc_gemm_f16(const uint16_t* A, const uint16_t* Bt, size_t M, size_t N,
                  size_t K, const void* bias, int bias_kind, int epilogue,
                  int out_kind, void* out, size_t row_begin, size_t row_count);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
