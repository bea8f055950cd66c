/*
 * liby_b200 - C ABI of the B200 (sm_100a) quantised-inference GEMM path.
 *
 * Plain pointers and sizes only. Every device pointer is a CUDA device
 * address of the current device; `stream` is a cudaStream_t passed as void*
 * (NULL = the default stream). Functions return 0 on success or a negative
 * Y_B200_ERR_* code; y_b200_last_error() gives the message for the calling
 * thread. No entry point falls back to the CPU.
 *
 * Each block names the reference interface it replaces (path inside the
 * reference project : line).
 */
#ifndef Y_B200_H
#define Y_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define Y_B200_API __attribute__((visibility("default")))
#else
#define Y_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- errors --------------------------------------------------------------- */
#define Y_B200_OK 0
#define Y_B200_ERR_INVALID (-1)     /* null pointer, bad enum, bad size        */
#define Y_B200_ERR_SHAPE (-2)       /* shape precondition violated              */
#define Y_B200_ERR_ALIGN (-3)       /* pointer or stride alignment              */
#define Y_B200_ERR_CUDA (-4)        /* a CUDA call failed                       */
#define Y_B200_ERR_WORKSPACE (-5)   /* workspace missing or too small           */
#define Y_B200_ERR_DEVICE (-6)      /* device reported a bounded-wait timeout   */
#define Y_B200_ERR_UNSUPPORTED (-7) /* not an sm_100 device, unknown kernel ... */

#define Y_B200_DEV_WAIT_TIMEOUT 1u

Y_B200_API const char* y_b200_last_error(void);
Y_B200_API const char* y_b200_version(void);
/* Reads and clears the device status word that kernels with bounded waits
 * write when a wait runs out. Returns 0 when clean, else Y_B200_ERR_DEVICE
 * with details in y_b200_last_error(). Synchronises `stream`. */
Y_B200_API int y_b200_device_status(void* stream);
/* Exercises that path without any fault: launches one small CTA that waits, for at most
 * `cycles` SM cycles, on a barrier nothing completes, lets the wait run out and records it
 * like a GEMM role would. The kernel returns normally; the next y_b200_device_status
 * reports Y_B200_ERR_DEVICE (role 0x7e57) and clears the word. */
Y_B200_API int y_b200_selftest_bounded_wait(unsigned long long cycles, void* stream);

/* ---- element kinds ---------------------------------------------------------- */
enum { Y_B200_F32 = 0, Y_B200_F16 = 1, Y_B200_BF16 = 2, Y_B200_E4M3 = 3 };
/* The reference's activation functor set (src/quantization_pass.rs:667-798: None, ReLU, GELU,
 * SiLU) plus the gated SwiGLU. GELU is the reference's own tanh form,
 * 0.5 x (1 + tanh(x (0.79788456 + 0.044715 x^2))); SiLU is x / (1 + exp(-x)). For BIAS_GELU and
 * BIAS_SILU the bias pointer may be NULL (no bias). */
enum { Y_B200_EPI_NONE = 0, Y_B200_EPI_BIAS = 1, Y_B200_EPI_BIAS_RELU = 2, Y_B200_EPI_SWIGLU = 3,
       Y_B200_EPI_BIAS_GELU = 4, Y_B200_EPI_BIAS_SILU = 5 };

/* ---- FP8 quantisation -------------------------------------------------------
 * Replaces the quantise+stage loops fused into the reference's FP8 GEMM
 * (src/ptx_emitter.rs:2595-2658 emit_fp8_quantize_pair / emit_fp8_pack_quad,
 * :2693-3053 stage_a/_b) and the host-side amax
 * (tests/test_fp8_gemm_correctness.py:99-100): q = e4m3_rn_satfinite(x * (1/scale)),
 * scale = max(amax/448, 1e-12), element i in byte i. */

/* amax_out: one device float; overwritten with max|x|. */
Y_B200_API int y_b200_amax(const void* x, int x_kind, size_t n, float* amax_out, void* stream);
/* scale_out[0] = max(amax[0]/448, 1e-12) (device to device). */
Y_B200_API int y_b200_scale_from_amax(const float* amax, float* scale_out, void* stream);
/* Static scale: q = e4m3(x * (1/scale[0])); scale is a device float. */
Y_B200_API int y_b200_quantize_fp8(const void* x, int x_kind, size_t n, const float* scale, void* q,
                        void* stream);
/* x is [rows, cols] row-major, q is [cols, rows] row-major (used to store the
 * reference's row-major B [K, N] as K-major [N, K] for the tensor cores). */
Y_B200_API int y_b200_quantize_fp8_transpose(const void* x, int x_kind, size_t rows, size_t cols,
                                  const float* scale, void* q, void* stream);
/* Dynamic per-tensor: amax pass, then quantise; scale_out (device float)
 * receives the scale. transpose != 0 writes q as [cols, rows]. */
Y_B200_API int y_b200_quantize_fp8_dynamic(const void* x, int x_kind, size_t rows, size_t cols,
                                int transpose, void* q, float* scale_out, void* stream);

/* ---- RMSNorm -> FP8 prologue -----------------------------------------------
 * Replaces rmsnorm_residual_<H> (src/ptx_emitter.rs:5773-6015) for the
 * column-parallel GEMM's A operand: no residual, runtime eps, output
 * quantised to e4m3 with a fresh per-tensor scale. hidden % 8 == 0.
 * workspace: y_b200_rmsnorm_workspace_bytes(rows) bytes of device memory. */
Y_B200_API size_t y_b200_rmsnorm_workspace_bytes(size_t rows);
Y_B200_API int y_b200_rmsnorm_quantize_fp8(const void* x_f16, const void* gamma_f16, size_t rows,
                                size_t hidden, float eps, void* q, float* scale_out,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ---- FP8 GEMM ---------------------------------------------------------------
 * Replaces gemm_fp8_<tag> (src/ptx_emitter.rs:3282-3580, entry
 * tests/gemm_fp8_256.ptx:5-11) and y_fp8_tensor_core_gemm_kernel
 * (tests/y_tensor_core_gemm.cu:4152-4159) with its fused epilogues
 * (src/ptx_emitter.rs:3530-3577 scale, :4729-4814 bias+ReLU,
 * :5481-5565 SwiGLU).
 *   C = epilogue((sa*sb) * (Aq @ Bq)), f32 accumulation in tensor memory.
 * a: [M, K] e4m3 row-major. bt: [N, K] e4m3 row-major (B stored K-major).
 * K % 16 == 0; M, N >= 1. Scales: when scale_a_dev / scale_b_dev are non-null
 * they are read on the device (no host sync), else the by-value floats are used.
 * EPI_SWIGLU: the N columns are gate|up interleaved (2j gate, 2j+1 up); c is
 * [M, N/2] bf16 and amax_out (device float, must be zeroed by the caller or
 * by y_b200_gemm_fp8_swiglu_requant) receives max|c|. */
#define Y_B200_MAX_REPLICAS 7
typedef struct y_b200_gemm_fp8_args {
    const void* a;
    const void* bt;
    void* c;
    int m, n, k;
    float scale_a, scale_b;
    const float* scale_a_dev;
    const float* scale_b_dev;
    const void* bias;  /* [N], bias_kind F16 or F32; NULL for EPI_NONE/SWIGLU */
    int bias_kind;
    int epilogue;      /* Y_B200_EPI_*  */
    int out_kind;      /* Y_B200_F32 / F16 / BF16 */
    float* amax_out;   /* EPI_SWIGLU only */
    int cta_n;         /* 0 = pick from the tile table; else 64, 128 or 256 */
    int max_ctas;      /* 0 = one persistent CTA per SM */
    int cta_m;         /* 0 = pick from the tile table; 128 = one CTA per tile; 256 = a pair of
                          CTAs (cluster of 2) shares each 256 x 256 tile (needs cta_n 0 or 256) */
    /* Fused all-gather of the output: besides c, the epilogue stores every element to
     * c_replicas[0 .. c_replica_count) at the same offset. The replicas are this rank's slot
     * in the other GPUs' gathered buffers (peer memory opened with y_b200_peer_open; plain
     * stores over NVLink, no multicast), so the transfer overlaps the GEMM tile by tile and
     * no separate collective runs. The caller orders the ranks afterwards (a barrier on the
     * stream) before anyone reads a gathered buffer. Not with EPI_SWIGLU. */
    void* c_replicas[Y_B200_MAX_REPLICAS];
    int c_replica_count;
} y_b200_gemm_fp8_args;

Y_B200_API int y_b200_gemm_fp8(const y_b200_gemm_fp8_args* args, void* stream);

/* ---- F16 GEMM ---------------------------------------------------------------
 * Replaces gemm_f16_<tag>, gemm_f16_bias_relu_<tag>, gemm_f16_swiglu_<tag>
 * (src/ptx_emitter.rs:4199-4694, :4729-4814, :5064-5565; entries
 * tests/gemm_f16_decode_m1.ptx:6-9, tests/gemm_f16_bias_relu_4096.ptx:6-10,
 * tests/gemm_f16_swiglu_4096.ptx:6-10) and y_tensor_core_gemm_kernel /
 * y_fused_gemm_bias_relu_fp16_kernel (tests/y_tensor_core_gemm.cu:102-107, :2712-2719):
 *   C = epilogue(alpha * (A @ B)), f16 operands, f32 accumulation in tensor memory
 *   (tcgen05.mma.kind::f16), the same kernels and epilogues as the FP8 GEMM.
 * a: [M, K] f16 row-major. bt: [N, K] f16 row-major (B stored K-major). K % 8 == 0.
 * alpha == 0 means 1. EPI_SWIGLU: bt rows are gate|up interleaved (2j gate, 2j+1 up),
 * c is [M, N/2], out_kind F32 or BF16. */
typedef struct y_b200_gemm_f16_args {
    const void* a;
    const void* bt;
    void* c;
    int m, n, k;
    float alpha;
    const void* bias;  /* [N], bias_kind F16 or F32; NULL for EPI_NONE/SWIGLU */
    int bias_kind;
    int epilogue;      /* Y_B200_EPI_*  */
    int out_kind;      /* Y_B200_F32 / F16 / BF16 */
    int cta_n, max_ctas, cta_m;  /* as in y_b200_gemm_fp8_args */
} y_b200_gemm_f16_args;
Y_B200_API int y_b200_gemm_f16(const y_b200_gemm_f16_args* args, void* stream);

/* Drop-ins for the reference entries, which take B row-major [K, N]:
 *   gemm_f16_<tag>(A, B, C) and gemm_f16_bias_relu_<tag>(A, B, Bias f32 [N], C):
 *     C [M, N] = A @ B (+ Bias, ReLU when bias != NULL / relu != 0); out_kind F32 (the compiled
 *     entries) or F16 (the runtime-shape .cu entries); bias_kind F32 or F16.
 *   gemm_f16_swiglu_<tag>(X, Wgate, Wup, Out): Out [M, N] f32 = silu(X @ Wgate) * (X @ Wup),
 *     Wgate and Wup separate [K, N] matrices.
 * Each call first copies the weights K-major into `workspace` (one HBM-bound pass; a caller
 * that keeps its weights K-major uses y_b200_gemm_f16 and skips it), then runs the GEMM.
 * K % 8 == 0. workspace: the matching *_workspace_bytes, 256-byte aligned. */
Y_B200_API size_t y_b200_gemm_f16_rowmajor_workspace_bytes(int n, int k);
Y_B200_API int y_b200_gemm_f16_rowmajor(const void* a_f16, const void* b_f16, const void* bias, int bias_kind,
                                        int relu, void* c, int out_kind, int m, int n, int k, void* workspace,
                                        size_t workspace_bytes, void* stream);
Y_B200_API size_t y_b200_gemm_f16_swiglu_workspace_bytes(int n, int k);
Y_B200_API int y_b200_gemm_f16_swiglu(const void* x_f16, const void* wgate_f16, const void* wup_f16, float* out,
                                      int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream);

/* Small-M F16 GEMM with the weights streamed once from HBM, row-major [K, N] as the
 * reference's gemm_f16_decode_m<M> entries take them (tests/gemm_f16_decode_m1.ptx:6-9):
 *   out [M, N] (F32 or F16) = x [M, K] f16 (row stride ldx elements) @ w [K, N] f16.
 * 1 <= M <= 32, K % 16 == 0, N % 8 == 0, ldx % 8 == 0, x and w 16-byte aligned; no workspace,
 * no atomics (K is split across the warps of a CTA and the CTAs of a cluster and reduced in a
 * fixed order). */
Y_B200_API int y_b200_gemm_f16_decode(const void* x_f16, int ldx, const void* w_f16, void* out, int out_kind,
                                      int m, int n, int k, void* stream);
/* The reference's split-K pair for decode shapes (tests/y_tensor_core_gemm.cu:4732-4738,
 * :4852-4858): partial sums over k_splits equal K ranges into workspace [k_splits, M, N] f32,
 * then their sum in split order rounded to f16. K % (16 * k_splits) == 0. */
Y_B200_API int y_b200_gemm_f16_splitk_workspace(const void* a_f16, const void* b_f16, float* workspace, int m,
                                                int n, int k, int k_splits, void* stream);
Y_B200_API int y_b200_splitk_reduction(const float* workspace, void* c_f16, size_t total, int m, int n,
                                       int k_splits, void* stream);

/* Launch geometry the library would use for this problem (the reference
 * embeds it in PTX comments, src/ptx_emitter.rs:3337, :4323-4331). */
typedef struct y_b200_launch_info {
    unsigned grid[3], block[3], cluster[3];
    unsigned dyn_smem_bytes;
    size_t workspace_bytes;
    int cta_m, cta_n, cta_k, stages;
    /* EpilogueFusionPass's statistic (src/quantization_pass.rs:802-819): 1 when an activation
     * (ReLU, SiLU) is fused into this kernel's accumulator write-back, else 0. */
    int fused_epilogues;
} y_b200_launch_info;
Y_B200_API int y_b200_gemm_fp8_launch_info(int m, int n, int k, int cta_n, y_b200_launch_info* out);

/* Drop-in for the reference entry gemm_fp8_<tag>(A, B, scale_a, scale_b, C):
 * A [M, K] f32, B [K, N] f32 row-major, C [M, N] f32; operands are quantised
 * on the device with the given scales, then multiplied. workspace holds the
 * e4m3 copies: y_b200_gemm_fp8_f32_workspace_bytes(m, n, k) bytes. */
Y_B200_API size_t y_b200_gemm_fp8_f32_workspace_bytes(int m, int n, int k);
Y_B200_API int y_b200_gemm_fp8_f32(const float* a, const float* b, float scale_a, float scale_b, float* c,
                        int m, int n, int k, void* workspace, size_t workspace_bytes,
                        void* stream);

/* The same GEMM for callers that cannot allocate device memory when they call:
 * an engine whose own pool already owns all of HBM, a latency-critical loop
 * where cudaMalloc (a device-wide lock, possibly a synchronisation) is not
 * allowed, a host that hands a plugin nothing but its inputs and outputs.
 * No counterpart in the reference, whose launch path always allocates its
 * buffers itself.
 * The e4m3 operand copies go to a fixed array inside the library image instead
 * of a workspace: every GPU that loads the library holds
 * Y_B200_STATIC_OPERAND_BYTES + 256 bytes of it until the process exits. That
 * memory is reserved when the CUDA module holding the array is loaded on a
 * device - with CUDA's default lazy loading, on the first call that touches it,
 * which is normally the first call of this entry - not per call. A caller whose
 * own pool is about to take the rest of HBM therefore makes one warm-up call
 * per device first (any small shape).
 * Limit: round256(M*K) + round256(N*K) <= Y_B200_STATIC_OPERAND_BYTES (for
 * example 2048 x 2048 x 2048); larger problems return Y_B200_ERR_WORKSPACE and
 * must use y_b200_gemm_fp8_f32. The call itself makes no cudaMalloc / cudaFree,
 * uses no allocating library routine and does not synchronise: it enqueues
 * three kernels on `stream` and returns.
 * The first call on each device looks up the array's device address (with that
 * device current); make that first call before any stream capture begins.
 * All calls on a device share the one array and it keeps the last call's
 * contents: calls that can overlap on the GPU (different streams, different
 * threads) race on it and must be serialised by the caller. Nothing in the
 * array needs clearing between calls. A bounded wait that runs out is recorded
 * in a status word inside the array (the first report is kept) and is read and
 * cleared by y_b200_device_status like the other entries' reports. */
#define Y_B200_STATIC_OPERAND_BYTES (8u << 20)
Y_B200_API int y_b200_gemm_fp8_f32_static(const float* a, const float* b, float scale_a, float scale_b,
                                          float* c, int m, int n, int k, void* stream);

/* Fused SwiGLU GEMM with FP8 re-quantisation (replaces gemm_f16_swiglu_<tag>,
 * src/ptx_emitter.rs:5064-5565, with FP8 operands and interleaved gate|up):
 * h = bf16(silu(g) * u) -> fresh per-tensor scale -> q = e4m3(h / scale).
 * q is [M, N/2] e4m3, scale_out a device float.
 * workspace: y_b200_swiglu_workspace_bytes(m, n) bytes (the bf16 h tensor
 * and the amax word). */
Y_B200_API size_t y_b200_swiglu_workspace_bytes(int m, int n);
Y_B200_API int y_b200_gemm_fp8_swiglu_requant(const y_b200_gemm_fp8_args* args, void* q, float* scale_out,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* Gated MLP on FP8 operands: out = (silu(A Wg) * (A Wu)) Wdown, the chain the
 * reference's SwiGLU benchmark stops short of ("down projection not included",
 * benchmark_y_swiglu_gemm_results.md:29). Three launches on one stream, no host
 * synchronisation between them:
 *   1. y_b200_gemm_fp8 with the SwiGLU epilogue: h = bf16(silu(g) * u), running amax;
 *   2. h -> e4m3 with the fresh per-tensor scale (kept on the device);
 *   3. y_b200_gemm_fp8: out = (scale_h * scale_down) * (hq @ Wdown_q), bf16 / f16 / f32.
 * a [M, K] e4m3; w_gate_up_t [2*I, K] e4m3 (rows 2j gate, 2j+1 up); w_down_t
 * [N_out, I] e4m3; out [M, N_out] of out_kind. scale_a_dev may be NULL (then
 * scale_a is used). I % 16 == 0 and K % 16 == 0.
 * workspace: y_b200_mlp_workspace_bytes(m, inter) bytes, 256-byte aligned. */
Y_B200_API size_t y_b200_mlp_workspace_bytes(int m, int inter);
Y_B200_API int y_b200_mlp_swiglu_fp8(const void* a, float scale_a, const float* scale_a_dev,
                                     const void* w_gate_up_t, float scale_gate_up, const void* w_down_t,
                                     float scale_down, void* out, int out_kind, int m, int k, int inter,
                                     int n_out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- INT4 weight-only decode GEMM -------------------------------------------
 * The reference has no INT4 kernel (src/ptx_emitter.rs:7321-7330 is a dead
 * stub); its decode entries gemm_f16_decode_m<M> (tests/gemm_f16_decode_m1.ptx:6-9)
 * stream F16 weights. Format defined here: symmetric, group 128 along K,
 * s = f16(amax_g/7), q = clamp(rne(w/s), -8, 7), two's-complement nibbles,
 * element k = 8*kw + j in nibble j of qweight[kw, n]; scales [K/128, N] f16.
 * K % 128 == 0, N % 16 == 0. */
Y_B200_API int y_b200_int4_quantize(const void* w_f16, size_t k, size_t n, uint32_t* qweight,
                         void* scales_f16, void* stream);
/* Bytes of the streaming layout the decode kernel reads (weights and scales
 * interleaved per 16-column x 128-row block). */
Y_B200_API size_t y_b200_int4_stream_bytes(size_t k, size_t n);
Y_B200_API int y_b200_int4_repack(const uint32_t* qweight, const void* scales_f16, size_t k, size_t n,
                       void* wstream, void* stream);
/* out[M, N] f16 = x[M, K] f16 @ dequant(W); f32 accumulation. 1 <= M <= 32. */
Y_B200_API int y_b200_gemm_int4_decode(const void* x_f16, const void* wstream, void* out_f16, int m, int n,
                            int k, void* stream);

/* Measurement aid with no counterpart in the reference: the time per launch, in
 * microseconds, of a kernel that only reads `bytes` (a multiple of 16) from bufs[i % nbufs]
 * in a chain of `launches` programmatic dependent launches, each reading one word the launch
 * before it wrote: the floor for any weight-streaming launch of that size in such a chain
 * (a chain of short launches cannot reach the bandwidth of one long copy). One warm-up chain,
 * then the median of `reps` (<= 64) timed chains is written to *us_per_launch.
 * scratch_256: 256 bytes of device memory. Synchronises the stream. */
Y_B200_API int y_b200_probe_chain_read(const void* const* bufs, int nbufs, size_t bytes, int launches, int reps,
                                       void* scratch_256, float* us_per_launch, void* stream);

/* ---- fused add + RMSNorm with the residual stream ------------------------------
 * Replaces rmsnorm_residual_<H> (src/ptx_emitter.rs:5773-6015; parameters X,
 * Residual, Weight, Out, NewResidual, all f16; one CTA of 256 threads per row):
 *   h = X + Residual (f32), Out = f16((h * rsqrt(mean(h^2) + eps)) * Weight),
 *   NewResidual = f16(h).
 * x, residual, out, new_residual [rows, hidden] f16; weight [hidden] f16. The reference
 * fixes eps = 1e-5 and hidden % 256 == 0; here eps is a parameter and hidden % 8 == 0. */
Y_B200_API int y_b200_rmsnorm_residual(const void* x_f16, const void* residual_f16, const void* weight_f16,
                                       size_t rows, size_t hidden, float eps, void* out_f16,
                                       void* new_residual_f16, void* stream);

/* ---- rotary position embedding ---------------------------------------------------
 * Replaces rope_<head_dim> (src/ptx_emitter.rs:6016-6260; parameters X f16, Positions
 * i32, Out f16; one warp per row, a row being one token's query or key vector of one
 * head): interleaved pairs (2i, 2i+1), theta_i = Positions[row] * base^(-2i/head_dim),
 *   out[2i] = x[2i] cos - x[2i+1] sin,  out[2i+1] = x[2i] sin + x[2i+1] cos.
 * The reference fixes base = 10000 and takes head_dim % 64 == 0; here base is a
 * parameter and head_dim is 64, 128 or 256. out may alias x. */
Y_B200_API int y_b200_rope(const void* x_f16, const int32_t* positions, void* out_f16, size_t rows, int head_dim,
                           float base, void* stream);

/* ---- paged decode attention --------------------------------------------------------
 * Replaces paged_decode_attention_<head_dim>_<q_heads>_<kv_heads>_<page_size>[_<warps>]
 * (src/ptx_emitter.rs:6267-6760; parameters Q, KCache, VCache, PageTable, SeqLens, Out,
 * MaxPages): one new query token per (sequence, query head) over a page-indexed f16 KV
 * cache, softmax(q . k / sqrt(head_dim)) v with f32 accumulation, query head h reading
 * KV head h / (q_heads / kv_heads).
 *   q, out     [num_seqs, num_q_heads, head_dim] f16
 *   kcache, vcache [num_pages, page_size, num_kv_heads, head_dim] f16
 *   page_table [num_seqs, max_pages] i32 (logical -> physical page), seq_lens [num_seqs] i32
 * A sequence of length 0 gives zeros. head_dim is 64, 128 or 256; at most 16 query heads
 * per KV head. The head counts, page size and head size are runtime values here.
 * workspace: y_b200_paged_decode_attention_workspace_bytes(...) bytes, 256-byte aligned.
 * It holds partial results when a sequence is cut across CTAs; whether the call does
 * that depends on num_seqs and num_kv_heads alone (and the SM count), not on the data. */
Y_B200_API size_t y_b200_paged_decode_attention_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                                                int head_dim);
Y_B200_API int y_b200_paged_decode_attention(const void* q_f16, const void* kcache_f16, const void* vcache_f16,
                                             const int32_t* page_table, const int32_t* seq_lens, void* out_f16,
                                             int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                             int page_size, int max_pages, void* workspace, size_t workspace_bytes,
                                             void* stream);

/* ---- peer memory for the fused all-gather ------------------------------------------
 * One process per GPU. y_b200_peer_alloc gives device memory that other processes of the
 * node can map: y_b200_peer_export writes an opaque 64-byte handle to send to them (any
 * host channel), y_b200_peer_open maps a received handle and returns a device pointer
 * valid in this process (stores to it travel over NVLink), y_b200_peer_close unmaps it.
 * Free with y_b200_peer_free after every peer has closed its mapping. */
#define Y_B200_PEER_HANDLE_BYTES 64
Y_B200_API int y_b200_peer_alloc(size_t bytes, void** ptr);
Y_B200_API int y_b200_peer_free(void* ptr);
Y_B200_API int y_b200_peer_export(const void* ptr, unsigned char handle[Y_B200_PEER_HANDLE_BYTES]);
Y_B200_API int y_b200_peer_open(const unsigned char handle[Y_B200_PEER_HANDLE_BYTES], void** peer_ptr);
Y_B200_API int y_b200_peer_close(void* peer_ptr);
/* Synchronous copy of a peer buffer (or any device memory) to the host, for checks. */
Y_B200_API int y_b200_peer_read(void* host_dst, const void* device_src, size_t bytes);

/* ---- input generator ---------------------------------------------------------
 * random_f16_bits (src/cuda_runtime.rs:657-682): element i = f(i + index0, seed),
 * a normal binary16 with exponent in 12..14. Written on the device. */
Y_B200_API int y_b200_fill_random_f16(void* out_f16, size_t n, uint64_t index0, uint64_t seed, void* stream);

/* ---- c_api.rs symbols (src/c_api.rs:27-212) -----------------------------------
 * Strings returned by these are owned by the library; free with y_free_string.
 * is_fp8 is one byte, as the reference's `bool` (src/c_api.rs:109, :183). */
Y_B200_API char* y_compile_to_ptx(const char* source, const char* target_sm, char** error_out);
Y_B200_API char* y_autotune_search_space_json(uint32_t m, uint32_t n, uint32_t k, bool is_fp8);
Y_B200_API char* y_autotune_select_config_json(uint32_t m, uint32_t n, uint32_t k, bool is_fp8);
Y_B200_API int32_t y_interpret_kernel(const char* source, char** error_out);
Y_B200_API uint32_t y_block_cdiv(uint32_t a, uint32_t b);
Y_B200_API void y_free_string(char* s);

#ifdef __cplusplus
}
#endif
#endif
