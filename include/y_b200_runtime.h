/*
 * Host launch API of liby_b200: a C-ABI mirror of the reference's CUDA driver
 * binding `CudaContext` (src/cuda_runtime.rs:335-630) - one device, one
 * context, the default stream - which is what its measured autotuner and the
 * external launchers drive. Handles are opaque; every failure is a NULL /
 * negative return with text in y_b200_last_error(), never an abort.
 *
 * Differences forced by the change of backend, each called out at its symbol:
 * kernels are prebuilt for sm_100a, so y_ctx_load_module takes the launch
 * descriptor that y_compile_to_ptx returns (or NULL) instead of PTX text, and
 * y_ctx_launch takes typed arguments because the FP8 entries carry two f32
 * scalars (the reference's launch only accepts 8-byte pointers,
 * src/cuda_runtime.rs:536-568).
 */
#ifndef Y_B200_RUNTIME_H
#define Y_B200_RUNTIME_H

#include "y_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct y_ctx y_ctx;
typedef struct y_buf y_buf;
typedef struct y_kernel y_kernel;

/* CudaContext::new (src/cuda_runtime.rs:330-364): device 0; NULL when there is
 * no driver or no device. Bound to the calling thread's current device. */
Y_B200_API y_ctx* y_ctx_create(void);
Y_B200_API void y_ctx_destroy(y_ctx* ctx);
Y_B200_API const char* y_ctx_device_name(const y_ctx* ctx);
/* device_attribute (src/cuda_runtime.rs:370-381): raw CUdevice_attribute ordinal. */
Y_B200_API int y_ctx_device_attribute(const y_ctx* ctx, int attrib, int* value_out);
/* (free, total) bytes, src/cuda_runtime.rs:470-480. */
Y_B200_API int y_ctx_mem_info(const y_ctx* ctx, size_t* free_out, size_t* total_out);
Y_B200_API int y_ctx_synchronize(const y_ctx* ctx);

/* DeviceBuffer (src/cuda_runtime.rs:243-275). Buffers must be freed before
 * their context. */
Y_B200_API y_buf* y_ctx_alloc(y_ctx* ctx, size_t len_bytes);
Y_B200_API void y_buf_free(y_buf* buf);
Y_B200_API uint64_t y_buf_device_ptr(const y_buf* buf);
Y_B200_API size_t y_buf_len_bytes(const y_buf* buf);
Y_B200_API int y_ctx_memset_u8(y_ctx* ctx, y_buf* buf, uint8_t value);
/* Range-checked copies (src/cuda_runtime.rs:402-456): an out-of-range request
 * is an error string, never a partial copy. */
Y_B200_API int y_ctx_memcpy_htod_at(y_ctx* ctx, y_buf* buf, size_t offset_bytes, const void* src, size_t n);
Y_B200_API int y_ctx_memcpy_dtoh_at(y_ctx* ctx, void* dst, size_t n, const y_buf* buf, size_t offset_bytes);
/* Copies min(len(dst), len(src)) bytes (src/cuda_runtime.rs:463-466). */
Y_B200_API int y_ctx_memcpy_dtod(y_ctx* ctx, y_buf* dst, const y_buf* src);

/* load_ptx (src/cuda_runtime.rs:492-534). `image` is the descriptor text
 * returned by y_compile_to_ptx (shape and family are read from it) or NULL
 * for the runtime-shape entries below. Entries:
 *   from a descriptor, by the kernel's own name:
 *     gemm_fp8_<tag>(A f32*, B f32*, scale_a f32, scale_b f32, C f32*)
 *     gemm_f16_<tag>(A f16*, B f16* [K,N], C f32*)                      tests/gemm_f16_decode_m1.ptx:6-9
 *     gemm_f16_bias_relu_<tag>(A f16*, B f16* [K,N], Bias f32* [N], C f32*)  tests/gemm_f16_bias_relu_4096.ptx:6-10
 *     gemm_f16_swiglu_<tag>(X f16*, Wgate f16* [K,N], Wup f16* [K,N], Out f32*)  tests/gemm_f16_swiglu_4096.ptx:6-10
 *     rmsnorm_residual_<H>, rope_<d>, paged_decode_attention_<d>_<qh>_<kvh>_<page>[_<warps>]
 *       (the kernel object owns the K-major weight copy the F16 families need; M <= 32 shapes of
 *        gemm_f16_<tag> stream the row-major weights as they lie and need none)
 *   runtime-shape, image == NULL:
 *     y_fp8_gemm(Aq u8* [M,K], Bqt u8* [N,K], C bf16*, scale_a f32, scale_b f32, M i32, N i32, K i32)
 *       (argument order of y_fp8_tensor_core_gemm_kernel, tests/y_tensor_core_gemm.cu:4152-4159;
 *        B is K-major here and C is bf16)
 *     y_fp8_gemm_bias_relu(Aq, Bqt, bias f16* [N], C bf16*, scale_a, scale_b, M, N, K, is_relu i32)
 *     y_fp8_gemm_swiglu(Aq, Bqt gate|up interleaved [N,K], C bf16* [M,N/2], scale_a, scale_b, M, N, K)
 *     y_tensor_core_gemm(A f16*, B f16* [K,N], C f16*, M, N, K)         tests/y_tensor_core_gemm.cu:102-107
 *     y_fused_gemm_bias_relu_fp16(A, B, bias f16*, C f16*, M, N, K, is_relu)  tests/y_tensor_core_gemm.cu:2712-2719
 *     y_fused_gemm_splitk_workspace(A, B, Workspace f32* [k_splits,M,N], M, N, K, k_splits)  :4732-4738
 *     y_splitk_reduction(Workspace, C f16*, total, M, N, k_splits)      :4852-4858
 *       (the split-K pair takes no launch geometry: the library cuts K itself)
 *     y_int4_decode_gemm(X f16*, Wstream u8*, Out f16*, M i32, N i32, K i32)
 *       (argument order of y_tensor_core_gemm_kernel, tests/y_tensor_core_gemm.cu:102-107)
 * Returns NULL with the reason in y_b200_last_error(). */
Y_B200_API y_kernel* y_ctx_load_module(y_ctx* ctx, const char* image, const char* entry);
Y_B200_API void y_kernel_free(y_kernel* kernel);
/* set_max_dynamic_smem (src/cuda_runtime.rs:287-298): checked against the
 * kernel's own requirement and the device opt-in ceiling. */
Y_B200_API int y_kernel_set_max_dynamic_smem(y_kernel* kernel, unsigned bytes);
/* Launch geometry of this kernel (for descriptor kernels: of its baked shape). */
Y_B200_API int y_kernel_launch_info(const y_kernel* kernel, y_b200_launch_info* out);

enum { Y_ARG_PTR = 0, Y_ARG_F32 = 1, Y_ARG_I32 = 2 };
typedef struct y_arg {
    int kind;
    union {
        uint64_t ptr;
        float f32;
        int32_t i32;
    } v;
} y_arg;

/* launch (src/cuda_runtime.rs:536-568). grid/block/shared_bytes may be NULL/0
 * to use the kernel's own geometry; if given they must equal it (a kernel is
 * never launched with a geometry it was not built for). */
Y_B200_API int y_ctx_launch(y_ctx* ctx, y_kernel* kernel, const unsigned grid[3], const unsigned block[3],
                            unsigned shared_bytes, const y_arg* args, int nargs);
/* time_launches (src/cuda_runtime.rs:581-629): `iters` back-to-back launches
 * bracketed by one pair of events; launch i uses argument set i % n_sets
 * (arg_sets is n_sets x nargs, row-major), which is how a caller rotates over
 * distinct weight buffers to keep the working set out of L2. Mean microseconds
 * per launch in *mean_us_out. */
Y_B200_API int y_ctx_time_launches(y_ctx* ctx, y_kernel* kernel, const unsigned grid[3],
                                   const unsigned block[3], unsigned shared_bytes, const y_arg* arg_sets,
                                   int n_sets, int nargs, unsigned iters, double* mean_us_out);

/* ---- pipelined host path of the column-parallel step -------------------------------
 * The asynchronous extension of the reference's synchronous host copies
 * (src/cuda_runtime.rs:402-456) for the step
 *   C [M, N_s] bf16 = fp8_gemm(e4m3(rmsnorm(X; gamma, eps)), Bt shard)
 * with X and C in PINNED host memory. y_colpar_submit_host enqueues the host-to-device copy
 * of this step, its three kernels and the device-to-host copy of its result on three
 * internal streams; consecutive submissions overlap (copy-in of step i + 1, kernels of step
 * i, copy-out of step i - 1). Device buffers are reused round-robin over `depth` slots
 * (1..8). A host output buffer may be read once y_colpar_synchronize has returned, or on
 * `caller_stream` after y_colpar_drain. The handle keeps the weight shard, its scale and
 * gamma by pointer: they stay owned by the caller and must outlive it. One handle per GPU
 * and host thread; create it with that GPU current.
 *   bqt_e4m3 [N_s, K] e4m3 K-major, scale_b_dev one device float, gamma_f16 [K]; K % 16 == 0. */
typedef struct y_colpar y_colpar;
Y_B200_API y_colpar* y_colpar_create(const void* bqt_e4m3, const float* scale_b_dev, const void* gamma_f16, float eps,
                                     int m, int k, int n_shard, int depth);
Y_B200_API void y_colpar_destroy(y_colpar* handle);
/* The step on device buffers, on `stream`, using slot `slot`'s scratch (no copies). */
Y_B200_API int y_colpar_forward(y_colpar* handle, const void* x_dev_f16, void* c_dev_bf16, int slot, void* stream);
/* Work already enqueued on `caller_stream` (e.g. the kernel that fills x_host) is ordered first. */
Y_B200_API int y_colpar_submit_host(y_colpar* handle, const void* x_host_f16, void* c_host_bf16, void* caller_stream);
Y_B200_API int y_colpar_drain(y_colpar* handle, void* caller_stream);
Y_B200_API int y_colpar_synchronize(y_colpar* handle);
Y_B200_API int y_colpar_host_bytes_per_step(const y_colpar* handle, size_t* h2d_out, size_t* d2h_out);

/* ---- autotuner hooks (src/autotuner.rs, src/empirical_autotune.rs) ------------ */
/* precision: 0 F16, 1 F32, 2 BF16, 3 FP8, 4 INT4. Strings are library-owned. */
Y_B200_API char* y_autotune_persist_key(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name);
/* "cta_m,cta_n,cta_k,warps_m,warps_n,num_stages" -> out[7] (last = num_warps); 0 on success. */
Y_B200_API int y_autotune_parse_persisted(const char* value, uint32_t out[7]);
Y_B200_API void y_autotune_set_profile_path(const char* path);
Y_B200_API int y_autotune_store(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name,
                                const uint32_t cand[6]);
/* 1 = exact hit, 2 = borrowed from the nearest measured shape (shape in nearest_out), 0 = none. */
Y_B200_API int y_autotune_lookup(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name,
                                 uint32_t out[7], uint32_t nearest_out[3]);
/* mode: 0 cached, 1 analytic, 2 measure, 3 remeasure. */
Y_B200_API void y_autotune_set_mode(int mode);
Y_B200_API void y_autotune_clear_cache(void);
Y_B200_API int y_autotune_is_launchable(const uint32_t cand[6], uint32_t k, int precision);
Y_B200_API double y_autotune_score(const uint32_t cand[6], uint32_t m, uint32_t n, uint32_t k, int precision);
Y_B200_API int y_autotune_tied(double best_a, double median_a, double best_b, double median_b);
/* results: n rows of {cta_m,cta_n,cta_k,warps_m,warps_n,stages, best_us, median_us} sorted fastest first. */
Y_B200_API size_t y_autotune_select_winner(const double* results, size_t n);
Y_B200_API size_t y_autotune_plan_weight_replicas(size_t b_bytes, size_t a_bytes, size_t c_bytes,
                                                  size_t l2_bytes, size_t free_bytes);
/* Measures every FP8 GEMM candidate at this shape on the current device, persists
 * the winner and returns the ranking as JSON (winner first); NULL on failure. */
Y_B200_API char* y_autotune_measure_fp8_json(uint32_t m, uint32_t n, uint32_t k);
/* Launch geometry scraped from descriptor / reference-style comment text
 * (src/empirical_autotune.rs:317-359): out = {grid_x, grid_y, threads, dyn_smem}. */
Y_B200_API int y_parse_launch_config(const char* text, uint32_t m, uint32_t n, uint32_t out[4]);

#ifdef __cplusplus
}
#endif
#endif
