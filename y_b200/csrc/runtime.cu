// Host launch API (see include/y_b200_runtime.h): the reference's CudaContext
// surface over the CUDA runtime, plus the autotuner hooks.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/y_b200_runtime.h"
#include "autotuner.cuh"
#include "common.cuh"
#include "frontend.h"

struct y_ctx {
    int device;
    char name[256];
};

struct y_buf {
    void* ptr;
    size_t len;
    int device;
};

enum class Entry {
    GemmFp8F32, Fp8Gemm, Fp8GemmBiasRelu, Fp8GemmSwiglu, Int4Decode, RmsnormResidual, Rope, PagedDecodeAttention,
    GemmF16, GemmF16BiasRelu, GemmF16Swiglu,                      // descriptor kernels, baked shape, f32 out
    TensorCoreGemm, FusedGemmBiasReluFp16, SplitkWorkspace, SplitkReduction  // runtime-shape .cu entries, f16 out
};

struct y_kernel {
    Entry entry;
    int m, n, k;          // baked shape for descriptor kernels, 0 otherwise
    void* workspace;      // owned; operand copies of the f32 drop-in entry
    size_t workspace_bytes;
    unsigned max_dyn_smem;
    int device;
    int page_size;        // paged decode attention only
};

namespace yb {
void decode_launch_geometry(int m, int n, int k, unsigned* grid, unsigned* block, unsigned* smem, int* slots, int* unit_k);
void f16_decode_launch_geometry(int n, int k, int sms, unsigned* grid, unsigned* block, unsigned* smem, int* stages, unsigned* cluster);
void umma_decode_launch_geometry(int n, int k, int sms, unsigned* grid, unsigned* block, unsigned* smem, int* stages, unsigned* cluster);
bool umma_decode_applies(int m, int n, int k);
}
using namespace yb;

namespace {

// Shapes the weight-streaming kernel takes (y_b200_gemm_f16_decode's preconditions); other
// F16 shapes go through the tensor-core GEMM.
bool uses_decode_kernel(int m, int n, int k) { return m <= 32 && k % 16 == 0 && n % 8 == 0; }

// Grows a kernel object's workspace (owned by it, freed with it).
int ensure_workspace(y_kernel* k, size_t need) {
    if (need <= k->workspace_bytes) return 0;
    if (k->workspace) cudaFree(k->workspace);
    k->workspace = nullptr;
    k->workspace_bytes = 0;
    int rc = check_cuda(cudaMalloc(&k->workspace, need), "cudaMalloc(kernel workspace)");
    if (rc) return rc;
    k->workspace_bytes = need;
    return 0;
}

// F16 GEMM with row-major B [K, N]: the weight-streaming kernel for decode shapes, else the
// K-major copy + tensor-core GEMM. `bias` may be null.
int run_f16_rowmajor(y_kernel* k, const void* a, const void* b, const void* bias, int bias_kind, int relu, void* c,
                     int out_kind, int m, int n, int kk) {
    if (!bias && uses_decode_kernel(m, n, kk)) return y_b200_gemm_f16_decode(a, kk, b, c, out_kind, m, n, kk, nullptr);
    int rc = ensure_workspace(k, y_b200_gemm_f16_rowmajor_workspace_bytes(n, kk));
    if (rc) return rc;
    return y_b200_gemm_f16_rowmajor(a, b, bias, bias_kind, relu, c, out_kind, m, n, kk, k->workspace, k->workspace_bytes,
                                    nullptr);
}

char* dup_cstr(const std::string& s) {
    char* p = static_cast<char*>(malloc(s.size() + 1));
    if (p) memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

int bind(const y_ctx* ctx) {
    if (!ctx) return fail(Y_B200_ERR_INVALID, "null context");
    return check_cuda(cudaSetDevice(ctx->device), "cudaSetDevice");
}

Precision precision_from_int(int p) {
    switch (p) {
        case 1: return Precision::F32;
        case 2: return Precision::BF16;
        case 3: return Precision::Fp8;
        case 4: return Precision::Int4;
        default: return Precision::F16;
    }
}

Candidate cand_from6(const uint32_t c[6]) { return {c[0], c[1], c[2], c[3], c[4], c[5], c[3] * c[4]}; }

void cand_to7(const Candidate& c, uint32_t out[7]) {
    out[0] = c.cta_m; out[1] = c.cta_n; out[2] = c.cta_k; out[3] = c.warps_m;
    out[4] = c.warps_n; out[5] = c.num_stages; out[6] = c.num_warps;
}

int kernel_info(const y_kernel* k, int m, int n, int kk, y_b200_launch_info* out) {
    memset(out, 0, sizeof *out);
    if (k->entry == Entry::Int4Decode) {
        int slots = 0, unit_k = 0;
        decode_launch_geometry(m, n, kk, &out->grid[0], &out->block[0], &out->dyn_smem_bytes, &slots, &unit_k);
        out->grid[1] = out->grid[2] = 1;
        out->block[1] = out->block[2] = 1;
        out->cluster[0] = out->cluster[1] = out->cluster[2] = 1;
        out->cta_m = m <= 8 ? 8 : (m <= 16 ? 16 : 32); out->cta_n = 16; out->cta_k = unit_k; out->stages = slots;
        return 0;
    }
    const bool f16 = k->entry == Entry::GemmF16 || k->entry == Entry::GemmF16BiasRelu || k->entry == Entry::GemmF16Swiglu ||
                     k->entry == Entry::TensorCoreGemm || k->entry == Entry::FusedGemmBiasReluFp16;
    if ((k->entry == Entry::GemmF16 || k->entry == Entry::TensorCoreGemm) && uses_decode_kernel(m, n, kk)) {
        const bool umma = umma_decode_applies(m, n, kk);  // 17..32 tokens: the tcgen05 kernel
        if (umma) umma_decode_launch_geometry(n, kk, 0, &out->grid[0], &out->block[0], &out->dyn_smem_bytes, &out->stages, &out->cluster[0]);
        else f16_decode_launch_geometry(n, kk, 0, &out->grid[0], &out->block[0], &out->dyn_smem_bytes, &out->stages, &out->cluster[0]);
        out->grid[1] = out->grid[2] = out->block[1] = out->block[2] = 1;
        out->cluster[1] = out->cluster[2] = 1;
        out->cta_m = m <= 8 ? 8 : (m <= 16 ? 16 : 32); out->cta_n = 64; out->cta_k = umma ? 64 : 32;
        return 0;
    }
    // An f16 problem runs the byte-tiled kernels on rows of 2 K bytes; SwiGLU on 2 N interleaved columns.
    const int n_eff = k->entry == Entry::GemmF16Swiglu ? 2 * n : n;
    int rc = y_b200_gemm_fp8_launch_info(m, n_eff, f16 ? 2 * kk : kk, 0, out);
    if (rc) return rc;
    if (k->entry == Entry::GemmFp8F32) out->workspace_bytes = y_b200_gemm_fp8_f32_workspace_bytes(m, n, kk);
    if (k->entry == Entry::GemmF16Swiglu) out->workspace_bytes = y_b200_gemm_f16_swiglu_workspace_bytes(n, kk);
    else if (f16) out->workspace_bytes = y_b200_gemm_f16_rowmajor_workspace_bytes(n, kk);
    out->fused_epilogues = (k->entry == Entry::GemmF16BiasRelu || k->entry == Entry::GemmF16Swiglu ||
                            k->entry == Entry::Fp8GemmBiasRelu || k->entry == Entry::Fp8GemmSwiglu ||
                            k->entry == Entry::FusedGemmBiasReluFp16) ? 1 : 0;
    return 0;
}

int expect_args(const y_arg* args, int nargs, const int* kinds, int want, const char* entry) {
    if (!args || nargs != want) return fail(Y_B200_ERR_INVALID, "%s takes %d arguments, got %d", entry, want, nargs);
    for (int i = 0; i < want; ++i)
        if (args[i].kind != kinds[i])
            return fail(Y_B200_ERR_INVALID, "%s: argument %d has kind %d, expected %d", entry, i, args[i].kind, kinds[i]);
    return 0;
}

int check_geometry(const y_kernel* k, int m, int n, int kk, const unsigned grid[3], const unsigned block[3],
                   unsigned smem) {
    if (!grid && !block && smem == 0) return 0;
    y_b200_launch_info info;
    int rc = kernel_info(k, m, n, kk, &info);
    if (rc) return rc;
    if (grid && (grid[0] != info.grid[0] || grid[1] != info.grid[1] || grid[2] != info.grid[2]))
        return fail(Y_B200_ERR_INVALID, "launch grid (%u,%u,%u) differs from the kernel's own (%u,%u,%u)", grid[0],
                    grid[1], grid[2], info.grid[0], info.grid[1], info.grid[2]);
    if (block && (block[0] != info.block[0] || block[1] != info.block[1] || block[2] != info.block[2]))
        return fail(Y_B200_ERR_INVALID, "launch block (%u,%u,%u) differs from the kernel's own (%u,1,1)", block[0],
                    block[1], block[2], info.block[0]);
    if (smem != 0 && smem != info.dyn_smem_bytes)
        return fail(Y_B200_ERR_INVALID, "dynamic shared memory %u differs from the kernel's own %u", smem,
                    info.dyn_smem_bytes);
    if (k->max_dyn_smem != 0 && k->max_dyn_smem < info.dyn_smem_bytes)
        return fail(Y_B200_ERR_INVALID, "set_max_dynamic_smem(%u) is below the %u bytes this kernel needs",
                    k->max_dyn_smem, info.dyn_smem_bytes);
    return 0;
}

int launch_once(y_kernel* k, const unsigned grid[3], const unsigned block[3], unsigned smem, const y_arg* a,
                int nargs) {
    switch (k->entry) {
        case Entry::GemmFp8F32: {
            static const int kinds[5] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_F32, Y_ARG_F32, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 5, "gemm_fp8_<tag>");
            if (rc) return rc;
            if ((rc = check_geometry(k, k->m, k->n, k->k, grid, block, smem))) return rc;
            return y_b200_gemm_fp8_f32(reinterpret_cast<const float*>(a[0].v.ptr),
                                       reinterpret_cast<const float*>(a[1].v.ptr), a[2].v.f32, a[3].v.f32,
                                       reinterpret_cast<float*>(a[4].v.ptr), k->m, k->n, k->k, k->workspace,
                                       k->workspace_bytes, nullptr);
        }
        case Entry::Fp8Gemm: {
            static const int kinds[8] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_F32,
                                         Y_ARG_F32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 8, "y_fp8_gemm");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[5].v.i32, a[6].v.i32, a[7].v.i32, grid, block, smem))) return rc;
            y_b200_gemm_fp8_args g = {};
            g.a = reinterpret_cast<const void*>(a[0].v.ptr);
            g.bt = reinterpret_cast<const void*>(a[1].v.ptr);
            g.c = reinterpret_cast<void*>(a[2].v.ptr);
            g.scale_a = a[3].v.f32; g.scale_b = a[4].v.f32;
            g.m = a[5].v.i32; g.n = a[6].v.i32; g.k = a[7].v.i32;
            g.out_kind = Y_B200_BF16;
            return y_b200_gemm_fp8(&g, nullptr);
        }
        case Entry::Fp8GemmBiasRelu: {
            // (Aq, Bqt, bias f16 [N], C bf16, scale_a, scale_b, M, N, K, is_relu): the FP8 form of
            // y_fused_gemm_bias_relu_fp16_kernel (tests/y_tensor_core_gemm.cu:2712-2719).
            static const int kinds[10] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_F32,
                                          Y_ARG_F32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 10, "y_fp8_gemm_bias_relu");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[6].v.i32, a[7].v.i32, a[8].v.i32, grid, block, smem))) return rc;
            y_b200_gemm_fp8_args g = {};
            g.a = reinterpret_cast<const void*>(a[0].v.ptr);
            g.bt = reinterpret_cast<const void*>(a[1].v.ptr);
            g.bias = reinterpret_cast<const void*>(a[2].v.ptr);
            g.bias_kind = Y_B200_F16;
            g.c = reinterpret_cast<void*>(a[3].v.ptr);
            g.scale_a = a[4].v.f32; g.scale_b = a[5].v.f32;
            g.m = a[6].v.i32; g.n = a[7].v.i32; g.k = a[8].v.i32;
            g.epilogue = a[9].v.i32 ? Y_B200_EPI_BIAS_RELU : Y_B200_EPI_BIAS;
            g.out_kind = Y_B200_BF16;
            return y_b200_gemm_fp8(&g, nullptr);
        }
        case Entry::Fp8GemmSwiglu: {
            // (Aq, Bqt gate|up interleaved [N, K], C bf16 [M, N/2], scale_a, scale_b, M, N, K)
            static const int kinds[8] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_F32,
                                         Y_ARG_F32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 8, "y_fp8_gemm_swiglu");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[5].v.i32, a[6].v.i32, a[7].v.i32, grid, block, smem))) return rc;
            y_b200_gemm_fp8_args g = {};
            g.a = reinterpret_cast<const void*>(a[0].v.ptr);
            g.bt = reinterpret_cast<const void*>(a[1].v.ptr);
            g.c = reinterpret_cast<void*>(a[2].v.ptr);
            g.scale_a = a[3].v.f32; g.scale_b = a[4].v.f32;
            g.m = a[5].v.i32; g.n = a[6].v.i32; g.k = a[7].v.i32;
            g.epilogue = Y_B200_EPI_SWIGLU;
            g.out_kind = Y_B200_BF16;
            return y_b200_gemm_fp8(&g, nullptr);
        }
        case Entry::GemmF16: {
            static const int kinds[3] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 3, "gemm_f16_<tag>");
            if (rc) return rc;
            if ((rc = check_geometry(k, k->m, k->n, k->k, grid, block, smem))) return rc;
            return run_f16_rowmajor(k, reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                    nullptr, 0, 0, reinterpret_cast<void*>(a[2].v.ptr), Y_B200_F32, k->m, k->n, k->k);
        }
        case Entry::GemmF16BiasRelu: {
            static const int kinds[4] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 4, "gemm_f16_bias_relu_<tag>");
            if (rc) return rc;
            if ((rc = check_geometry(k, k->m, k->n, k->k, grid, block, smem))) return rc;
            if (!a[2].v.ptr) return fail(Y_B200_ERR_INVALID, "gemm_f16_bias_relu_<tag>: null Bias");
            return run_f16_rowmajor(k, reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                    reinterpret_cast<const void*>(a[2].v.ptr), Y_B200_F32, 1,
                                    reinterpret_cast<void*>(a[3].v.ptr), Y_B200_F32, k->m, k->n, k->k);
        }
        case Entry::GemmF16Swiglu: {
            static const int kinds[4] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 4, "gemm_f16_swiglu_<tag>");
            if (rc) return rc;
            if ((rc = check_geometry(k, k->m, k->n, k->k, grid, block, smem))) return rc;
            if ((rc = ensure_workspace(k, y_b200_gemm_f16_swiglu_workspace_bytes(k->n, k->k)))) return rc;
            return y_b200_gemm_f16_swiglu(reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                          reinterpret_cast<const void*>(a[2].v.ptr), reinterpret_cast<float*>(a[3].v.ptr),
                                          k->m, k->n, k->k, k->workspace, k->workspace_bytes, nullptr);
        }
        case Entry::TensorCoreGemm: {
            // (A f16, B f16 [K, N], C f16, M, N, K): y_tensor_core_gemm_kernel, tests/y_tensor_core_gemm.cu:102-107
            static const int kinds[6] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 6, "y_tensor_core_gemm");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[3].v.i32, a[4].v.i32, a[5].v.i32, grid, block, smem))) return rc;
            return run_f16_rowmajor(k, reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                    nullptr, 0, 0, reinterpret_cast<void*>(a[2].v.ptr), Y_B200_F16, a[3].v.i32, a[4].v.i32,
                                    a[5].v.i32);
        }
        case Entry::FusedGemmBiasReluFp16: {
            // (A, B, bias f16, C f16, M, N, K, is_relu): tests/y_tensor_core_gemm.cu:2712-2719
            static const int kinds[8] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 8, "y_fused_gemm_bias_relu_fp16");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[4].v.i32, a[5].v.i32, a[6].v.i32, grid, block, smem))) return rc;
            if (!a[2].v.ptr) return fail(Y_B200_ERR_INVALID, "y_fused_gemm_bias_relu_fp16: null bias");
            return run_f16_rowmajor(k, reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                    reinterpret_cast<const void*>(a[2].v.ptr), Y_B200_F16, a[7].v.i32 != 0,
                                    reinterpret_cast<void*>(a[3].v.ptr), Y_B200_F16, a[4].v.i32, a[5].v.i32, a[6].v.i32);
        }
        case Entry::SplitkWorkspace: {
            // (A, B, Workspace f32 [k_splits, M, N], M, N, K, k_splits): tests/y_tensor_core_gemm.cu:4732-4738
            static const int kinds[7] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 7, "y_fused_gemm_splitk_workspace");
            if (rc) return rc;
            if (grid || block || smem)
                return fail(Y_B200_ERR_INVALID, "y_fused_gemm_splitk_workspace: pass no launch geometry (the library splits K itself)");
            if (a[3].v.i32 < 1 || a[3].v.i32 > 32)
                return fail(Y_B200_ERR_SHAPE, "y_fused_gemm_splitk_workspace: M=%d outside the decode range 1..32", a[3].v.i32);
            return y_b200_gemm_f16_splitk_workspace(reinterpret_cast<const void*>(a[0].v.ptr),
                                                    reinterpret_cast<const void*>(a[1].v.ptr),
                                                    reinterpret_cast<float*>(a[2].v.ptr), a[3].v.i32, a[4].v.i32, a[5].v.i32,
                                                    a[6].v.i32, nullptr);
        }
        case Entry::SplitkReduction: {
            // (Workspace, C f16, total, M, N, k_splits): tests/y_tensor_core_gemm.cu:4852-4858
            static const int kinds[6] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 6, "y_splitk_reduction");
            if (rc) return rc;
            if (grid || block || smem) return fail(Y_B200_ERR_INVALID, "y_splitk_reduction: pass no launch geometry");
            return y_b200_splitk_reduction(reinterpret_cast<const float*>(a[0].v.ptr), reinterpret_cast<void*>(a[1].v.ptr),
                                           (size_t)(a[2].v.i32 < 0 ? 0 : a[2].v.i32), a[3].v.i32, a[4].v.i32, a[5].v.i32,
                                           nullptr);
        }
        case Entry::Int4Decode: {
            static const int kinds[6] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32, Y_ARG_I32, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 6, "y_int4_decode_gemm");
            if (rc) return rc;
            if ((rc = check_geometry(k, a[3].v.i32, a[4].v.i32, a[5].v.i32, grid, block, smem))) return rc;
            return y_b200_gemm_int4_decode(reinterpret_cast<const void*>(a[0].v.ptr),
                                           reinterpret_cast<const void*>(a[1].v.ptr),
                                           reinterpret_cast<void*>(a[2].v.ptr), a[3].v.i32, a[4].v.i32,
                                           a[5].v.i32, nullptr);
        }
        case Entry::RmsnormResidual: {
            // (X, Residual, Weight, Out, NewResidual); one CTA of 256 threads per row, so the
            // grid is the number of rows (src/ptx_emitter.rs:5773-5790). eps is the reference's 1e-5.
            static const int kinds[5] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 5, "rmsnorm_residual_<H>");
            if (rc) return rc;
            if (!grid || grid[0] == 0 || grid[1] != 1 || grid[2] != 1)
                return fail(Y_B200_ERR_INVALID, "rmsnorm_residual_<H>: the launch grid must be (rows, 1, 1)");
            if (block && (block[0] != 256 || block[1] != 1 || block[2] != 1))
                return fail(Y_B200_ERR_INVALID, "rmsnorm_residual_<H>: launch block (%u,%u,%u) differs from the kernel's own (256,1,1)",
                            block[0], block[1], block[2]);
            return y_b200_rmsnorm_residual(reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                                           reinterpret_cast<const void*>(a[2].v.ptr), grid[0], (size_t)k->k, 1e-5f,
                                           reinterpret_cast<void*>(a[3].v.ptr), reinterpret_cast<void*>(a[4].v.ptr), nullptr);
        }
        case Entry::Rope: {
            // (X, Positions, Out); the reference launches one 32-thread CTA per row
            // (tests/benchmark_y_rmsnorm_rope.py:156), so the grid is the number of rows.
            static const int kinds[3] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR};
            int rc = expect_args(a, nargs, kinds, 3, "rope_<head_dim>");
            if (rc) return rc;
            if (!grid || grid[0] == 0 || grid[1] != 1 || grid[2] != 1)
                return fail(Y_B200_ERR_INVALID, "rope_<head_dim>: the launch grid must be (rows, 1, 1)");
            if (block && (block[0] != 32 || block[1] != 1 || block[2] != 1))
                return fail(Y_B200_ERR_INVALID, "rope_<head_dim>: launch block (%u,%u,%u) differs from the entry's (32,1,1)",
                            block[0], block[1], block[2]);
            return y_b200_rope(reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const int32_t*>(a[1].v.ptr),
                               reinterpret_cast<void*>(a[2].v.ptr), grid[0], k->k, 10000.0f, nullptr);
        }
        case Entry::PagedDecodeAttention: {
            // (Q, KCache, VCache, PageTable, SeqLens, Out, MaxPages); the reference's grid is
            // (num_q_heads, num_seqs, 1) (src/ptx_emitter.rs:6321-6323): the sequence count comes from it.
            static const int kinds[7] = {Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_PTR, Y_ARG_I32};
            int rc = expect_args(a, nargs, kinds, 7, "paged_decode_attention_<...>");
            if (rc) return rc;
            if (!grid || (int)grid[0] != k->m || grid[1] == 0 || grid[2] != 1)
                return fail(Y_B200_ERR_INVALID, "paged_decode_attention: the launch grid must be (%d, num_seqs, 1)", k->m);
            const int num_seqs = (int)grid[1];
            const size_t need = y_b200_paged_decode_attention_workspace_bytes(num_seqs, k->m, k->n, k->k);
            if (need > k->workspace_bytes) {  // grown on demand, owned by the kernel object
                if (k->workspace) cudaFree(k->workspace);
                k->workspace = nullptr;
                k->workspace_bytes = 0;
                if ((rc = check_cuda(cudaMalloc(&k->workspace, need), "cudaMalloc(attention workspace)"))) return rc;
                k->workspace_bytes = need;
            }
            return y_b200_paged_decode_attention(
                reinterpret_cast<const void*>(a[0].v.ptr), reinterpret_cast<const void*>(a[1].v.ptr),
                reinterpret_cast<const void*>(a[2].v.ptr), reinterpret_cast<const int32_t*>(a[3].v.ptr),
                reinterpret_cast<const int32_t*>(a[4].v.ptr), reinterpret_cast<void*>(a[5].v.ptr), num_seqs, k->m, k->n,
                k->k, k->page_size, a[6].v.i32, k->workspace, k->workspace_bytes, nullptr);
        }
    }
    return fail(Y_B200_ERR_UNSUPPORTED, "unknown kernel entry");
}

std::string field_between(const std::string& hay, const std::string& start, const std::string& end) {
    size_t s = hay.find(start);
    if (s == std::string::npos) return std::string();
    s += start.size();
    size_t e = hay.find(end, s);
    if (e == std::string::npos) return std::string();
    return hay.substr(s, e - s);
}

}  // namespace

// ---- context ---------------------------------------------------------------------
extern "C" y_ctx* y_ctx_create(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        set_error("no CUDA driver or device");
        return nullptr;
    }
    cudaDeviceProp prop;
    if (cudaSetDevice(0) != cudaSuccess || cudaFree(nullptr) != cudaSuccess ||
        cudaGetDeviceProperties(&prop, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("device 0 refused to initialise");
        return nullptr;
    }
    y_ctx* ctx = static_cast<y_ctx*>(calloc(1, sizeof(y_ctx)));
    if (!ctx) return nullptr;
    ctx->device = 0;
    snprintf(ctx->name, sizeof ctx->name, "%s", prop.name);
    return ctx;
}

extern "C" void y_ctx_destroy(y_ctx* ctx) { free(ctx); }

extern "C" const char* y_ctx_device_name(const y_ctx* ctx) { return ctx ? ctx->name : ""; }

extern "C" int y_ctx_device_attribute(const y_ctx* ctx, int attrib, int* value_out) {
    if (!ctx || !value_out) return fail(Y_B200_ERR_INVALID, "y_ctx_device_attribute: null argument");
    // Driver ordinals the path reads, mapped onto runtime attributes.
    cudaDeviceAttr a;
    switch (attrib) {
        case 16: a = cudaDevAttrMultiProcessorCount; break;
        case 38: a = cudaDevAttrL2CacheSize; break;            // CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE
        case 39: a = cudaDevAttrMaxThreadsPerMultiProcessor; break;
        case 75: a = cudaDevAttrComputeCapabilityMajor; break;
        case 76: a = cudaDevAttrComputeCapabilityMinor; break;
        case 81: a = cudaDevAttrMaxSharedMemoryPerMultiprocessor; break;
        case 97: a = cudaDevAttrMaxSharedMemoryPerBlockOptin; break;
        case 13: a = cudaDevAttrClockRate; break;
        case 36: a = cudaDevAttrMemoryClockRate; break;
        case 37: a = cudaDevAttrGlobalMemoryBusWidth; break;
        default: a = static_cast<cudaDeviceAttr>(attrib); break;
    }
    return check_cuda(cudaDeviceGetAttribute(value_out, a, ctx->device), "cudaDeviceGetAttribute");
}

extern "C" int y_ctx_mem_info(const y_ctx* ctx, size_t* free_out, size_t* total_out) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!free_out || !total_out) return fail(Y_B200_ERR_INVALID, "y_ctx_mem_info: null output");
    return check_cuda(cudaMemGetInfo(free_out, total_out), "cudaMemGetInfo");
}

extern "C" int y_ctx_synchronize(const y_ctx* ctx) {
    int rc = bind(ctx);
    if (rc) return rc;
    return check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

// ---- buffers -----------------------------------------------------------------------
extern "C" y_buf* y_ctx_alloc(y_ctx* ctx, size_t len_bytes) {
    if (bind(ctx)) return nullptr;
    void* p = nullptr;
    if (check_cuda(cudaMalloc(&p, len_bytes ? len_bytes : 1), "cudaMalloc")) return nullptr;
    y_buf* b = static_cast<y_buf*>(calloc(1, sizeof(y_buf)));
    if (!b) { cudaFree(p); return nullptr; }
    b->ptr = p; b->len = len_bytes; b->device = ctx->device;
    return b;
}

extern "C" void y_buf_free(y_buf* buf) {
    if (!buf) return;
    if (buf->ptr) cudaFree(buf->ptr);
    free(buf);
}

extern "C" uint64_t y_buf_device_ptr(const y_buf* buf) { return buf ? reinterpret_cast<uint64_t>(buf->ptr) : 0; }
extern "C" size_t y_buf_len_bytes(const y_buf* buf) { return buf ? buf->len : 0; }

extern "C" int y_ctx_memset_u8(y_ctx* ctx, y_buf* buf, uint8_t value) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!buf) return fail(Y_B200_ERR_INVALID, "y_ctx_memset_u8: null buffer");
    return check_cuda(cudaMemset(buf->ptr, value, buf->len), "cudaMemset");
}

extern "C" int y_ctx_memcpy_htod_at(y_ctx* ctx, y_buf* buf, size_t offset_bytes, const void* src, size_t n) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!buf || (!src && n)) return fail(Y_B200_ERR_INVALID, "y_ctx_memcpy_htod_at: null argument");
    if (offset_bytes > buf->len || n > buf->len - offset_bytes)
        return fail(Y_B200_ERR_INVALID, "memcpy_htod_at out of range: offset %zu + %zu bytes > buffer %zu bytes",
                    offset_bytes, n, buf->len);
    return check_cuda(cudaMemcpy(static_cast<char*>(buf->ptr) + offset_bytes, src, n, cudaMemcpyHostToDevice),
                      "cudaMemcpy(HtoD)");
}

extern "C" int y_ctx_memcpy_dtoh_at(y_ctx* ctx, void* dst, size_t n, const y_buf* buf, size_t offset_bytes) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!buf || (!dst && n)) return fail(Y_B200_ERR_INVALID, "y_ctx_memcpy_dtoh_at: null argument");
    if (offset_bytes > buf->len || n > buf->len - offset_bytes)
        return fail(Y_B200_ERR_INVALID, "memcpy_dtoh_at out of range: offset %zu + %zu bytes > buffer %zu bytes",
                    offset_bytes, n, buf->len);
    return check_cuda(cudaMemcpy(dst, static_cast<const char*>(buf->ptr) + offset_bytes, n, cudaMemcpyDeviceToHost),
                      "cudaMemcpy(DtoH)");
}

extern "C" int y_ctx_memcpy_dtod(y_ctx* ctx, y_buf* dst, const y_buf* src) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!dst || !src) return fail(Y_B200_ERR_INVALID, "y_ctx_memcpy_dtod: null buffer");
    const size_t n = dst->len < src->len ? dst->len : src->len;
    return check_cuda(cudaMemcpy(dst->ptr, src->ptr, n, cudaMemcpyDeviceToDevice), "cudaMemcpy(DtoD)");
}

// ---- kernels -----------------------------------------------------------------------
extern "C" y_kernel* y_ctx_load_module(y_ctx* ctx, const char* image, const char* entry) {
    if (bind(ctx)) return nullptr;
    if (!entry) { set_error("y_ctx_load_module: null entry name"); return nullptr; }
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ctx->device);
    if (major != 10) {
        fail(Y_B200_ERR_UNSUPPORTED, "y_ctx_load_module: device is sm_%d0, the kernels are built for sm_100a only", major);
        return nullptr;
    }
    y_kernel k = {};
    k.device = ctx->device;
    const std::string name(entry);
    if (image == nullptr) {
        if (name == "y_fp8_gemm") k.entry = Entry::Fp8Gemm;
        else if (name == "y_fp8_gemm_bias_relu") k.entry = Entry::Fp8GemmBiasRelu;
        else if (name == "y_fp8_gemm_swiglu") k.entry = Entry::Fp8GemmSwiglu;
        else if (name == "y_int4_decode_gemm") k.entry = Entry::Int4Decode;
        else if (name == "y_tensor_core_gemm") k.entry = Entry::TensorCoreGemm;
        else if (name == "y_fused_gemm_bias_relu_fp16") k.entry = Entry::FusedGemmBiasReluFp16;
        else if (name == "y_fused_gemm_splitk_workspace") k.entry = Entry::SplitkWorkspace;
        else if (name == "y_splitk_reduction") k.entry = Entry::SplitkReduction;
        else { fail(Y_B200_ERR_UNSUPPORTED, "y_ctx_load_module: no built-in entry named '%s'", entry); return nullptr; }
    } else {
        // Find "// [Y B200 KERNEL] entry=<name> family=<f>" and the shape line after it.
        const std::string img(image);
        const std::string tag = "entry=" + name + " family=";
        size_t at = img.find(tag);
        if (at == std::string::npos) {
            fail(Y_B200_ERR_UNSUPPORTED, "y_ctx_load_module: the image has no kernel named '%s'", entry);
            return nullptr;
        }
        const std::string fam = img.substr(at + tag.size(), img.find_first_of(" \n", at + tag.size()) - at - tag.size());
        if (fam == "rmsnorm_residual") {
            // rmsnorm_residual_<H>: the hidden size is the name's suffix; rows come with the launch grid
            const long long hidden = atoll(name.c_str() + strlen("rmsnorm_residual_"));
            if (name.rfind("rmsnorm_residual_", 0) != 0 || hidden <= 0 || hidden % 8 != 0 || hidden > 0x7fffffff) {
                fail(Y_B200_ERR_INVALID, "y_ctx_load_module: '%s' does not name a hidden size that is a multiple of 8", entry);
                return nullptr;
            }
            k.entry = Entry::RmsnormResidual;
            k.k = (int)hidden;
            y_kernel* res = static_cast<y_kernel*>(malloc(sizeof(y_kernel)));
            if (!res) return nullptr;
            *res = k;
            return res;
        }
        if (fam == "paged_decode_attention") {
            // paged_decode_attention_<head_dim>_<q_heads>_<kv_heads>_<page_size>[_<warps>]
            int dims[5] = {0, 0, 0, 0, 0};
            const int got = sscanf(name.c_str(), "paged_decode_attention_%d_%d_%d_%d_%d", &dims[0], &dims[1], &dims[2],
                                   &dims[3], &dims[4]);
            if (got < 4 || (dims[0] != 64 && dims[0] != 128 && dims[0] != 256) || dims[1] < 1 || dims[2] < 1 ||
                dims[1] % dims[2] != 0 || dims[1] / dims[2] > 16 || dims[3] < 1) {
                fail(Y_B200_ERR_INVALID, "y_ctx_load_module: '%s' does not name head_dim (64/128/256), query heads, KV heads "
                     "(dividing the query heads, at most 16 per KV head) and page size", entry);
                return nullptr;
            }
            k.entry = Entry::PagedDecodeAttention;
            k.k = dims[0]; k.m = dims[1]; k.n = dims[2];
            k.page_size = dims[3];
            y_kernel* res = static_cast<y_kernel*>(malloc(sizeof(y_kernel)));
            if (!res) return nullptr;
            *res = k;
            return res;
        }
        if (fam == "rope") {
            const long long head_dim = atoll(name.c_str() + strlen("rope_"));
            if (name.rfind("rope_", 0) != 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256)) {
                fail(Y_B200_ERR_INVALID, "y_ctx_load_module: '%s' does not name a head size of 64, 128 or 256", entry);
                return nullptr;
            }
            k.entry = Entry::Rope;
            k.k = (int)head_dim;
            y_kernel* res = static_cast<y_kernel*>(malloc(sizeof(y_kernel)));
            if (!res) return nullptr;
            *res = k;
            return res;
        }
        const bool f16_family = fam == "gemm_f16" || fam == "gemm_f16_bias_relu" || fam == "gemm_f16_swiglu";
        if (fam != "gemm_fp8" && !f16_family) {
            fail(Y_B200_ERR_UNSUPPORTED, "y_ctx_load_module: family '%s' of '%s' has no sm_100a kernel in this library",
                 fam.c_str(), entry);
            return nullptr;
        }
        const std::string rest = img.substr(at);
        long long m = atoll(field_between(rest, "] M=", " ").c_str());
        long long n = atoll(field_between(rest, " N=", " ").c_str());
        long long kk = atoll(field_between(rest, " K=", " ").c_str());
        if (m <= 0 || n <= 0 || kk <= 0 || m > 0x7fffffff || n > 0x7fffffff || kk > 0x7fffffff) {
            fail(Y_B200_ERR_INVALID, "y_ctx_load_module: could not read M/N/K of '%s' from the image", entry);
            return nullptr;
        }
        k.m = (int)m; k.n = (int)n; k.k = (int)kk;
        if (f16_family) {
            // The reference's preconditions (src/ptx_emitter.rs:4252-4260, :5110-5112), checked again
            // here because a descriptor is only text.
            if (k.k % 8 != 0 || 2LL * k.n > 0x7fffffff) {
                fail(Y_B200_ERR_SHAPE, "y_ctx_load_module: F16 GEMM '%s' needs K %% 8 == 0", entry);
                return nullptr;
            }
            k.entry = fam == "gemm_f16" ? Entry::GemmF16 : fam == "gemm_f16_bias_relu" ? Entry::GemmF16BiasRelu : Entry::GemmF16Swiglu;
            size_t need = 0;  // decode shapes stream the weights as they lie and need none
            if (k.entry == Entry::GemmF16Swiglu) need = y_b200_gemm_f16_swiglu_workspace_bytes(k.n, k.k);
            else if (k.entry == Entry::GemmF16BiasRelu || !uses_decode_kernel(k.m, k.n, k.k))
                need = y_b200_gemm_f16_rowmajor_workspace_bytes(k.n, k.k);
            if (need && check_cuda(cudaMalloc(&k.workspace, need), "cudaMalloc(workspace)")) return nullptr;
            k.workspace_bytes = need;
        } else {
            k.entry = Entry::GemmFp8F32;
            k.workspace_bytes = y_b200_gemm_fp8_f32_workspace_bytes(k.m, k.n, k.k);
            if (check_cuda(cudaMalloc(&k.workspace, k.workspace_bytes), "cudaMalloc(workspace)")) return nullptr;
        }
    }
    y_kernel* out = static_cast<y_kernel*>(malloc(sizeof(y_kernel)));
    if (!out) { if (k.workspace) cudaFree(k.workspace); return nullptr; }
    *out = k;
    return out;
}

extern "C" void y_kernel_free(y_kernel* kernel) {
    if (!kernel) return;
    if (kernel->workspace) cudaFree(kernel->workspace);
    free(kernel);
}

extern "C" int y_kernel_set_max_dynamic_smem(y_kernel* kernel, unsigned bytes) {
    if (!kernel) return fail(Y_B200_ERR_INVALID, "y_kernel_set_max_dynamic_smem: null kernel");
    int optin = 0;
    YB_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, kernel->device));
    if (bytes > (unsigned)optin)
        return fail(Y_B200_ERR_INVALID, "requested %u bytes of dynamic shared memory, the device allows %d", bytes, optin);
    kernel->max_dyn_smem = bytes;
    return 0;
}

extern "C" int y_kernel_launch_info(const y_kernel* kernel, y_b200_launch_info* out) {
    if (!kernel || !out) return fail(Y_B200_ERR_INVALID, "y_kernel_launch_info: null argument");
    if (kernel->entry != Entry::GemmFp8F32 && kernel->entry != Entry::GemmF16 && kernel->entry != Entry::GemmF16BiasRelu &&
        kernel->entry != Entry::GemmF16Swiglu)
        return fail(Y_B200_ERR_INVALID, "y_kernel_launch_info: runtime-shape entries have no baked geometry; use y_b200_gemm_fp8_launch_info");
    return kernel_info(kernel, kernel->m, kernel->n, kernel->k, out);
}

extern "C" int y_ctx_launch(y_ctx* ctx, y_kernel* kernel, const unsigned grid[3], const unsigned block[3],
                            unsigned shared_bytes, const y_arg* args, int nargs) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!kernel) return fail(Y_B200_ERR_INVALID, "y_ctx_launch: null kernel");
    return launch_once(kernel, grid, block, shared_bytes, args, nargs);
}

extern "C" int y_ctx_time_launches(y_ctx* ctx, y_kernel* kernel, const unsigned grid[3], const unsigned block[3],
                                   unsigned shared_bytes, const y_arg* arg_sets, int n_sets, int nargs,
                                   unsigned iters, double* mean_us_out) {
    int rc = bind(ctx);
    if (rc) return rc;
    if (!kernel || !mean_us_out) return fail(Y_B200_ERR_INVALID, "y_ctx_time_launches: null argument");
    if (iters == 0) return fail(Y_B200_ERR_INVALID, "time_launches called with iters = 0");
    if (!arg_sets || n_sets <= 0) return fail(Y_B200_ERR_INVALID, "time_launches called with no argument sets");
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    YB_CUDA(cudaEventCreate(&e0));
    if ((rc = check_cuda(cudaEventCreate(&e1), "cudaEventCreate"))) { cudaEventDestroy(e0); return rc; }
    rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (!rc) rc = check_cuda(cudaEventRecord(e0, nullptr), "cudaEventRecord");
    for (unsigned i = 0; i < iters && !rc; ++i)
        rc = launch_once(kernel, grid, block, shared_bytes, arg_sets + (size_t)(i % (unsigned)n_sets) * nargs, nargs);
    if (!rc) rc = check_cuda(cudaEventRecord(e1, nullptr), "cudaEventRecord");
    if (!rc) rc = check_cuda(cudaEventSynchronize(e1), "cudaEventSynchronize");
    float ms = 0.0f;
    if (!rc) rc = check_cuda(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc) return rc;
    *mean_us_out = (double)ms * 1000.0 / (double)iters;
    return 0;
}

// ---- autotuner hooks ---------------------------------------------------------------
extern "C" char* y_autotune_persist_key(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name) {
    return dup_cstr(persist_key(m, n, k, precision_from_int(precision), gpu_name ? gpu_name : ""));
}

extern "C" int y_autotune_parse_persisted(const char* value, uint32_t out[7]) {
    Candidate c;
    if (!value || !out || !parse_persisted_value(value, &c)) return -1;
    cand_to7(c, out);
    return 0;
}

extern "C" void y_autotune_set_profile_path(const char* path) { set_profile_path(path ? path : ""); }

extern "C" int y_autotune_store(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name,
                                const uint32_t cand[6]) {
    if (!cand) return -1;
    return store_persisted(m, n, k, precision_from_int(precision), gpu_name ? gpu_name : "", cand_from6(cand)) ? 0 : -1;
}

extern "C" int y_autotune_lookup(uint32_t m, uint32_t n, uint32_t k, int precision, const char* gpu_name,
                                 uint32_t out[7], uint32_t nearest_out[3]) {
    if (!out) return 0;
    const Precision p = precision_from_int(precision);
    const std::string gpu = gpu_name ? gpu_name : "";
    Candidate c;
    if (load_persisted(m, n, k, p, gpu, &c)) { cand_to7(c, out); return 1; }
    uint32_t shape[3] = {0, 0, 0};
    if (load_persisted_nearest(m, n, k, p, gpu, &c, shape)) {
        cand_to7(c, out);
        if (nearest_out) memcpy(nearest_out, shape, sizeof shape);
        return 2;
    }
    return 0;
}

extern "C" void y_autotune_set_mode(int mode) {
    set_tuning_mode(mode == 1 ? TuningMode::Analytic : mode == 2 ? TuningMode::Measure
                                : mode == 3 ? TuningMode::Remeasure : TuningMode::Cached);
}

extern "C" void y_autotune_clear_cache(void) { clear_autotune_cache(); }

extern "C" int y_autotune_is_launchable(const uint32_t cand[6], uint32_t k, int precision) {
    return cand && is_launchable(cand_from6(cand), k, precision_from_int(precision)) ? 1 : 0;
}

extern "C" double y_autotune_score(const uint32_t cand[6], uint32_t m, uint32_t n, uint32_t k, int precision) {
    return cand ? score_candidate(cand_from6(cand), m, n, k, precision_from_int(precision), 148) : -1.0;
}

extern "C" int y_autotune_tied(double best_a, double median_a, double best_b, double median_b) {
    Timing a{best_a, median_a, median_a}, b{best_b, median_b, median_b};
    return a.tied_with(b) ? 1 : 0;
}

extern "C" size_t y_autotune_select_winner(const double* r, size_t n) {
    std::vector<Measured> v;
    for (size_t i = 0; r && i < n; ++i) {
        const double* row = r + 8 * i;
        Candidate c{(uint32_t)row[0], (uint32_t)row[1], (uint32_t)row[2], (uint32_t)row[3],
                    (uint32_t)row[4], (uint32_t)row[5], (uint32_t)row[3] * (uint32_t)row[4]};
        v.push_back({c, Timing{row[6], row[7], row[7] * 1.05}, 0.0, true});
    }
    return select_winner(v);
}

extern "C" size_t y_autotune_plan_weight_replicas(size_t b_bytes, size_t a_bytes, size_t c_bytes, size_t l2_bytes,
                                                  size_t free_bytes) {
    return plan_weight_replicas(b_bytes, a_bytes, c_bytes, l2_bytes, free_bytes);
}

extern "C" char* y_autotune_measure_fp8_json(uint32_t m, uint32_t n, uint32_t k) {
    std::vector<Measured> ranked;
    std::string err;
    if (tune_gemm_fp8(m, n, k, &ranked, &err) != 0 || ranked.empty()) {
        set_error("%s", err.c_str());
        return nullptr;
    }
    store_persisted(m, n, k, Precision::Fp8, current_gpu_name(), ranked[0].candidate);
    std::string out = "[";
    for (size_t i = 0; i < ranked.size(); ++i) {
        char buf[384];
        const Measured& r = ranked[i];
        snprintf(buf, sizeof buf,
                 "%s{\"cta_m\":%u,\"cta_n\":%u,\"cta_k\":%u,\"warps_m\":%u,\"warps_n\":%u,\"num_stages\":%u,"
                 "\"num_warps\":%u,\"best_us\":%.3f,\"median_us\":%.3f,\"max_us\":%.3f,\"tflops\":%.2f}",
                 i ? "," : "", r.candidate.cta_m, r.candidate.cta_n, r.candidate.cta_k, r.candidate.warps_m,
                 r.candidate.warps_n, r.candidate.num_stages, r.candidate.num_warps, r.timing.best_us,
                 r.timing.median_us, r.timing.max_us, r.tflops);
        out += buf;
    }
    out += "]";
    return dup_cstr(out);
}

// "... | CTA 64x128x32 | 2x2 warps | ..." and "Dynamic shared memory required: N bytes"
// (src/empirical_autotune.rs:317-359). grid_x walks N, grid_y walks M.
extern "C" int y_parse_launch_config(const char* text, uint32_t m, uint32_t n, uint32_t out[4]) {
    if (!text || !out) return fail(Y_B200_ERR_INVALID, "y_parse_launch_config: null argument");
    const std::string all(text);
    std::string line;
    size_t pos = 0;
    bool found = false;
    while (pos <= all.size()) {
        size_t e = all.find('\n', pos);
        if (e == std::string::npos) e = all.size();
        line = all.substr(pos, e - pos);
        if (line.find("TENSOR CORE GEMM]") != std::string::npos) { found = true; break; }
        pos = e + 1;
    }
    if (!found) return fail(Y_B200_ERR_INVALID, "text has no '[Y TENSOR CORE GEMM]' comment");
    const std::string cta = field_between(line, "| CTA ", " |");
    unsigned a = 0, b = 0, c = 0;
    if (sscanf(cta.c_str(), "%ux%ux%u", &a, &b, &c) != 3 || a == 0 || b == 0)
        return fail(Y_B200_ERR_INVALID, "malformed CTA field '%s'", cta.c_str());
    size_t wend = line.find(" warps");
    if (wend == std::string::npos) return fail(Y_B200_ERR_INVALID, "could not find the warps field");
    size_t wbeg = line.rfind("| ", wend);
    unsigned wm = 0, wn = 0;
    if (wbeg == std::string::npos || sscanf(line.c_str() + wbeg + 2, "%ux%u", &wm, &wn) != 2)
        return fail(Y_B200_ERR_INVALID, "malformed warps field");
    const std::string smem = field_between(all, "Dynamic shared memory required: ", " bytes");
    out[0] = (n + b - 1) / b;
    out[1] = (m + a - 1) / a;
    out[2] = wm * wn * 32;
    out[3] = smem.empty() ? 0u : (uint32_t)strtoul(smem.c_str(), nullptr, 10);
    return 0;
}
