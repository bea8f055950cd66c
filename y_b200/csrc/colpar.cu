// Pipelined host path of the column-parallel step behind the C ABI (see include/y_b200_runtime.h):
// X arrives in pinned host memory, C leaves to pinned host memory, and the copy-in of step
// i + 1, the kernels of step i and the copy-out of step i - 1 run on three streams at once,
// so both directions of the host link and the GPU overlap. The reference's launch path has only
// synchronous copies (src/cuda_runtime.rs:402-456); this is their asynchronous extension.
#include <new>
#include <vector>

#include "../../include/y_b200_runtime.h"
#include "common.cuh"

struct y_colpar {
    int device;
    int m, k, n_shard, depth;
    float eps;
    const void* bqt;
    const float* scale_b_dev;
    const void* gamma;
    cudaStream_t s_in, s_cmp, s_out;
    std::vector<void*> x, aq, c, ws;   // per slot: f16 X, e4m3 A, bf16 C, prologue workspace
    std::vector<float*> sa;            // per slot: the activation scale (stays on the device)
    std::vector<cudaEvent_t> in_done, cmp_done, out_done;
    size_t ws_bytes;
    unsigned long long count;
};

using namespace yb;

namespace {

void release(y_colpar* p) {
    if (!p) return;
    for (void* q : p->x) if (q) cudaFree(q);
    for (void* q : p->aq) if (q) cudaFree(q);
    for (void* q : p->c) if (q) cudaFree(q);
    for (void* q : p->ws) if (q) cudaFree(q);
    for (float* q : p->sa) if (q) cudaFree(q);
    for (cudaEvent_t e : p->in_done) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : p->cmp_done) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : p->out_done) if (e) cudaEventDestroy(e);
    if (p->s_in) cudaStreamDestroy(p->s_in);
    if (p->s_cmp) cudaStreamDestroy(p->s_cmp);
    if (p->s_out) cudaStreamDestroy(p->s_out);
    delete p;
}

// The step on `st`: RMSNorm -> e4m3 prologue into the slot's buffers, then the FP8 GEMM.
int run_step(y_colpar* p, const void* x_dev, void* c_dev, int slot, cudaStream_t st) {
    int rc = y_b200_rmsnorm_quantize_fp8(x_dev, p->gamma, (size_t)p->m, (size_t)p->k, p->eps, p->aq[slot], p->sa[slot],
                                         p->ws[slot], p->ws_bytes, st);
    if (rc) return rc;
    y_b200_gemm_fp8_args g = {};
    g.a = p->aq[slot]; g.bt = p->bqt; g.c = c_dev;
    g.m = p->m; g.n = p->n_shard; g.k = p->k;
    g.scale_a_dev = p->sa[slot]; g.scale_b_dev = p->scale_b_dev;
    g.epilogue = Y_B200_EPI_NONE;
    g.out_kind = Y_B200_BF16;
    return y_b200_gemm_fp8(&g, st);
}

}  // namespace

extern "C" y_colpar* y_colpar_create(const void* bqt_e4m3, const float* scale_b_dev, const void* gamma_f16, float eps, int m,
                                     int k, int n_shard, int depth) {
    if (!bqt_e4m3 || !scale_b_dev || !gamma_f16) { fail(Y_B200_ERR_INVALID, "y_colpar_create: null pointer"); return nullptr; }
    if (m < 1 || n_shard < 1 || k < 16 || k % 16 != 0 || depth < 1 || depth > 8) {
        fail(Y_B200_ERR_SHAPE, "y_colpar_create: need M, N >= 1, K %% 16 == 0 and 1 <= depth <= 8 (M=%d N=%d K=%d depth=%d)", m,
             n_shard, k, depth);
        return nullptr;
    }
    y_colpar* p = new (std::nothrow) y_colpar();
    if (!p) return nullptr;
    p->m = m; p->k = k; p->n_shard = n_shard; p->depth = depth; p->eps = eps;
    p->bqt = bqt_e4m3; p->scale_b_dev = scale_b_dev; p->gamma = gamma_f16;
    p->ws_bytes = y_b200_rmsnorm_workspace_bytes((size_t)m);
    p->x.assign(depth, nullptr); p->aq.assign(depth, nullptr); p->c.assign(depth, nullptr); p->ws.assign(depth, nullptr);
    p->sa.assign(depth, nullptr);
    p->in_done.assign(depth, nullptr); p->cmp_done.assign(depth, nullptr); p->out_done.assign(depth, nullptr);
    bool ok = cudaGetDevice(&p->device) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&p->s_cmp, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < depth && ok; ++i) {
        ok = ok && cudaMalloc(&p->x[i], (size_t)m * k * 2) == cudaSuccess;
        ok = ok && cudaMalloc(&p->aq[i], (size_t)m * k) == cudaSuccess;
        ok = ok && cudaMalloc(&p->c[i], (size_t)m * n_shard * 2) == cudaSuccess;
        ok = ok && cudaMalloc(&p->ws[i], p->ws_bytes) == cudaSuccess;
        ok = ok && cudaMalloc(reinterpret_cast<void**>(&p->sa[i]), 256) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&p->in_done[i], cudaEventDisableTiming) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&p->cmp_done[i], cudaEventDisableTiming) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&p->out_done[i], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
        check_cuda(cudaGetLastError(), "y_colpar_create (streams, events or device buffers)");
        release(p);
        return nullptr;
    }
    return p;
}

extern "C" void y_colpar_destroy(y_colpar* p) {
    if (!p) return;
    cudaStreamSynchronize(p->s_in);
    cudaStreamSynchronize(p->s_cmp);
    cudaStreamSynchronize(p->s_out);
    release(p);
}

extern "C" int y_colpar_forward(y_colpar* p, const void* x_dev_f16, void* c_dev_bf16, int slot, void* stream) {
    if (!p || !x_dev_f16 || !c_dev_bf16) return fail(Y_B200_ERR_INVALID, "y_colpar_forward: null argument");
    if (slot < 0 || slot >= p->depth) return fail(Y_B200_ERR_INVALID, "y_colpar_forward: slot %d outside 0..%d", slot, p->depth - 1);
    return run_step(p, x_dev_f16, c_dev_bf16, slot, static_cast<cudaStream_t>(stream));
}

extern "C" int y_colpar_submit_host(y_colpar* p, const void* x_host_f16, void* c_host_bf16, void* caller_stream) {
    if (!p || !x_host_f16 || !c_host_bf16) return fail(Y_B200_ERR_INVALID, "y_colpar_submit_host: null argument");
    const int i = (int)(p->count % (unsigned long long)p->depth);
    cudaStream_t caller = static_cast<cudaStream_t>(caller_stream);
    // Work the caller enqueued earlier on its stream (e.g. filling x_host) comes first.
    cudaEvent_t start = nullptr;
    YB_CUDA(cudaEventCreateWithFlags(&start, cudaEventDisableTiming));
    int rc = check_cuda(cudaEventRecord(start, caller), "cudaEventRecord");
    if (!rc) rc = check_cuda(cudaStreamWaitEvent(p->s_in, start, 0), "cudaStreamWaitEvent");
    cudaEventDestroy(start);  // released once the pending wait has consumed it
    if (rc) return rc;
    if (p->count >= (unsigned long long)p->depth) {
        YB_CUDA(cudaStreamWaitEvent(p->s_in, p->cmp_done[i], 0));   // the kernels that last read this slot's X are done
    }
    YB_CUDA(cudaMemcpyAsync(p->x[i], x_host_f16, (size_t)p->m * p->k * 2, cudaMemcpyHostToDevice, p->s_in));
    YB_CUDA(cudaEventRecord(p->in_done[i], p->s_in));
    YB_CUDA(cudaStreamWaitEvent(p->s_cmp, p->in_done[i], 0));
    if (p->count >= (unsigned long long)p->depth) {
        YB_CUDA(cudaStreamWaitEvent(p->s_cmp, p->out_done[i], 0));  // the copy that last read this slot's C is done
    }
    if ((rc = run_step(p, p->x[i], p->c[i], i, p->s_cmp))) return rc;
    YB_CUDA(cudaEventRecord(p->cmp_done[i], p->s_cmp));
    YB_CUDA(cudaStreamWaitEvent(p->s_out, p->cmp_done[i], 0));
    YB_CUDA(cudaMemcpyAsync(c_host_bf16, p->c[i], (size_t)p->m * p->n_shard * 2, cudaMemcpyDeviceToHost, p->s_out));
    YB_CUDA(cudaEventRecord(p->out_done[i], p->s_out));
    p->count += 1;
    return 0;
}

extern "C" int y_colpar_drain(y_colpar* p, void* caller_stream) {
    if (!p) return fail(Y_B200_ERR_INVALID, "y_colpar_drain: null handle");
    cudaStream_t caller = static_cast<cudaStream_t>(caller_stream);
    const unsigned long long live = p->count < (unsigned long long)p->depth ? p->count : (unsigned long long)p->depth;
    for (unsigned long long i = 0; i < live; ++i) YB_CUDA(cudaStreamWaitEvent(caller, p->out_done[i], 0));
    return 0;
}

extern "C" int y_colpar_synchronize(y_colpar* p) {
    if (!p) return fail(Y_B200_ERR_INVALID, "y_colpar_synchronize: null handle");
    YB_CUDA(cudaStreamSynchronize(p->s_in));
    YB_CUDA(cudaStreamSynchronize(p->s_cmp));
    YB_CUDA(cudaStreamSynchronize(p->s_out));
    return 0;
}

extern "C" int y_colpar_host_bytes_per_step(const y_colpar* p, size_t* h2d_out, size_t* d2h_out) {
    if (!p || !h2d_out || !d2h_out) return fail(Y_B200_ERR_INVALID, "y_colpar_host_bytes_per_step: null argument");
    *h2d_out = (size_t)p->m * p->k * 2;
    *d2h_out = (size_t)p->m * p->n_shard * 2;
    return 0;
}
