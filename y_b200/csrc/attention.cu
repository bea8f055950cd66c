// Paged decode attention: one new query token per (sequence, query head) attends over a
// page-indexed f16 KV cache (the reference's paged_decode_attention_<d>_<qh>_<kvh>_<page>,
// src/ptx_emitter.rs:6267-6760).
//
// The kernel is KV-cache streaming: every K and V byte of a sequence is read once. To make
// that true under grouped-query attention, a CTA owns one KV head of one sequence and works
// on ALL query heads that share it (the reference launches one CTA per query head, so its
// KV reads repeat num_q_heads / num_kv_heads times). The group's queries are the 16-row
// operand of mma.sync.m16n8k16 (rows beyond the group are zero), 16 tokens at a time:
//   S[16 x 16 tokens] = Q[16 x D] K^T      (K rows from shared memory via ldmatrix)
//   online softmax per query row in the exp2 domain, running (m, l)
//   O[16 x D] += P[16 x 16] V[16 x D]      (V via ldmatrix.trans)
// Each warp streams its own 16-token K/V tiles with per-thread 16-byte cp.async copies,
// three tiles deep, into XOR-swizzled rows (no bank conflicts for ldmatrix), so there is no
// block-level synchronisation inside the token loop. Warps of a CTA take tiles round-robin
// and merge their (m, l, O) states through shared memory at the end. A long sequence is
// also cut across CTAs ("splits": the grid would otherwise be num_seqs x num_kv_heads CTAs,
// a fraction of 148 SMs at small batch); each split writes its (m, l, O) and a second small
// kernel merges them. Sequence length zero gives zeros.
#include "common.cuh"

namespace yb {
namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kAttnDepth = 3;     // K/V tiles in flight per warp
constexpr int kTileTokens = 16;
constexpr int kMaxSplits = 32;
constexpr float kNegBig = -1e30f;  // running-max sentinel (finite: -inf - -inf would be NaN)

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// 16-byte asynchronous copy; `valid` false writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct AttnParams {
    const __half* q;
    const __half* kcache;
    const __half* vcache;
    const int* page_table;
    const int* seq_lens;
    __half* out;
    float* part_o;   // [seq][q_head][split][D] when splits > 1
    float* part_ml;  // [seq][q_head][split][2]
    int num_q_heads, num_kv_heads, page_size, max_pages, splits;
    float scale_log2e;  // (1 / sqrt(D)) * log2(e)
};

template <int D>
struct AttnCfg {
    static constexpr int row_bytes = D * 2;
    static constexpr int chunks_per_row = D / 8;  // 16-byte chunks
    static constexpr int tile_bytes = kTileTokens * row_bytes;
    static constexpr int stage_bytes = 2 * tile_bytes;  // K then V
    static constexpr int warp_bytes = kAttnDepth * stage_bytes;
    static constexpr int merge_bytes = (16 * D + 32) * 4;  // one warp's O, m, l as f32
    static constexpr int smem_bytes = kAttnWarps * (warp_bytes > merge_bytes ? warp_bytes : merge_bytes);
};

template <int D>
__global__ void __launch_bounds__(kAttnThreads)
    paged_decode_attention_kernel(const AttnParams p) {
    using Cfg = AttnCfg<D>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, c4 = lane & 3;
    const int kvh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z;
    const int group = p.num_q_heads / p.num_kv_heads;  // query heads per KV head, <= 16
    pdl_wait();  // q and the newest K/V rows come from the kernels before this one
    // A length beyond the page table's reach would index past this sequence's row of it;
    // lengths are device data the host never sees, so they are clamped here.
    const int seq_len = min(max(p.seq_lens[seq], 0), p.max_pages * p.page_size);
    const int tiles = (seq_len + kTileTokens - 1) / kTileTokens;
    const int tiles_per_split = (tiles + p.splits - 1) / p.splits;
    const int tile_begin = split * tiles_per_split;
    const int tile_end = min(tiles, tile_begin + tiles_per_split);

    uint8_t* my_stage = smem + (size_t)warp * Cfg::warp_bytes;
    const uint32_t stage0 = smem_u32(my_stage);

    // ---- Q fragments of the group: row r < group is query head kvh * group + r ------------------
    uint32_t qa[D / 16][4];
    {
        const __half* qbase = p.q + ((size_t)seq * p.num_q_heads + (size_t)kvh * group) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int k0 = ks * 16 + 2 * c4;
            qa[ks][0] = gq < group ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)gq * D + k0) : 0u;
            qa[ks][1] = gq + 8 < group ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(gq + 8) * D + k0) : 0u;
            qa[ks][2] = gq < group ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)gq * D + k0 + 8) : 0u;
            qa[ks][3] = gq + 8 < group ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)(gq + 8) * D + k0 + 8) : 0u;
        }
    }

    // ---- this warp's tiles: tile_begin + warp, + kAttnWarps, ... -------------------------------
    const int* pt_row = p.page_table + (size_t)seq * p.max_pages;
    auto request = [&](int tile, int slot) {
        if (tile < tile_end) {
            const int t0 = tile * kTileTokens;
            // lanes 0..15 look up the cache row of token t0 + lane; everyone gets rows by shuffle
            long long row_elem = -1;  // element offset of the token's [D] row of this KV head
            if (lane < kTileTokens && t0 + lane < seq_len) {
                const int t = t0 + lane;
                const int page = pt_row[t / p.page_size];
                row_elem = (((long long)page * p.page_size + t % p.page_size) * p.num_kv_heads + kvh) * D;
            }
            const uint32_t kdst = stage0 + slot * Cfg::stage_bytes;
#pragma unroll
            for (int i = 0; i < Cfg::tile_bytes / 16 / 32; ++i) {
                const int ch = lane + 32 * i;
                const int r = ch / Cfg::chunks_per_row, c = ch % Cfg::chunks_per_row;
                const long long re = __shfl_sync(0xffffffffu, row_elem, r);
                const bool valid = re >= 0;
                const size_t off = (size_t)(valid ? re : 0) + (size_t)c * 8;
                const uint32_t dst = kdst + r * Cfg::row_bytes + ((c ^ (r & 7)) * 16);
                cp_async_16_zfill(dst, p.kcache + off, valid);
                cp_async_16_zfill(dst + Cfg::tile_bytes, p.vcache + off, valid);
            }
        }
        cp_commit();
    };
    int ahead = tile_begin + warp;
#pragma unroll 1
    for (int i = 0; i < kAttnDepth; ++i, ahead += kAttnWarps) request(ahead, i);

    float m_run[2] = {kNegBig, kNegBig};  // rows gq and gq + 8
    float l_run[2] = {0.0f, 0.0f};        // this lane's share of the row sums
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    int slot = 0;
    for (int tile = tile_begin + warp; tile < tile_end; tile += kAttnWarps) {
        cp_wait<kAttnDepth - 1>();
        __syncwarp();
        const uint32_t kbase = stage0 + slot * Cfg::stage_bytes, vbase = kbase + Cfg::tile_bytes;
        // ---- S = Q K^T for 16 tokens: two 8-token column tiles ---------------------------------
        float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
        {
            const int mi = lane >> 3, ri = lane & 7;
            const int r = ri + 8 * (mi >> 1);  // token row of the 8x8 block this lane addresses
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int c = 2 * ks + (mi & 1);
                uint32_t kb[4];
                ldmatrix_x4(kbase + r * Cfg::row_bytes + ((c ^ (r & 7)) * 16), kb);
                mma16816(s[0], qa[ks], kb[0], kb[1]);
                mma16816(s[1], qa[ks], kb[2], kb[3]);
            }
        }
        // ---- online softmax (exp2 domain); tokens past the sequence end are masked out --------
        const int t0 = tile * kTileTokens;
        float mx[2] = {kNegBig, kNegBig};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = t0 + 8 * nt + 2 * c4 + (e & 1);
                const float v = t < seq_len ? s[nt][e] * p.scale_log2e : kNegBig;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
        uint32_t pa[4];
        {
            float pv[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // a masked token has s = -1e30: exp2 of it is 0 whatever the running max is,
                    // except when the whole row is still at the sentinel (no token yet), so test it
                    const float pe = s[nt][e] <= kNegBig ? 0.0f : exp2f(s[nt][e] - m_run[e >> 1]);
                    pv[nt][e] = pe;
                    l_run[e >> 1] += pe;
                }
            pa[0] = pack_f16x2(pv[0][0], pv[0][1]);  // row gq,     tokens 2c..2c+1
            pa[1] = pack_f16x2(pv[0][2], pv[0][3]);  // row gq + 8, tokens 2c..2c+1
            pa[2] = pack_f16x2(pv[1][0], pv[1][1]);  // row gq,     tokens 8 + 2c..
            pa[3] = pack_f16x2(pv[1][2], pv[1][3]);  // row gq + 8, tokens 8 + 2c..
        }
        // ---- O = O * corr + P V -------------------------------------------------------------------
        {
            const int mi = lane >> 3, ri = lane & 7;
            const int r = ri + 8 * (mi & 1);  // token row addressed by this lane
#pragma unroll
            for (int j = 0; j < D / 8; j += 2) {
                const int c = j + (mi >> 1);
                uint32_t vb[4];
                ldmatrix_x4_trans(vbase + r * Cfg::row_bytes + ((c ^ (r & 7)) * 16), vb);
                o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
                o[j + 1][0] *= corr[0]; o[j + 1][1] *= corr[0]; o[j + 1][2] *= corr[1]; o[j + 1][3] *= corr[1];
                mma16816(o[j], pa, vb[0], vb[1]);
                mma16816(o[j + 1], pa, vb[2], vb[3]);
            }
        }
        __syncwarp();
        request(ahead, slot);
        ahead += kAttnWarps;
        if (++slot == kAttnDepth) slot = 0;
    }
    cp_wait<0>();
    pdl_launch_dependents();  // the merge kernel (or the caller's next one) may become resident

    // ---- merge the warps' states, then write the CTA's result -----------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    __syncthreads();  // every warp is done with its staging area, which the merge reuses
    float* mo = reinterpret_cast<float*>(smem + (size_t)warp * Cfg::merge_bytes);  // [16][D] then m[16], l[16]
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        *reinterpret_cast<float2*>(mo + gq * D + j * 8 + 2 * c4) = make_float2(o[j][0], o[j][1]);
        *reinterpret_cast<float2*>(mo + (gq + 8) * D + j * 8 + 2 * c4) = make_float2(o[j][2], o[j][3]);
    }
    if (c4 == 0) {
        mo[16 * D + gq] = m_run[0];
        mo[16 * D + gq + 8] = m_run[1];
        mo[16 * D + 16 + gq] = l_run[0];
        mo[16 * D + 16 + gq + 8] = l_run[1];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < group * D; e += kAttnThreads) {
        const int r = e / D, d = e % D;
        float M = kNegBig;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w)
            M = fmaxf(M, reinterpret_cast<const float*>(smem + (size_t)w * Cfg::merge_bytes)[16 * D + r]);
        float L = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float* wo = reinterpret_cast<const float*>(smem + (size_t)w * Cfg::merge_bytes);
            const float f = exp2f(wo[16 * D + r] - M);  // a warp without tokens: exp2(-1e30 - M) = 0
            L += f * wo[16 * D + 16 + r];
            acc += f * wo[r * D + d];
        }
        const int qh = kvh * group + r;
        if (p.splits == 1) {
            p.out[((size_t)seq * p.num_q_heads + qh) * D + d] = __float2half_rn(L > 0.0f ? acc / L : 0.0f);
        } else {
            const size_t slot_id = ((size_t)seq * p.num_q_heads + qh) * p.splits + split;
            p.part_o[slot_id * D + d] = acc;
            if (d == 0) {
                p.part_ml[slot_id * 2] = M;
                p.part_ml[slot_id * 2 + 1] = L;
            }
        }
    }
}

// grid (num_q_heads, num_seqs), D threads: out = sum_i 2^(m_i - M) O_i / sum_i 2^(m_i - M) l_i
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __half* __restrict__ out, int num_q_heads, int splits, int D) {
    const size_t head = (size_t)blockIdx.y * num_q_heads + blockIdx.x;
    const float* ml = part_ml + head * splits * 2;
    pdl_wait();  // the splits' partial states are complete and visible
    float M = kNegBig;
    for (int i = 0; i < splits; ++i) M = fmaxf(M, ml[2 * i]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.0f, acc = 0.0f;
        for (int i = 0; i < splits; ++i) {
            const float f = exp2f(ml[2 * i] - M);
            L += f * ml[2 * i + 1];
            acc += f * part_o[(head * splits + i) * D + d];
        }
        out[head * D + d] = __float2half_rn(L > 0.0f ? acc / L : 0.0f);
    }
}

// CTAs of the kernel that one SM holds at a time: shared memory decides (three K/V tiles per
// warp in flight), 227 KB per SM less 1 KB that the system keeps per resident CTA.
int ctas_per_sm(int head_dim) {
    const int smem = head_dim == 64 ? AttnCfg<64>::smem_bytes
                     : head_dim == 128 ? AttnCfg<128>::smem_bytes
                                       : AttnCfg<256>::smem_bytes;
    const int n = (227 * 1024) / (smem + 1024);
    return n < 1 ? 1 : (n > 4 ? 4 : n);
}

int choose_splits(int num_seqs, int num_kv_heads, int head_dim) {
    // As many CTAs as are resident at once, and no more: a few CTAs left over for a second
    // wave would stream their share alone, far below the HBM rate. Empty splits (a sequence
    // shorter than its share) write neutral states.
    const long long base = (long long)num_seqs * num_kv_heads;
    long long want = (long long)sm_count() * ctas_per_sm(head_dim) / base;
    if (want < 1) want = 1;
    if (want > kMaxSplits) want = kMaxSplits;
    return (int)want;
}

template <int D>
int launch_attention(const AttnParams& p, int num_seqs, cudaStream_t st) {
    using Cfg = AttnCfg<D>;
    static bool configured[64] = {};
    int dev = 0;
    YB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        YB_CUDA(cudaFuncSetAttribute(paged_decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::smem_bytes));
        configured[dev] = true;
    }
    dim3 grid((unsigned)p.num_kv_heads, (unsigned)num_seqs, (unsigned)p.splits);
    YB_CUDA(launch_pdl(paged_decode_attention_kernel<D>, grid, dim3(kAttnThreads), Cfg::smem_bytes, st, p));
    if (p.splits > 1) {
        dim3 mgrid((unsigned)p.num_q_heads, (unsigned)num_seqs);
        YB_CUDA(launch_pdl(attention_merge_kernel, mgrid, dim3(D < 128 ? D : 128), 0, st, p.part_o, p.part_ml, p.out,
                           p.num_q_heads, p.splits, D));
    }
    return 0;
}

}  // namespace
}  // namespace yb

using namespace yb;

extern "C" size_t y_b200_paged_decode_attention_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                                                int head_dim) {
    if (num_seqs < 1 || num_q_heads < 1 || num_kv_heads < 1 || head_dim < 1) return 0;
    const int splits = choose_splits(num_seqs, num_kv_heads, head_dim);
    if (splits == 1) return 256;
    const size_t heads = (size_t)num_seqs * num_q_heads * splits;
    return ((heads * head_dim * 4 + 255) & ~(size_t)255) + ((heads * 8 + 255) & ~(size_t)255);
}

extern "C" int y_b200_paged_decode_attention(const void* q_f16, const void* kcache_f16, const void* vcache_f16,
                                             const int32_t* page_table, const int32_t* seq_lens, void* out_f16,
                                             int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                             int page_size, int max_pages, void* workspace, size_t workspace_bytes,
                                             void* stream) {
    if (!q_f16 || !kcache_f16 || !vcache_f16 || !page_table || !seq_lens || !out_f16)
        return fail(Y_B200_ERR_INVALID, "y_b200_paged_decode_attention: null pointer");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        return fail(Y_B200_ERR_SHAPE, "y_b200_paged_decode_attention: head_dim=%d must be 64, 128 or 256", head_dim);
    if (num_seqs < 0 || num_q_heads < 1 || num_kv_heads < 1 || num_q_heads % num_kv_heads != 0 ||
        num_q_heads / num_kv_heads > 16 || page_size < 1 || max_pages < 1)
        return fail(Y_B200_ERR_SHAPE,
                    "y_b200_paged_decode_attention: need num_q_heads a multiple of num_kv_heads with at most 16 query "
                    "heads per KV head, page_size >= 1, max_pages >= 1 (q=%d kv=%d page=%d max_pages=%d)",
                    num_q_heads, num_kv_heads, page_size, max_pages);
    if ((reinterpret_cast<uintptr_t>(q_f16) & 15u) || (reinterpret_cast<uintptr_t>(kcache_f16) & 15u) ||
        (reinterpret_cast<uintptr_t>(vcache_f16) & 15u) || (reinterpret_cast<uintptr_t>(out_f16) & 1u))
        return fail(Y_B200_ERR_ALIGN, "y_b200_paged_decode_attention: q and the caches must be 16-byte aligned");
    if (num_seqs == 0) return Y_B200_OK;
    if (num_seqs > 65535) return fail(Y_B200_ERR_SHAPE, "y_b200_paged_decode_attention: at most 65535 sequences per call");
    AttnParams p = {};
    p.q = static_cast<const __half*>(q_f16);
    p.kcache = static_cast<const __half*>(kcache_f16);
    p.vcache = static_cast<const __half*>(vcache_f16);
    p.page_table = page_table;
    p.seq_lens = seq_lens;
    p.out = static_cast<__half*>(out_f16);
    p.num_q_heads = num_q_heads;
    p.num_kv_heads = num_kv_heads;
    p.page_size = page_size;
    p.max_pages = max_pages;
    p.splits = choose_splits(num_seqs, num_kv_heads, head_dim);
    p.scale_log2e = (float)(1.4426950408889634 / sqrt((double)head_dim));
    if (p.splits > 1) {
        const size_t need = y_b200_paged_decode_attention_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim);
        if (!workspace || workspace_bytes < need)
            return fail(Y_B200_ERR_WORKSPACE, "y_b200_paged_decode_attention: workspace needs %zu bytes", need);
        if (reinterpret_cast<uintptr_t>(workspace) & 255u)
            return fail(Y_B200_ERR_ALIGN, "y_b200_paged_decode_attention: workspace needs 256-byte alignment");
        const size_t heads = (size_t)num_seqs * num_q_heads * p.splits;
        p.part_o = static_cast<float*>(workspace);
        p.part_ml = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((heads * head_dim * 4 + 255) & ~(size_t)255));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (head_dim) {
        case 64: return launch_attention<64>(p, num_seqs, st);
        case 128: return launch_attention<128>(p, num_seqs, st);
        default: return launch_attention<256>(p, num_seqs, st);
    }
}
