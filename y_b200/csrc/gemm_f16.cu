// F16-operand entries around the tensor-core GEMM: the K-major weight copy that lets the
// reference's row-major B [K, N] feed the tcgen05 kernels, the drop-ins for gemm_f16_<tag>,
// gemm_f16_bias_relu_<tag> and gemm_f16_swiglu_<tag>, and the small-M weight-streaming GEMM
// behind gemm_f16_decode_m<M> with the reference's split-K pair on top of it.
#include "common.cuh"

namespace yb {
namespace {

// ---- K-major weight copy -----------------------------------------------------------------
// dst[(c * dst_mul + dst_off) * rows + r] = src[r * cols + c] for a row-major f16 matrix
// src [rows, cols]: the transpose, optionally written to every dst_mul-th row (the SwiGLU
// entry interleaves gate and up columns this way). 64 x 64 tiles through shared memory,
// 16-byte accesses on both sides when the shape allows, element-wise at ragged edges.
constexpr int kTT = 64;
constexpr int kTPad = 66;  // row stride of 33 words: the scattered 2-byte writes and the 4-byte reads both spread over all banks

__global__ void __launch_bounds__(256)
    transpose_f16_kernel(const uint16_t* __restrict__ src, int rows, int cols, uint16_t* __restrict__ dst,
                         int dst_mul, int dst_off) {
    __shared__ __align__(16) uint16_t tile[kTT][kTPad];  // tile[c][r]
    pdl_wait();
    pdl_launch_dependents();
    const int r0 = blockIdx.y * kTT, c0 = blockIdx.x * kTT;
    const bool vec_in = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const bool vec_out = rows % 8 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = (threadIdx.x >> 3) + 32 * i, c8 = (threadIdx.x & 7) * 8;
        const int gr = r0 + r, gc = c0 + c8;
        uint16_t v[8];
        if (gr < rows && vec_in && gc + 8 <= cols) {
            const uint4 u = *reinterpret_cast<const uint4*>(src + (size_t)gr * cols + gc);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] = (uint16_t)(w[j] & 0xffffu); v[2 * j + 1] = (uint16_t)(w[j] >> 16); }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (gr < rows && gc + j < cols) ? src[(size_t)gr * cols + gc + j] : (uint16_t)0;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[c8 + j][r] = v[j];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = (threadIdx.x >> 3) + 32 * i, r8 = (threadIdx.x & 7) * 8;
        const int gc = c0 + c, gr = r0 + r8;
        if (gc >= cols || gr >= rows) continue;
        const uint32_t* t32 = reinterpret_cast<const uint32_t*>(&tile[c][r8]);
        const uint32_t w[4] = {t32[0], t32[1], t32[2], t32[3]};
        uint16_t* d = dst + ((size_t)gc * dst_mul + dst_off) * rows + gr;
        if (vec_out && gr + 8 <= rows) {
            *reinterpret_cast<uint4*>(d) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            for (int j = 0; j < 8; ++j)
                if (gr + j < rows) d[j] = (uint16_t)(w[j >> 1] >> (16 * (j & 1)));
        }
    }
}

int launch_transpose(const void* src, int rows, int cols, void* dst, int dst_mul, int dst_off, cudaStream_t st) {
    dim3 grid((unsigned)((cols + kTT - 1) / kTT), (unsigned)((rows + kTT - 1) / kTT));
    return check_cuda(launch_pdl(transpose_f16_kernel, grid, dim3(256), 0, st, static_cast<const uint16_t*>(src), rows, cols,
                                 static_cast<uint16_t*>(dst), dst_mul, dst_off),
                      "transpose_f16_kernel launch");
}

// ---- small-M weight-streaming GEMM ---------------------------------------------------------
// out [M, N] = x [M, K] @ w [K, N], M <= 32. HBM-bound: the K * N * 2 bytes of w are read once.
// A CTA of 8 warps owns 64 output columns, i.e. a 128-byte run of every weight row it reads
// (64-byte runs reached a quarter of the HBM copy rate: too little per DRAM page). K is cut two
// ways. Across CTAs: a thread-block cluster of S CTAs shares the 64 columns, CTA r taking the
// r-th contiguous K slab, so that small N still fills the GPU (N = 4096: 64 column blocks x 4).
// Inside a CTA: the slab is cut into steps of 32 rows, warp v takes the v-th contiguous eighth
// of them and streams it through a private ring of 4 KB slots filled by per-thread 16-byte
// cp.async copies (no producer warp, no barrier another agent has to complete). A step is two
// mma.sync.m16n8k16 per 16 columns and 8 tokens: the weights are the 16-row operand, read from
// the slot with ldmatrix.trans (w is row-major along N), the tokens the 8-wide one, so up to 8
// tokens cost one MMA per 256 weights. (With the tokens as the 16-row operand it was one per
// 128 weights whatever the token count, and at K = N = 4096 the steps of a CTA took as long as
// the tensor pipe needs for them: mma.sync issues one m16n8k16 every 16 cycles per scheduler.)
//
// The 32 rows of a step are dealt to the two MMAs so that a thread's token fragments are
// contiguous in memory: thread (g, c) of a warp holds token g (and g + 8, ... for more than 8
// tokens) at k = 8c .. 8c + 7 of the step (one 16-byte load per token and step), the first MMA
// takes k = 8c .. 8c + 3 as its slots (2c, 2c + 1, 2c + 8, 2c + 9) and the second
// k = 8c + 4 .. 8c + 7. ldmatrix takes a row address per lane, so reading the weight rows in
// that order costs nothing. (With the natural order a thread's fragments are 4-byte pieces;
// those loads, four per 16 rows, held the kernel at 0.58 of the copy rate at K = N = 4096 and
// 0.69 at N = 11008.) The 16-byte units of a slot row are XOR-swizzled with the row index,
// so the eight row addresses of an ldmatrix phase hit eight different bank groups.
//
// The partial tiles of a cluster meet without anyone waiting twice: after its cross-warp sum
// every CTA stores each 1/S of its tile into the shared memory of the CTA that owns that part
// (distributed shared memory, a region the rings never touch), one cluster barrier follows, and
// every CTA adds the S parts it received in rank order and writes its share of the output.
// All sums are added in a fixed order (warp order, then cluster rank order): no atomics,
// overwrite semantics, run-to-run identical.
constexpr int kDecWarps = 8;
constexpr int kDecCols = 64;
constexpr int kDecStepRows = 32;
constexpr int kDecStages = 3;  // slots of a warp's ring (two are used with 9 to 16 tokens, see the kernel)
constexpr int kDecSlotBytes = kDecStepRows * kDecCols * 2;  // 4 KB
constexpr int kDecRingBytes = kDecWarps * kDecStages * kDecSlotBytes;  // 96 KB
constexpr int kDecRecvBytes = 2 * 8 * 32 * 16;  // one reduced tile of up to 32 tokens x 64 columns, f32: 8 KB
constexpr int kDecSmemBytes = kDecRingBytes + kDecRecvBytes;  // 104 KB: two CTAs per SM

__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst_smem, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void st_shared_cluster_f32x4(uint32_t cluster_addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// XOR key of a slot row's 16-byte units. The eight rows one ldmatrix phase reads are
// 8c' + j + const (c' = 0..3, j = 0, 1): their keys are the eight values 2c' + j.
__device__ __forceinline__ int swizzle_key(int row) { return ((row >> 3) << 1) | (row & 1); }

template <int NT, typename OutT>
__global__ void __launch_bounds__(kDecWarps * 32, 2)
    f16_decode_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ w, OutT* __restrict__ out,
                      int M, int N, int K) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(), nranks = cluster_nctarank();
    // First phase of the cluster barrier: "this CTA runs" (nobody waits for it before the tail).
    if (nranks > 1) cluster_arrive_relaxed();
    const int n0 = (int)(blockIdx.x / nranks) * kDecCols;
    // This CTA's K slab, in steps of 32 rows (the host makes the step count a multiple of the
    // cluster size; the last step of the matrix may hold 16 rows of zeros).
    const int slab_steps = (K + kDecStepRows - 1) / kDecStepRows / (int)nranks;
    const int per_warp = (slab_steps + kDecWarps - 1) / kDecWarps;
    const int my_steps = max(0, min(per_warp, slab_steps - warp * per_warp));
    const int step0 = (int)rank * slab_steps + warp * per_warp;  // this warp's first step
    // Steps in flight per warp. With two token tiles two are faster than three (7.7 against
    // 7.9 us at 16 tokens, K = N = 4096; 17.0 against 17.8 at N = 11008); with one tile the third
    // pays (6.5 against 6.7 us at up to 8 tokens).
    constexpr int kStages = NT == 2 ? 2 : kDecStages;
    const uint32_t ring = smem_u32(smem) + warp * (kDecStages * kDecSlotBytes);
    pdl_launch_dependents();

    // This lane's eight 16-byte units of a slot: rows lane / 8 + 4 j, unit lane % 8.
    const int crow = lane >> 3, cunit = lane & 7;
    const bool col_ok = n0 + cunit * 8 < N;  // N % 8 == 0: a unit is wholly inside or outside
    const int krow0 = kDecStepRows * step0 + crow;
    // columns beyond N and rows beyond K are zero-filled without a read from a valid address
    const __half* wsrc = w + (col_ok ? n0 + cunit * 8 : 0);
    auto request = [&](int i) {  // step i of this warp into slot i % kStages; always commits a group
        if (i < my_steps) {
            const uint32_t slot = ring + (i % kStages) * kDecSlotBytes;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int row = crow + 4 * j, k = krow0 + kDecStepRows * i + 4 * j;
                const bool ok = col_ok && k < K;
                cp_async_16_zfill(slot + row * 128 + ((cunit ^ swizzle_key(row)) << 4), wsrc + (size_t)(ok ? k : 0) * N, ok);
            }
        }
        cp_async_commit();
    };
    // The weights do not depend on the kernel before this one: the ring fills before the wait.
#pragma unroll 1
    for (int i = 0; i < kStages; ++i) request(i);
    pdl_wait();  // x is the previous kernel's output

    const int g = lane >> 2, c = lane & 3;
    // ldmatrix row of this lane: matrices 0 and 2 of an x4 call are the MMA's K slots 0..7,
    // matrices 1 and 3 its slots 8..15; slot 2c' + j (+ 8) of MMA e is row 8c' + 4e + j (+ 2)
    // of the step. Call t reads the 16-byte units 2t and 2t + 1.
    const int khalf = (lane >> 3) & 1, munit = lane >> 4;
    const int mrow0 = 8 * ((lane & 7) >> 1) + 2 * khalf + (lane & 1);  // MMA 0; MMA 1 is 4 rows further

    // acc[t][j]: weight columns 16t + g (+ 8) of the CTA's 64, tokens 8j + 2c (+ 1)
    float acc[4][NT][4];
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][j][i] = 0.0f;

    // Token fragments of one step: token 8j + g, k = 32 (step0 + i) + 8c + (0..7).
    auto load_a = [&](int i, uint4 (&a)[NT]) {
        const int k0 = kDecStepRows * (step0 + i) + 8 * c;
        const bool live = i < my_steps && k0 < K;  // K % 8 == 0
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int tok = 8 * j + g;
            a[j] = make_uint4(0u, 0u, 0u, 0u);
            if (live && tok < M) a[j] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + k0));
        }
    };
    // Token fragments are loaded this many steps before their MMAs. With four token tiles a
    // deeper prefetch costs the registers that let two CTAs share an SM.
    constexpr int kAhead = NT == 1 ? 4 : 2;
    uint4 a[kAhead][NT];
#pragma unroll
    for (int j = 0; j < kAhead; ++j) load_a(j, a[j]);
#pragma unroll 1
    for (int i0 = 0; i0 < my_steps; i0 += kAhead) {
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
            const int i = i0 + j;
            if (i < my_steps) {  // uniform across the warp
                cp_async_wait<kStages - 1>();  // all but the newest kStages - 1 groups: step i has landed
                __syncwarp();
                const uint32_t slot = ring + (i % kStages) * kDecSlotBytes;
                // The weights are the 16-row operand (16 columns x 16 K slots per MMA, so up to 8
                // tokens cost one MMA per 256 weights), the tokens the 8-wide one. ldmatrix call t
                // returns (K slots 0..7, columns 16t..16t+7), (slots 8..15, same columns), and
                // the same two for columns 16t+8..16t+15: fragment registers 0, 2, 1, 3. With
                // more than 16 tokens the two MMAs' weight fragments are read one after the other
                // (16 registers instead of 32, which a token prefetch two steps deep needs:
                // 11.0 against 11.3 us at 32 tokens, K = N = 4096; at 16 tokens it costs 4 %).
                auto mmas = [&](int e, const uint32_t (&b)[4][4]) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint32_t wf[4] = {b[t][0], b[t][2], b[t][1], b[t][3]};
#pragma unroll
                        for (int jt = 0; jt < NT; ++jt)
                            mma_16816(acc[t][jt], wf, e == 0 ? a[j][jt].x : a[j][jt].z, e == 0 ? a[j][jt].y : a[j][jt].w);
                    }
                };
                auto read_weights = [&](int e, uint32_t (&b)[4][4]) {
                    const int r = mrow0 + 4 * e;
#pragma unroll
                    for (int t = 0; t < 4; ++t)
                        ldmatrix_x4_trans(slot + r * 128 + (((2 * t + munit) ^ swizzle_key(r)) << 4), b[t]);
                };
                if constexpr (NT <= 2) {
                    uint32_t b0[4][4], b1[4][4];
                    read_weights(0, b0);
                    read_weights(1, b1);
                    __syncwarp();  // every lane has read the slot
                    request(i + kStages);
                    mmas(0, b0);
                    mmas(1, b1);
                } else {
                    uint32_t b[4][4];
                    read_weights(0, b);
                    mmas(0, b);
                    read_weights(1, b);
                    __syncwarp();  // every lane has read the slot
                    request(i + kStages);
                    mmas(1, b);
                }
                load_a(i + kAhead, a[j]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // the rings are free: they become the reduction area
    float* red = reinterpret_cast<float*>(smem);
    constexpr int kPerWarp = 4 * NT * 32 * 4;  // floats a warp contributes (at most 8 KB)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int j = 0; j < NT; ++j)
            *reinterpret_cast<float4*>(red + warp * kPerWarp + ((t * NT + j) * 32 + lane) * 4) =
                make_float4(acc[t][j][0], acc[t][j][1], acc[t][j][2], acc[t][j][3]);
    __syncthreads();
    // Cross-warp sum in warp order: thread e4 adds the warps' copies of one lane's four
    // accumulators of one (token tile, column tile), all reads issued together, and hands the
    // result to the CTA that owns that part of the tile (part r of rank r's region there).
    constexpr int kPerWarp4 = kPerWarp / 4;
    const int chunk = kPerWarp4 / (int)nranks;  // nranks is 1, 2, 4 or 8
    const uint32_t recv = smem_u32(smem) + kDecRingBytes;  // [nranks][chunk] float4, written by the cluster
    if (nranks > 1) cluster_wait_acquire();  // every CTA of the cluster runs: its shared memory may be written
    for (int e4 = threadIdx.x; e4 < kPerWarp4; e4 += kDecWarps * 32) {
        float4 p[kDecWarps];
#pragma unroll
        for (int wv = 0; wv < kDecWarps; ++wv) p[wv] = *reinterpret_cast<const float4*>(red + wv * kPerWarp + e4 * 4);
        float4 v = p[0];
#pragma unroll
        for (int wv = 1; wv < kDecWarps; ++wv) {
            v.x += p[wv].x;
            v.y += p[wv].y;
            v.z += p[wv].z;
            v.w += p[wv].w;
        }
        const int owner = e4 / chunk, idx = e4 - owner * chunk;
        st_shared_cluster_f32x4(mapa_shared(recv + 16u * (uint32_t)((int)rank * chunk + idx), (uint32_t)owner), v);
    }
    // Second phase: every part has been stored (release) and is visible here (acquire). After it
    // nobody touches another CTA's shared memory, so a CTA may leave as soon as it has written.
    if (nranks > 1) {
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < chunk; idx += kDecWarps * 32) {
        const float4* part = reinterpret_cast<const float4*>(smem + kDecRingBytes) + idx;
        float4 p[8];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r)
            if (r < nranks) p[r] = part[(int)r * chunk];
        float4 v = p[0];
#pragma unroll
        for (uint32_t r = 1; r < 8; ++r)
            if (r < nranks) {
                v.x += p[r].x;
                v.y += p[r].y;
                v.z += p[r].z;
                v.w += p[r].w;
            }
        const int e4 = (int)rank * chunk + idx;
        const int l = e4 & 31, tj = e4 >> 5;
        const int col = n0 + 16 * (tj / NT) + (l >> 2), tok = 8 * (tj % NT) + 2 * (l & 3);
        const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int cc = col + 8 * (i >> 1), tt = tok + (i & 1);  // N % 8 == 0: cc < N whenever col < N
            if (cc < N && tt < M) {
                if constexpr (sizeof(OutT) == 4) out[(size_t)tt * N + cc] = vv[i];
                else out[(size_t)tt * N + cc] = __float2half_rn(vv[i]);
            }
        }
    }
}

// Cluster size (K slabs per 64-column block): the largest of 8, 4, 2, 1 that divides the number
// of 32-row steps and keeps the grid within two CTAs per SM, so narrow matrices still spread
// over the whole GPU.
int decode_k_slabs(int n, int k, int sms = 0) {
    const int blocks = (n + kDecCols - 1) / kDecCols;
    const int steps = (k + kDecStepRows - 1) / kDecStepRows;
    const int cap = 2 * (sms > 0 ? sms : sm_count());
    for (int s = 8; s > 1; s >>= 1)
        if (steps % s == 0 && blocks * s <= cap) return s;
    return 1;
}

template <int NT, typename OutT>
int launch_f16_decode(const void* x, int ldx, const void* w, void* out, int m, int n, int k, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    YB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        YB_CUDA(cudaFuncSetAttribute(f16_decode_kernel<NT, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes));
        configured[dev] = true;
    }
    const int slabs = decode_k_slabs(n, k);
    const unsigned grid = (unsigned)((n + kDecCols - 1) / kDecCols) * (unsigned)slabs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDecWarps * 32);
    cfg.dynamicSmemBytes = kDecSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)slabs;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return check_cuda(cudaLaunchKernelEx(&cfg, f16_decode_kernel<NT, OutT>, static_cast<const __half*>(x), ldx,
                                         static_cast<const __half*>(w), static_cast<OutT*>(out), m, n, k),
                      "f16_decode_kernel launch");
}

// C [M, N] f16 = sum over splits (in split order) of workspace [k_splits, M, N] f32.
__global__ void __launch_bounds__(256)
    splitk_reduction_kernel(const float* __restrict__ ws, __half* __restrict__ c, size_t total, int k_splits) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (size_t)gridDim.x * 256) {
        float v = ws[i];
        for (int s = 1; s < k_splits; ++s) v += ws[(size_t)s * total + i];
        c[i] = __float2half_rn(v);
    }
}

size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

// Launch geometry of the weight-streaming kernel for the host launch API.
// `sms` > 0: for a GPU with that many multiprocessors (no device needed); 0: the current device.
void f16_decode_launch_geometry(int n, int k, int sms, unsigned* grid, unsigned* block, unsigned* smem, int* stages,
                                unsigned* cluster) {
    *cluster = (unsigned)decode_k_slabs(n, k, sms);
    *grid = (unsigned)((n + kDecCols - 1) / kDecCols) * *cluster;
    *block = kDecWarps * 32;
    *smem = kDecSmemBytes;
    *stages = kDecStages;
}

}  // namespace yb

namespace yb {
bool umma_decode_applies(int m, int n, int k);
int launch_umma_decode(const void* x, int ldx, const void* w, void* out, bool out_f32, int m, int n, int k, cudaStream_t st);
}  // namespace yb

using namespace yb;

extern "C" int y_b200_gemm_f16_decode(const void* x_f16, int ldx, const void* w_f16, void* out, int out_kind, int m, int n,
                                      int k, void* stream) {
    if (!x_f16 || !w_f16 || !out) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_decode: null pointer");
    if (m < 1 || m > 32) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: M=%d outside 1..32", m);
    if (k < 16 || k % 16 != 0 || n < 8 || n % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: need K %% 16 == 0 and N %% 8 == 0 (K=%d N=%d)", k, n);
    if (ldx < k || ldx % 8 != 0) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: ldx=%d must be a multiple of 8 and >= K", ldx);
    if (out_kind != Y_B200_F32 && out_kind != Y_B200_F16)
        return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_decode: out_kind must be F32 or F16");
    if ((reinterpret_cast<uintptr_t>(w_f16) & 15u) || (reinterpret_cast<uintptr_t>(x_f16) & 15u))
        return fail(Y_B200_ERR_ALIGN, "y_b200_gemm_f16_decode: w and x must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // 17..32 tokens: the tcgen05 kernel (decode_umma.cu) where its shape rules hold; mma.sync
    // issues too slowly for four token tiles per weight fragment.
    if (umma_decode_applies(m, n, k) && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) return launch_umma_decode(x_f16, ldx, w_f16, out, out_kind == Y_B200_F32, m, n, k, st);
    if (out_kind == Y_B200_F32)
        return m <= 8    ? launch_f16_decode<1, float>(x_f16, ldx, w_f16, out, m, n, k, st)
               : m <= 16 ? launch_f16_decode<2, float>(x_f16, ldx, w_f16, out, m, n, k, st)
                         : launch_f16_decode<4, float>(x_f16, ldx, w_f16, out, m, n, k, st);
    return m <= 8    ? launch_f16_decode<1, __half>(x_f16, ldx, w_f16, out, m, n, k, st)
           : m <= 16 ? launch_f16_decode<2, __half>(x_f16, ldx, w_f16, out, m, n, k, st)
                     : launch_f16_decode<4, __half>(x_f16, ldx, w_f16, out, m, n, k, st);
}

extern "C" int y_b200_gemm_f16_splitk_workspace(const void* a_f16, const void* b_f16, float* workspace, int m, int n, int k,
                                                int k_splits, void* stream) {
    if (!a_f16 || !b_f16 || !workspace) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_splitk_workspace: null pointer");
    if (k_splits < 1 || k < 1 || k % (16 * k_splits) != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_splitk_workspace: K=%d must be a multiple of 16 * k_splits (%d)", k, k_splits);
    const int ks = k / k_splits;
    for (int s = 0; s < k_splits; ++s) {
        int rc = y_b200_gemm_f16_decode(static_cast<const __half*>(a_f16) + (size_t)s * ks, k,
                                        static_cast<const __half*>(b_f16) + (size_t)s * ks * n,
                                        workspace + (size_t)s * m * n, Y_B200_F32, m, n, ks, stream);
        if (rc) return rc;
    }
    return 0;
}

extern "C" int y_b200_splitk_reduction(const float* workspace, void* c_f16, size_t total, int m, int n, int k_splits,
                                       void* stream) {
    if (!workspace || !c_f16) return fail(Y_B200_ERR_INVALID, "y_b200_splitk_reduction: null pointer");
    if (m < 1 || n < 1 || k_splits < 1 || total != (size_t)m * (size_t)n)
        return fail(Y_B200_ERR_SHAPE, "y_b200_splitk_reduction: total must equal M * N and k_splits >= 1");
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    return check_cuda(launch_pdl(splitk_reduction_kernel, dim3((unsigned)blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                 workspace, static_cast<__half*>(c_f16), total, k_splits),
                      "splitk_reduction_kernel launch");
}

extern "C" size_t y_b200_gemm_f16_rowmajor_workspace_bytes(int n, int k) {
    if (n < 1 || k < 1) return 0;
    return round256((size_t)n * (size_t)k * 2);
}

extern "C" int y_b200_gemm_f16_rowmajor(const void* a_f16, const void* b_f16, const void* bias, int bias_kind, int relu,
                                        void* c, int out_kind, int m, int n, int k, void* workspace, size_t workspace_bytes,
                                        void* stream) {
    if (!a_f16 || !b_f16 || !c) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_rowmajor: null pointer");
    if (m < 1 || n < 1 || k < 1 || k % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_rowmajor: need M, N >= 1 and K %% 8 == 0 (M=%d N=%d K=%d)", m, n, k);
    const size_t need = y_b200_gemm_f16_rowmajor_workspace_bytes(n, k);
    if (!workspace || workspace_bytes < need)
        return fail(Y_B200_ERR_WORKSPACE, "y_b200_gemm_f16_rowmajor: workspace needs %zu bytes", need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u)
        return fail(Y_B200_ERR_ALIGN, "y_b200_gemm_f16_rowmajor: workspace needs 256-byte alignment");
    int rc = launch_transpose(b_f16, k, n, workspace, 1, 0, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
    y_b200_gemm_f16_args g = {};
    g.a = a_f16; g.bt = workspace; g.c = c;
    g.m = m; g.n = n; g.k = k;
    g.bias = bias; g.bias_kind = bias_kind;
    g.epilogue = bias ? (relu ? Y_B200_EPI_BIAS_RELU : Y_B200_EPI_BIAS) : Y_B200_EPI_NONE;
    if (!bias && relu) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_rowmajor: ReLU is fused with the bias add; pass a bias");
    g.out_kind = out_kind;
    return y_b200_gemm_f16(&g, stream);
}

extern "C" size_t y_b200_gemm_f16_swiglu_workspace_bytes(int n, int k) {
    if (n < 1 || k < 1) return 0;
    return round256((size_t)2 * (size_t)n * (size_t)k * 2);
}

extern "C" int y_b200_gemm_f16_swiglu(const void* x_f16, const void* wgate_f16, const void* wup_f16, float* out, int m, int n,
                                      int k, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x_f16 || !wgate_f16 || !wup_f16 || !out) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_swiglu: null pointer");
    if (m < 1 || n < 1 || k < 1 || k % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_swiglu: need M, N >= 1 and K %% 8 == 0 (M=%d N=%d K=%d)", m, n, k);
    if (n > 0x3fffffff) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_swiglu: N too large");
    const size_t need = y_b200_gemm_f16_swiglu_workspace_bytes(n, k);
    if (!workspace || workspace_bytes < need)
        return fail(Y_B200_ERR_WORKSPACE, "y_b200_gemm_f16_swiglu: workspace needs %zu bytes", need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255u)
        return fail(Y_B200_ERR_ALIGN, "y_b200_gemm_f16_swiglu: workspace needs 256-byte alignment");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // One K-major matrix [2N, K]: row 2j is column j of Wgate, row 2j + 1 column j of Wup, so
    // that a gate/up pair sits in adjacent accumulator columns of the same tile.
    int rc = launch_transpose(wgate_f16, k, n, workspace, 2, 0, st);
    if (rc) return rc;
    if ((rc = launch_transpose(wup_f16, k, n, workspace, 2, 1, st))) return rc;
    y_b200_gemm_f16_args g = {};
    g.a = x_f16; g.bt = workspace; g.c = out;
    g.m = m; g.n = 2 * n; g.k = k;
    g.epilogue = Y_B200_EPI_SWIGLU;
    g.out_kind = Y_B200_F32;
    return y_b200_gemm_f16(&g, stream);
}
