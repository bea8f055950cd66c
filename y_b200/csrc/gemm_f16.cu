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
// r-th contiguous K slab, so that small N still fills the GPU (N = 4096: 64 column blocks x 4);
// the slabs' partial tiles meet in the first CTA's shared memory over distributed shared memory
// and are added there in rank order. Inside a CTA: the slab is cut into steps of 16 rows, warp
// v takes the v-th contiguous eighth of them and streams it through a private ring of 2 KB
// slots filled by per-thread 16-byte cp.async copies (no producer warp, no barrier another
// agent has to complete). A step is one mma.sync.m16n8k16 per 8 columns and 16 tokens: the
// tokens are the 16-row operand, the weights the 8-wide one, read from the slot with
// ldmatrix.trans (w is row-major along N). The token fragments come straight from global
// memory, four steps ahead of their use: consecutive steps of a warp share 128-byte lines of x
// (with steps dealt round-robin to the warps every fragment load went to L2 and the kernel
// spent its time on the long scoreboard: 7 stall cycles per issue, 12 % L1 hits). The 16-byte
// units of a slot row are XOR-swizzled with the row index, so the eight row addresses of an
// ldmatrix phase hit eight different bank groups. All sums are added in a fixed order (warp
// order, then cluster rank order): no atomics, overwrite semantics, run-to-run identical.
constexpr int kDecWarps = 8;
constexpr int kDecCols = 64;
constexpr int kDecStages = 5;
constexpr int kDecSlotBytes = 16 * kDecCols * 2;  // 2 KB
constexpr int kDecSmemBytes = kDecWarps * kDecStages * kDecSlotBytes;  // 80 KB: two CTAs per SM

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
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}

template <int MT, typename OutT>
__global__ void __launch_bounds__(kDecWarps * 32)
    f16_decode_kernel(const __half* __restrict__ x, int ldx, const __half* __restrict__ w, OutT* __restrict__ out,
                      int M, int N, int K) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(), nranks = cluster_nctarank();
    const int n0 = (int)(blockIdx.x / nranks) * kDecCols;
    // This CTA's K slab, in steps of 16 rows (the host makes K / 16 a multiple of the cluster size).
    const int slab_steps = K / 16 / (int)nranks;
    const int per_warp = (slab_steps + kDecWarps - 1) / kDecWarps;
    const int my_steps = max(0, min(per_warp, slab_steps - warp * per_warp));
    const int step0 = (int)rank * slab_steps + warp * per_warp;  // this warp's first step
    const uint32_t ring = smem_u32(smem) + warp * (kDecStages * kDecSlotBytes);
    pdl_launch_dependents();

    // This lane's four 16-byte units of a slot: rows lane / 8 + 4 j, unit lane % 8.
    const int crow = lane >> 3, cunit = lane & 7;
    const bool col_ok = n0 + cunit * 8 < N;  // N % 8 == 0: a unit is wholly inside or outside
    // columns beyond N are zero-filled without a read; their source address stays inside the matrix
    const __half* wsrc = w + (size_t)(16 * step0 + crow) * N + (col_ok ? n0 + cunit * 8 : 0);
    const size_t step_stride = (size_t)16 * N;  // this warp's next step
    auto request = [&](int i) {  // step i of this warp into slot i % kDecStages; always commits a group
        if (i < my_steps) {
            const uint32_t slot = ring + (i % kDecStages) * kDecSlotBytes;
            const __half* s = wsrc + (size_t)i * step_stride;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = crow + 4 * j;
                cp_async_16_zfill(slot + row * 128 + ((cunit ^ (row & 7)) << 4), s + (size_t)(4 * j) * N, col_ok);
            }
        }
        cp_async_commit();
    };
    // The weights do not depend on the kernel before this one: the ring fills before the wait.
#pragma unroll 1
    for (int i = 0; i < kDecStages; ++i) request(i);
    pdl_wait();  // x is the previous kernel's output

    const int g = lane >> 2, c = lane & 3;
    // ldmatrix row address of this lane inside a slot; call t reads the 16-byte units 2t and 2t + 1
    const int mrow = (lane & 7) + 8 * ((lane >> 3) & 1), munit = lane >> 4;

    float acc[MT][8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;

    // Token fragments of one step: rows g and g + 8 of each 16-token tile, k = k0 + 2c (+1), k0 + 8 + 2c (+1).
    auto load_a = [&](int i, uint32_t (&a)[MT][4]) {
        const int k0 = 16 * (step0 + i) + 2 * c;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int ra = 16 * mt + g, rb = ra + 8;
            const bool live = i < my_steps;
            a[mt][0] = a[mt][2] = a[mt][1] = a[mt][3] = 0u;
            if (live && ra < M) {
                a[mt][0] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)ra * ldx + k0));
                a[mt][2] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)ra * ldx + k0 + 8));
            }
            if (live && rb < M) {
                a[mt][1] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)rb * ldx + k0));
                a[mt][3] = __ldg(reinterpret_cast<const uint32_t*>(x + (size_t)rb * ldx + k0 + 8));
            }
        }
    };
    // Token fragments are loaded this many steps before their MMAs. With two 16-token tiles the
    // deeper prefetch costs the registers that let two CTAs share an SM (measured: 22 us against
    // 14.6 us at 32 tokens, K = N = 4096), so it stays at one step there.
    constexpr int kAhead = MT == 1 ? 4 : 1;
    uint32_t a[kAhead][MT][4];
#pragma unroll
    for (int j = 0; j < kAhead; ++j) load_a(j, a[j]);
#pragma unroll 1
    for (int i0 = 0; i0 < my_steps; i0 += kAhead) {
#pragma unroll
        for (int j = 0; j < kAhead; ++j) {
            const int i = i0 + j;
            if (i < my_steps) {  // uniform across the warp
                cp_async_wait<kDecStages - 1>();  // all but the newest kDecStages - 1 groups: step i has landed
                __syncwarp();
                const uint32_t slot = ring + (i % kDecStages) * kDecSlotBytes;
                uint32_t b[4][4];
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    ldmatrix_x4_trans(slot + mrow * 128 + (((2 * t + munit) ^ (mrow & 7)) << 4), b[t]);
                __syncwarp();  // every lane has read the slot
                request(i + kDecStages);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        mma_16816(acc[mt][2 * t], a[j][mt], b[t][0], b[t][1]);
                        mma_16816(acc[mt][2 * t + 1], a[j][mt], b[t][2], b[t][3]);
                    }
                load_a(i + kAhead, a[j]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // the rings are free: they become the reduction area
    float* red = reinterpret_cast<float*>(smem);
    constexpr int kPerWarp = MT * 8 * 32 * 4;  // floats a warp contributes (at most 8 KB)
    float* tile = red + kDecWarps * kPerWarp;   // this CTA's reduced tile, read by the cluster's first CTA
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
            *reinterpret_cast<float4*>(red + warp * kPerWarp + ((mt * 8 + nt) * 32 + lane) * 4) =
                make_float4(acc[mt][nt][0], acc[mt][nt][1], acc[mt][nt][2], acc[mt][nt][3]);
    __syncthreads();
    for (int e = threadIdx.x; e < kPerWarp; e += kDecWarps * 32) {
        float v = red[e];
#pragma unroll
        for (int wv = 1; wv < kDecWarps; ++wv) v += red[wv * kPerWarp + e];
        tile[e] = v;
    }
    if (nranks > 1) cluster_sync_all();  // every CTA's tile is complete and visible across the cluster
    if (rank == 0) {
        const uint32_t tile_addr = smem_u32(tile);
        for (int e = threadIdx.x; e < kPerWarp; e += kDecWarps * 32) {
            float v = tile[e];
            for (uint32_t r = 1; r < nranks; ++r) v += ld_shared_cluster_f32(mapa_shared(tile_addr + 4u * (uint32_t)e, r));
            const int i = e & 3, l = (e >> 2) & 31, nt = (e >> 7) & 7, mt = e >> 10;
            const int row = 16 * mt + (l >> 2) + 8 * (i >> 1);
            const int col = n0 + 8 * nt + 2 * (l & 3) + (i & 1);
            if (row < M && col < N) {
                if constexpr (sizeof(OutT) == 4) out[(size_t)row * N + col] = v;
                else out[(size_t)row * N + col] = __float2half_rn(v);
            }
        }
    }
    if (nranks > 1) cluster_sync_all();  // no CTA leaves while its tile can still be read
}

// Cluster size (K slabs per 64-column block): the largest of 8, 4, 2, 1 that divides K / 16 and
// keeps the grid within two CTAs per SM, so narrow matrices still spread over the whole GPU.
int decode_k_slabs(int n, int k) {
    const int blocks = (n + kDecCols - 1) / kDecCols;
    const int cap = 2 * sm_count();
    for (int s = 8; s > 1; s >>= 1)
        if ((k / 16) % s == 0 && blocks * s <= cap) return s;
    return 1;
}

template <int MT, typename OutT>
int launch_f16_decode(const void* x, int ldx, const void* w, void* out, int m, int n, int k, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    YB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        YB_CUDA(cudaFuncSetAttribute(f16_decode_kernel<MT, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes));
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
    return check_cuda(cudaLaunchKernelEx(&cfg, f16_decode_kernel<MT, OutT>, static_cast<const __half*>(x), ldx,
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
void f16_decode_launch_geometry(int n, int k, unsigned* grid, unsigned* block, unsigned* smem, int* stages, unsigned* cluster) {
    *cluster = (unsigned)decode_k_slabs(n, k);
    *grid = (unsigned)((n + kDecCols - 1) / kDecCols) * *cluster;
    *block = kDecWarps * 32;
    *smem = kDecSmemBytes;
    *stages = kDecStages;
}

}  // namespace yb

using namespace yb;

extern "C" int y_b200_gemm_f16_decode(const void* x_f16, int ldx, const void* w_f16, void* out, int out_kind, int m, int n,
                                      int k, void* stream) {
    if (!x_f16 || !w_f16 || !out) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_decode: null pointer");
    if (m < 1 || m > 32) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: M=%d outside 1..32", m);
    if (k < 16 || k % 16 != 0 || n < 8 || n % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: need K %% 16 == 0 and N %% 8 == 0 (K=%d N=%d)", k, n);
    if (ldx < k || ldx % 2 != 0) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_f16_decode: ldx=%d must be even and >= K", ldx);
    if (out_kind != Y_B200_F32 && out_kind != Y_B200_F16)
        return fail(Y_B200_ERR_INVALID, "y_b200_gemm_f16_decode: out_kind must be F32 or F16");
    if ((reinterpret_cast<uintptr_t>(w_f16) & 15u) || (reinterpret_cast<uintptr_t>(x_f16) & 3u))
        return fail(Y_B200_ERR_ALIGN, "y_b200_gemm_f16_decode: w must be 16-byte and x 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_kind == Y_B200_F32)
        return m <= 16 ? launch_f16_decode<1, float>(x_f16, ldx, w_f16, out, m, n, k, st)
                       : launch_f16_decode<2, float>(x_f16, ldx, w_f16, out, m, n, k, st);
    return m <= 16 ? launch_f16_decode<1, __half>(x_f16, ldx, w_f16, out, m, n, k, st)
                   : launch_f16_decode<2, __half>(x_f16, ldx, w_f16, out, m, n, k, st);
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
