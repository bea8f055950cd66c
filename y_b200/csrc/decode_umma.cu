// F16 weight-streaming GEMM for 17..32 tokens on the tcgen05 tensor cores.
//
// out [M, N] = x [M, K] @ w [K, N], the same contract as y_b200_gemm_f16_decode (the reference's
// gemm_f16_decode_m<M> entries, src/ptx_emitter.rs:4199-4694, with B row-major [K, N]). The
// mma.sync kernel in gemm_f16.cu is bound by the issue rate of mma.sync from 17 tokens on
// (four MMAs per 256 weights, one every 16 cycles per scheduler: 3.8 us of tensor-pipe time at
// K = N = 4096 against 5 us of HBM time, and the two do not overlap inside a launch). Here one
// tcgen05.mma multiplies 128 output columns x 16 K rows of weights by all tokens at once:
//
//   D [128 token rows (32 used), 64 columns] += A [128, 16] * B [16, 64]
//
// with the WEIGHTS as the B operand in MN-major form: w is row-major along N, so a TMA box of
// 64 K rows x 64 columns (128-byte rows, SWIZZLE_128B) lands in shared memory exactly as the
// canonical MN-major SWIZZLE_128B layout wants it (8 units of 16 bytes along N, 8 K rows per
// 1024-byte atom; atoms along K 1024 bytes apart = stride byte offset). No transposing copy,
// no ldmatrix. The tokens are the A
// operand, K-major: a box of 64 K x 32 rows of x (rows beyond M are zero-filled by TMA). The
// MMA reads 128 rows of A; rows 32..127 are whatever follows the box in shared memory, which
// only feeds accumulator rows 32..127, and those are never read.
//
// A CTA owns 64 columns (as wide as the box: twice the column blocks of a 128-column tile, so
// half the cluster size for the same number of CTAs) and one K slab; the slabs of a thread-block cluster meet as in the
// mma.sync kernel: every CTA stores each 1/S of its 32 x 64 tile into the owning CTA's shared
// memory, one cluster barrier, every CTA adds its S parts in rank order and writes its share.
// Roles: warp 0 issues the TMA loads (weights before griddepcontrol.wait, tokens after it) and
// then drains tensor memory (lanes 0..31 belong to warp 0); warp 1 allocates tensor memory and
// issues the MMAs. Every wait is bounded and reports through the per-device status word.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/y_b200.h"
#include "common.cuh"

namespace yb {
namespace {

constexpr int kUdCols = 64;     // output columns per CTA = N of the MMA = one 128-byte run of a weight row
constexpr int kUdKB = 64;       // K rows per stage (one 128-byte swizzle span of x)
// Two rings with barriers of their own, both eight K blocks deep. A token ring of four blocks
// beside a weight ring of ten was slower (9.7 against 8.9 us at 32 tokens, K = N = 4096): the
// token boxes arrive about 1500 cycles after they are requested, behind the weight boxes, so
// they need the same lead.
constexpr int kUdWStages = 8;
constexpr int kUdAStages = 8;
constexpr int kUdTokRows = 32;  // rows of the token box
constexpr int kUdABytes = kUdTokRows * kUdKB * 2;  // 4 KB
constexpr int kUdWBytes = kUdKB * kUdCols * 2;     // 8 KB: one box of 64 K rows x 64 columns
constexpr int kUdRecvBytes = kUdTokRows * kUdCols * 4;  // 8 KB
constexpr int kUdThreads = 128;
// [A stages][W stages][recv][barriers]; the MMA reads 16 KB from each A stage's start, which
// stays inside the buffer because the W stages follow.
constexpr int kUdOffW = kUdAStages * kUdABytes;
constexpr int kUdOffRecv = kUdOffW + kUdWStages * kUdWBytes;
constexpr int kUdOffBars = kUdOffRecv + kUdRecvBytes;
constexpr int kUdNumBars = 2 * kUdWStages + 2 * kUdAStages + 1;
constexpr int kUdSmemBytes = kUdOffBars + kUdNumBars * 8 + 16 + 1024;  // + alignment slack
static_assert(kUdABytes % 1024 == 0 && kUdWBytes % 1024 == 0, "operand tiles start on swizzle-atom boundaries");
static_assert(kUdOffW + kUdWStages * kUdWBytes >= (kUdAStages - 1) * kUdABytes + 128 * kUdKB * 2, "the 128-row A read of the last stage stays inside the buffer");
static_assert(2 * (kUdSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM");

struct UdParams {
    void* out;
    int M, N, K, out_f32;
    DeviceStatus* status;
};

// Shared-memory descriptor of an MN-major SWIZZLE_128B operand: 64-element groups along N
// `lbo` bytes apart, 8-row groups along K `sbo` bytes apart.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void st_cluster_f32x4(uint32_t cluster_addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

__global__ void __launch_bounds__(kUdThreads, 2)
    f16_decode_umma_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                           const UdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;  // the swizzle is a function of the address
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    const uint32_t wfull0 = base + kUdOffBars, wempty0 = wfull0 + 8 * kUdWStages;
    const uint32_t afull0 = wempty0 + 8 * kUdWStages, aempty0 = afull0 + 8 * kUdAStages, tfull = aempty0 + 8 * kUdAStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kUdOffBars + kUdNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(), nranks = cluster_size();
    const int n0 = (int)(blockIdx.x / nranks) * kUdCols;
    // K blocks of 64 rows; the host makes their number a multiple of the cluster size. The last
    // block of the matrix may reach beyond K: TMA zero-fills those rows of both operands.
    const int slab_kb = (p.K + kUdKB - 1) / kUdKB / (int)nranks;
    const int kb0 = (int)rank * slab_kb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kUdWStages; ++s) {
            mbar_init(wfull0 + 8 * s, 1);
            mbar_init(wempty0 + 8 * s, 1);
        }
        for (int s = 0; s < kUdAStages; ++s) {
            mbar_init(afull0 + 8 * s, 1);
            mbar_init(aempty0 + 8 * s, 1);
        }
        mbar_init(tfull, 1);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kUdCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // First phase of the cluster barrier: "this CTA runs" (nobody waits for it before the tail).
    if (nranks > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (elect_one()) {
            auto load_w = [&](int kb, int s) {
                mbar_expect_tx(wfull0 + 8 * s, kUdWBytes);
                tma_load_2d(base + kUdOffW + s * kUdWBytes, &tmap_w, wfull0 + 8 * s, n0, (kb0 + kb) * kUdKB);
            };
            auto load_x = [&](int kb, int s) {
                mbar_expect_tx(afull0 + 8 * s, kUdABytes);
                tma_load_2d(base + s * kUdABytes, &tmap_x, afull0 + 8 * s, (kb0 + kb) * kUdKB, 0);
            };
            // The weights do not depend on the kernel before this one; the tokens do.
            const int first_w = slab_kb < kUdWStages ? slab_kb : kUdWStages;
            const int first_a = slab_kb < kUdAStages ? slab_kb : kUdAStages;
            for (int kb = 0; kb < first_w; ++kb) load_w(kb, kb);
            pdl_wait();
            for (int kb = 0; kb < first_a; ++kb) load_x(kb, kb);
            // Once the MMAs of K block j have completed, token stage j % A and weight stage j % W
            // are free for the blocks one ring further on.
            uint32_t sa = 0, pa = 0, sw = 0, pw = 0;
            for (int j = 0; j + kUdAStages < slab_kb; ++j) {
                if (!mbar_wait(aempty0 + 8 * sa, pa, abort_flag)) {
                    report_timeout(p.status, abort_flag, 0x50u, (unsigned)j);
                    break;
                }
                load_x(j + kUdAStages, (int)sa);
                if (++sa == kUdAStages) { sa = 0; pa ^= 1u; }
                if (j + kUdWStages < slab_kb) {
                    if (!mbar_wait(wempty0 + 8 * sw, pw, abort_flag)) {
                        report_timeout(p.status, abort_flag, 0x53u, (unsigned)j);
                        break;
                    }
                    load_w(j + kUdWStages, (int)sw);
                    if (++sw == kUdWStages) { sw = 0; pw ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc(128, kUdCols, 0u, 0u) | (1u << 16);  // B is MN-major
            uint32_t sa = 0, pa = 0, sw = 0, pw = 0;
            bool ok = true;
            for (int kb = 0; kb < slab_kb; ++kb) {
                if (!mbar_wait(wfull0 + 8 * sw, pw, abort_flag) || !mbar_wait(afull0 + 8 * sa, pa, abort_flag)) {
                    report_timeout(p.status, abort_flag, 0x51u, (unsigned)kb);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint64_t a_desc = make_kmajor_sw128_desc(base + sa * kUdABytes);
                const uint32_t w_addr = base + kUdOffW + sw * kUdWBytes;
#pragma unroll
                for (int kk = 0; kk < kUdKB / 16; ++kk)
                    umma_f16(tmem_base, a_desc + (uint64_t)(kk * 2),
                             make_mnmajor_sw128_desc(w_addr + kk * 2048, kUdWBytes, 1024u), idesc, (uint32_t)((kb | kk) != 0));
                // both stages are free once these MMAs have read them
                tc_commit(aempty0 + 8 * sa);
                tc_commit(wempty0 + 8 * sw);
                if (++sa == kUdAStages) { sa = 0; pa ^= 1u; }
                if (++sw == kUdWStages) { sw = 0; pw ^= 1u; }
            }
            if (ok) tc_commit(tfull);
        }
        __syncwarp();
    }

    // ------------------------------ epilogue ----------------------------------
    // Every CTA of the cluster runs by now: its shared memory may be written.
    if (nranks > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const int cpo = kUdCols / (int)nranks;  // columns per owner: 64, 32, 16 or 8
    const uint32_t recv = base + kUdOffRecv;  // [source rank][32 tokens][cpo] f32, written by the cluster
    if (warp == 0) {
        bool have = mbar_wait(tfull, 0u, abort_flag);
        if (!have) report_timeout(p.status, abort_flag, 0x52u, 0u);
        tc_fence_after();
        // Lane t of warp 0 holds token t: 32 columns per load. A dead accumulator is replaced by
        // zeros so that the peers' sums stay finite; the status word carries the error.
        uint32_t r[kUdCols / 32][32];
#pragma unroll
        for (int h = 0; h < kUdCols / 32; ++h) {
            if (have) {
                tmem_ld_32x32(tmem_base + (uint32_t)(32 * h), r[h]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[h][i] = 0u;
            }
        }
        if (have) tc_wait_ld();
#pragma unroll
        for (int h = 0; h < kUdCols / 32; ++h)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const int c = 32 * h + i, owner = c / cpo;
                const uint32_t dst = recv + (uint32_t)((((int)rank * kUdTokRows + lane) * cpo + (c - owner * cpo)) * 4);
                st_cluster_f32x4(mapa_shared(dst, (uint32_t)owner), __uint_as_float(r[h][i]), __uint_as_float(r[h][i + 1]),
                                 __uint_as_float(r[h][i + 2]), __uint_as_float(r[h][i + 3]));
            }
        tc_fence_before();
    }
    // Second phase: every part has been stored (release) and is visible here (acquire). After it
    // nobody touches another CTA's shared memory.
    if (nranks > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
        __syncthreads();
    }
    {
        const float* part = reinterpret_cast<const float*>(base_ptr + kUdOffRecv);
        const int quads = cpo / 4;  // float4 per token row of this CTA's share
        for (int f = threadIdx.x; f < kUdTokRows * quads; f += kUdThreads) {
            const int tok = f / quads, q = f - tok * quads;
            float4 v = *reinterpret_cast<const float4*>(part + (tok * cpo + 4 * q));
            for (int r = 1; r < (int)nranks; ++r) {
                const float4 u = *reinterpret_cast<const float4*>(part + ((r * kUdTokRows + tok) * cpo + 4 * q));
                v.x += u.x;
                v.y += u.y;
                v.z += u.z;
                v.w += u.w;
            }
            const int col = n0 + (int)rank * cpo + 4 * q;  // N % 8 == 0: the four columns are inside or outside together
            if (tok < p.M && col < p.N) {
                if (p.out_f32) {
                    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)tok * p.N + col) = v;
                } else {
                    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(static_cast<__half*>(p.out) + (size_t)tok * p.N + col) = pk;
                }
            }
        }
    }
    // ------------------------------ teardown -------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kUdCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn ud_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// Row-major f16 matrix [rows, cols] with a row pitch of `ld` elements; box = 64 columns x box_rows rows.
// A launch of a few microseconds cannot afford two driver calls for maps it built a moment ago
// (decode loops present the same weight matrices and activation buffers again and again), so
// each host thread keeps the maps of its last 64 distinct operands.
struct UdMapKey {
    const void* base;
    int rows, cols, ld, box_rows;
    bool operator==(const UdMapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
constexpr int kUdMapCache = 64;
struct UdMapCache {
    UdMapKey key[kUdMapCache];
    CUtensorMap map[kUdMapCache];
    int used = 0, next = 0;
};

int ud_make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    static thread_local UdMapCache cache;
    const UdMapKey key = {base, rows, cols, ld, box_rows};
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == key) {
            *map = cache.map[i];
            return 0;
        }
    EncodeTiledFn enc = ud_encode_fn();
    if (!enc) return fail(Y_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(Y_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
    const int slot = cache.used < kUdMapCache ? cache.used++ : (cache.next = (cache.next + 1) % kUdMapCache);
    cache.key[slot] = key;
    cache.map[slot] = *map;
    return 0;
}

}  // namespace

// Cluster size for the tcgen05 decode kernel: the largest of 8, 4, 2, 1 that divides the number of K blocks and
// keeps the grid within two CTAs per SM.
int umma_decode_slabs(int n, int k, int sms = 0) {
    const int blocks = (n + kUdCols - 1) / kUdCols, kbs = (k + kUdKB - 1) / kUdKB;
    const int cap = 2 * (sms > 0 ? sms : sm_count());
    for (int s = 8; s > 1; s >>= 1)
        if (kbs % s == 0 && blocks * s <= cap) return s;
    return 1;
}

bool umma_decode_applies(int m, int n, int k) { return m > 16 && m <= 32 && k >= 16 && k % 16 == 0 && n % 8 == 0; }

// `sms` > 0: for a GPU with that many multiprocessors (no device needed); 0: the current device.
void umma_decode_launch_geometry(int n, int k, int sms, unsigned* grid, unsigned* block, unsigned* smem, int* stages,
                                 unsigned* cluster) {
    *cluster = (unsigned)umma_decode_slabs(n, k, sms);
    *grid = (unsigned)((n + kUdCols - 1) / kUdCols) * *cluster;
    *block = kUdThreads;
    *smem = kUdSmemBytes;
    *stages = kUdWStages;
}

// x [M, K] f16 with row pitch ldx, w [K, N] f16 row-major, out [M, N] f32 or f16.
int launch_umma_decode(const void* x, int ldx, const void* w, void* out, bool out_f32, int m, int n, int k, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    YB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        YB_CUDA(cudaFuncSetAttribute(f16_decode_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kUdSmemBytes));
        configured[dev] = true;
    }
    CUtensorMap tx, tw;
    if (int rc = ud_make_map(&tx, x, m, k, ldx, kUdTokRows)) return rc;
    if (int rc = ud_make_map(&tw, w, k, n, n, kUdKB)) return rc;  // box: 64 columns x 64 K rows
    UdParams p;
    p.out = out;
    p.M = m;
    p.N = n;
    p.K = k;
    p.out_f32 = out_f32 ? 1 : 0;
    p.status = device_status_ptr();
    const int slabs = umma_decode_slabs(n, k);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n + kUdCols - 1) / kUdCols) * (unsigned)slabs);
    cfg.blockDim = dim3(kUdThreads);
    cfg.dynamicSmemBytes = kUdSmemBytes;
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
    return check_cuda(cudaLaunchKernelEx(&cfg, f16_decode_umma_kernel, tx, tw, p), "f16_decode_umma_kernel launch");
}

}  // namespace yb
