// INT4 weight-only path: group quantise/pack, repack into the streaming layout,
// and the small-M decode GEMM.
//
// The decode GEMM is HBM-bound weight streaming (K*N/2 bytes of weights read
// exactly once), so it is built around keeping every SM's share of the stream
// in flight from the first cycle: the streaming layout makes each CTA's share
// one contiguous byte range, a producer warp issues it as 1-D bulk copies into
// a shared-memory ring (up to ~165 KB outstanding per SM), and 16 consumer warps
// (8 for 32-token launches) dequantise in registers and feed mma.sync.m16n8k16 (f16 x f16 -> f32)
// with the weights as the 16-row operand and the M <= 32 tokens as the 8-wide
// operand. The group scale multiplies each group's f32 partial sum, so the
// integer weights enter the MMA exactly. K is split across the warps of a
// CTA and reduced in shared memory in a fixed order: no atomics, results
// overwrite the output and are run-to-run identical.
#include "common.cuh"

namespace yb {
namespace {

// ---- quantise -----------------------------------------------------------------
// grid (N/2/128, K/128); thread = 2 adjacent columns of one 128-row group.
__global__ void __launch_bounds__(128)
    int4_quantize_kernel(const __half* __restrict__ w, size_t K, size_t N,
                         uint32_t* __restrict__ qweight, __half* __restrict__ scales) {
    const size_t n = 2 * ((size_t)blockIdx.x * 128 + threadIdx.x);
    if (n >= N) return;
    const size_t g = blockIdx.y;
    const __half* base = w + g * 128 * N + n;
    float a0 = 0.0f, a1 = 0.0f;
    for (int k = 0; k < 128; ++k) {
        float2 f = __half22float2(*reinterpret_cast<const __half2*>(base + (size_t)k * N));
        a0 = fmaxf(a0, fabsf(f.x));
        a1 = fmaxf(a1, fabsf(f.y));
    }
    const __half h0 = __float2half_rn(__fdiv_rn(a0, 7.0f));
    const __half h1 = __float2half_rn(__fdiv_rn(a1, 7.0f));
    *reinterpret_cast<__half2*>(scales + g * N + n) = __halves2half2(h0, h1);
    const float s0 = __half2float(h0), s1 = __half2float(h1);
    for (int kw = 0; kw < 16; ++kw) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float2 f = __half22float2(
                *reinterpret_cast<const __half2*>(base + (size_t)(kw * 8 + j) * N));
            int q0 = 0, q1 = 0;
            if (s0 > 0.0f) q0 = max(-8, min(7, __float2int_rn(__fdiv_rn(f.x, s0))));
            if (s1 > 0.0f) q1 = max(-8, min(7, __float2int_rn(__fdiv_rn(f.y, s1))));
            w0 |= ((uint32_t)q0 & 0xfu) << (4 * j);
            w1 |= ((uint32_t)q1 & 0xfu) << (4 * j);
        }
        *reinterpret_cast<uint2*>(qweight + (g * 16 + kw) * N + n) = make_uint2(w0, w1);
    }
}

// ---- repack ----------------------------------------------------------------------
// Streaming layout: one 1056-byte block per (16-column tile, 128-row group),
// tiles outermost. Bytes [0,1024): half h, lane, 16-byte unit of four words;
// with gq = lane/4, c = lane%4, word i holds the eight K-consecutive weights
// k = 128g + 32(2h + i/2) + 8c + (0..7) of column 16*tile + gq + 8(i%2),
// offset-binary (q+8), logical element j at nibble {0,4,1,5,2,6,3,7}[j].
// Bytes [1024,1056): the tile's 16 f16 group scales.
constexpr int kBlkBytes = 1056;
constexpr int kBlkWords = kBlkBytes / 4;  // 264

__global__ void __launch_bounds__(256)
    int4_repack_kernel(const uint32_t* __restrict__ qweight, const uint16_t* __restrict__ scales,
                       size_t ngroups, size_t N, size_t total_words,
                       uint32_t* __restrict__ stream) {
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < total_words;
         idx += (size_t)gridDim.x * 256) {
        const size_t blk = idx / kBlkWords;
        const int wi = (int)(idx % kBlkWords);
        const size_t t = blk / ngroups, g = blk % ngroups;
        uint32_t outw;
        if (wi < 256) {
            const int h = wi / 128, lane = (wi % 128) / 4, i = wi % 4;
            const int gq = lane / 4, c = lane % 4;
            const size_t kw = g * 16 + (size_t)(4 * (2 * h + i / 2) + c);
            const size_t col = t * 16 + (size_t)(gq + 8 * (i % 2));
            const uint32_t src = qweight[kw * N + col] ^ 0x88888888u;
            // nibble positions 0,4,1,5,2,6,3,7 for logical elements 0..7
            outw = (src & 0xfu) | ((src >> 4) & 0xfu) << 16 | ((src >> 8) & 0xfu) << 4 |
                   ((src >> 12) & 0xfu) << 20 | ((src >> 16) & 0xfu) << 8 |
                   ((src >> 20) & 0xfu) << 24 | ((src >> 24) & 0xfu) << 12 |
                   ((src >> 28) & 0xfu) << 28;
        } else {
            const int sp = wi - 256;  // scale pair 0..7
            const uint16_t* s = scales + g * N + t * 16 + 2 * sp;
            outw = (uint32_t)s[0] | ((uint32_t)s[1] << 16);
        }
        stream[idx] = outw;
    }
}

// ---- decode GEMM ------------------------------------------------------------------


// NT = 8-token operand tiles (M <= 8 * NT). round_tiles = 16-column weight tiles
// whose accumulators a warp keeps in registers at once.
template <int NT>
struct DecodeCfg {
    // Consumer warps = K groups per ring slot (one group per warp). 32-token launches keep
    // 4x the accumulators and activation fragments per thread, so they run 8 warps (more
    // registers per thread) instead of 16.
    static constexpr int warps = NT == 4 ? 8 : 16;
    static constexpr int threads = (warps + 1) * 32;
    static constexpr int unit_bytes = warps * kBlkBytes;
    static constexpr int round_tiles = 5;
    static constexpr int slots = NT == 1 ? 10 : (NT == 2 ? 8 : 16);
    static constexpr int red_floats = warps * round_tiles * NT * 128;
    static constexpr int ring_bytes = slots * unit_bytes;
    static constexpr int smem_bytes = ring_bytes + red_floats * 4 + 2 * slots * 8 + 16;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Dequantisation costs one logic instruction per f16 pair. With u = q + 8 the
// stored offset-binary nibble:
//   (w & 0x000F000F) | 0x6400  is the f16 pair 1024 + u = q + 1032   (ulp 1 at 1024)
//   (w & 0x00F000F0) | 0x5400  is the f16 pair   64 + u = q +   72   (ulp 1/16 at 64)
// The offsets are not subtracted per weight. They are the same for every weight
// column, so their contribution to a group's partial sum,
// 1032 * sum(x over the "lo" K slots) + 72 * sum(x over the "hi" K slots), is
// computed once per (group, token) by one MMA pass with a constant operand and
// the group's accumulator starts at its negative. All products are exact in f32.
__device__ __forceinline__ uint32_t deq_lo(uint32_t w) { return (w & 0x000f000fu) | 0x64006400u; }
__device__ __forceinline__ uint32_t deq_hi(uint32_t w) { return (w & 0x00f000f0u) | 0x54005400u; }
constexpr uint32_t kOffsetLo = 0x64086408u;  // f16 pair (1032, 1032)
constexpr uint32_t kOffsetHi = 0x54805480u;  // f16 pair (72, 72)

template <int THREADS>
__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

template <int NT>
__global__ void __launch_bounds__(DecodeCfg<NT>::threads, 1)
    int4_decode_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ wstream,
                       __half* __restrict__ out, int M, int N, int K, DeviceStatus* status) {
    using Cfg = DecodeCfg<NT>;
    constexpr int kRoundTiles = Cfg::round_tiles;
    constexpr int kConsumerWarps = Cfg::warps, kUnitGroups = Cfg::warps, kUnitBytes = Cfg::unit_bytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + Cfg::ring_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::ring_bytes + Cfg::red_floats * 4);
    volatile uint32_t* abort_flag =
        reinterpret_cast<volatile uint32_t*>(smem + Cfg::ring_bytes + Cfg::red_floats * 4 +
                                             2 * Cfg::slots * 8);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + Cfg::slots);
    const uint32_t ring0 = smem_u32(ring);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::slots; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Programmatic dependent launch: the next kernel in the stream may start its own
    // prologue and weight copies while this one is still running (the weights are not
    // written by anything in the stream), which hides the launch gap between decode
    // GEMMs of consecutive layers. Whatever can depend on earlier kernels (the
    // activations, the output buffer) is only touched after griddepcontrol.wait below.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int ngroups = K / 128;
    const int phases = (ngroups + kUnitGroups - 1) / kUnitGroups;
    const int T = N / 16;
    const int t_begin = (int)(((long long)blockIdx.x * T) / gridDim.x);
    const int t_end = (int)(((long long)(blockIdx.x + 1) * T) / gridDim.x);

    if (warp == kConsumerWarps) {
        // ---- producer: stream this CTA's contiguous share through the ring ----
        if (lane == 0) {
            uint32_t slot = 0, sphase = 0;
            bool ok = true;
            for (int r0 = t_begin; r0 < t_end && ok; r0 += kRoundTiles) {
                const int rt = min(kRoundTiles, t_end - r0);
                for (int p = 0; p < phases && ok; ++p) {
                    const int ng = min(kUnitGroups, ngroups - p * kUnitGroups);
                    for (int t = 0; t < rt; ++t) {
                        if (!mbar_wait(empty0 + 8 * slot, sphase ^ 1u, abort_flag)) {
                            report_timeout(status, abort_flag, 0x100u, (unsigned)(r0 + t));
                            ok = false;
                            break;
                        }
                        const uint32_t bytes = (uint32_t)ng * kBlkBytes;
                        mbar_expect_tx(full0 + 8 * slot, bytes);
                        bulk_load_1d(ring0 + slot * kUnitBytes,
                                     wstream + ((size_t)(r0 + t) * ngroups + (size_t)p * kUnitGroups) *
                                                   kBlkBytes,
                                     bytes, full0 + 8 * slot);
                        if (++slot == Cfg::slots) { slot = 0; sphase ^= 1u; }
                    }
                }
            }
        }
    } else {
        // ---- consumers -------------------------------------------------------
        asm volatile("griddepcontrol.wait;" ::: "memory");  // earlier kernels' writes to x / out are complete
        const int gq = lane >> 2, c = lane & 3;
        uint32_t slot = 0, sphase = 0;  // ring position of the next unit
        bool dead = false;
        for (int r0 = t_begin; r0 < t_end; r0 += kRoundTiles) {
            const int rt = min(kRoundTiles, t_end - r0);
            float acc[kRoundTiles][NT][4];
#pragma unroll
            for (int t = 0; t < kRoundTiles; ++t)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[t][j][i] = 0.0f;

            for (int p = 0; p < phases; ++p) {
                const int g = p * kUnitGroups + warp;
                const bool valid = g < ngroups;
                // Activation fragments of this warp's group: token gq + 8j,
                // k = 128g + 32pp + 8c + (0..7).
                uint4 xf[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int tok = gq + 8 * j;
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) {
                        xf[j][pp] = make_uint4(0, 0, 0, 0);
                        if (valid && tok < M)
                            xf[j][pp] = __ldg(reinterpret_cast<const uint4*>(
                                x + (size_t)tok * K + (size_t)g * 128 + pp * 32 + c * 8));
                    }
                }
                // Offset contribution of this group (see deq_lo / deq_hi): identical for
                // all 16 weight columns, so one MMA pass with a constant operand.
                float neg_off[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) {
                        mma_16816(o, kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[j][pp].x, xf[j][pp].y);
                        mma_16816(o, kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[j][pp].z, xf[j][pp].w);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) neg_off[j][i] = -o[i];
                }
#pragma unroll
                for (int t = 0; t < kRoundTiles; ++t) {
                    if (t < rt) {
                        if (!dead && !mbar_wait(full0 + 8 * slot, sphase, abort_flag)) {
                            report_timeout(status, abort_flag, 0x200u + warp, (unsigned)(r0 + t));
                            dead = true;
                        }
                        if (valid && !dead) {
                            const uint8_t* blk = ring + slot * kUnitBytes + warp * kBlkBytes;
                            const uint4 u0 = *reinterpret_cast<const uint4*>(blk + lane * 16);
                            const uint4 u1 = *reinterpret_cast<const uint4*>(blk + 512 + lane * 16);
                            const __half* sc = reinterpret_cast<const __half*>(blk + 1024);
                            const float s_lo = __half2float(sc[gq]);
                            const float s_hi = __half2float(sc[gq + 8]);
                            const uint32_t wA[4] = {u0.x, u0.z, u1.x, u1.z};  // column gq
                            const uint32_t wB[4] = {u0.y, u0.w, u1.y, u1.w};  // column gq + 8
                            float tmp[NT][4];
#pragma unroll
                            for (int j = 0; j < NT; ++j)
#pragma unroll
                                for (int i = 0; i < 4; ++i) tmp[j][i] = neg_off[j][i];
#pragma unroll
                            for (int pp = 0; pp < 4; ++pp) {
                                const uint32_t hA = wA[pp] >> 8, hB = wB[pp] >> 8;
                                const uint32_t a0 = deq_lo(wA[pp]), a1 = deq_lo(wB[pp]);
                                const uint32_t a2 = deq_hi(wA[pp]), a3 = deq_hi(wB[pp]);
                                const uint32_t e0 = deq_lo(hA), e1 = deq_lo(hB);
                                const uint32_t e2 = deq_hi(hA), e3 = deq_hi(hB);
#pragma unroll
                                for (int j = 0; j < NT; ++j) {
                                    mma_16816(tmp[j], a0, a1, a2, a3, xf[j][pp].x, xf[j][pp].y);
                                    mma_16816(tmp[j], e0, e1, e2, e3, xf[j][pp].z, xf[j][pp].w);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < NT; ++j) {
                                acc[t][j][0] = fmaf(s_lo, tmp[j][0], acc[t][j][0]);
                                acc[t][j][1] = fmaf(s_lo, tmp[j][1], acc[t][j][1]);
                                acc[t][j][2] = fmaf(s_hi, tmp[j][2], acc[t][j][2]);
                                acc[t][j][3] = fmaf(s_hi, tmp[j][3], acc[t][j][3]);
                            }
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty0 + 8 * slot);
                        if (++slot == Cfg::slots) { slot = 0; sphase ^= 1u; }
                    }
                }
            }

            // ---- cross-warp reduction in warp order, then store --------------
            float* mine = red + (size_t)warp * (kRoundTiles * NT * 128);
#pragma unroll
            for (int t = 0; t < kRoundTiles; ++t)
#pragma unroll
                for (int j = 0; j < NT; ++j)
                    *reinterpret_cast<float4*>(mine + (t * NT + j) * 128 + lane * 4) =
                        make_float4(acc[t][j][0], acc[t][j][1], acc[t][j][2], acc[t][j][3]);
            consumer_bar<kConsumerWarps * 32>();
            const int nout = rt * NT * 128;
            for (int e = threadIdx.x; e < nout; e += kConsumerWarps * 32) {
                float v = red[e];
#pragma unroll
                for (int w = 1; w < kConsumerWarps; ++w) v += red[w * (kRoundTiles * NT * 128) + e];
                const int t = e / (NT * 128), j = (e / 128) % NT, l = (e % 128) / 4, i = e % 4;
                const int col = (r0 + t) * 16 + (l >> 2) + 8 * (i >> 1);
                const int tok = 8 * j + 2 * (l & 3) + (i & 1);
                if (tok < M) out[(size_t)tok * N + col] = __float2half_rn(v);
            }
            consumer_bar<kConsumerWarps * 32>();
        }
    }
}

template <int NT>
int launch_decode(const void* x, const void* wstream, void* out, int m, int n, int k,
                  cudaStream_t st) {
    using Cfg = DecodeCfg<NT>;
    static bool configured[64] = {};
    int dev = 0;
    YB_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        YB_CUDA(cudaFuncSetAttribute(int4_decode_kernel<NT>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::smem_bytes));
        configured[dev] = true;
    }
    const int tiles = n / 16;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)Cfg::threads);
    cfg.dynamicSmemBytes = Cfg::smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, int4_decode_kernel<NT>, static_cast<const __half*>(x),
                                         static_cast<const uint8_t*>(wstream), static_cast<__half*>(out), m, n, k,
                                         device_status_ptr()),
                      "int4_decode_kernel launch");
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Launch geometry of the decode kernel for the host launch API.
void decode_launch_geometry(int m, int n, unsigned* grid, unsigned* block, unsigned* smem, int* slots,
                            int* unit_k) {
    const int tiles = n > 0 ? n / 16 : 0;
    *grid = (unsigned)(tiles < sm_count() ? tiles : sm_count());
    if (m <= 8) { *block = DecodeCfg<1>::threads; *smem = DecodeCfg<1>::smem_bytes; *slots = DecodeCfg<1>::slots; *unit_k = DecodeCfg<1>::warps * 128; }
    else if (m <= 16) { *block = DecodeCfg<2>::threads; *smem = DecodeCfg<2>::smem_bytes; *slots = DecodeCfg<2>::slots; *unit_k = DecodeCfg<2>::warps * 128; }
    else { *block = DecodeCfg<4>::threads; *smem = DecodeCfg<4>::smem_bytes; *slots = DecodeCfg<4>::slots; *unit_k = DecodeCfg<4>::warps * 128; }
}

}  // namespace yb

using namespace yb;

extern "C" int y_b200_int4_quantize(const void* w_f16, size_t k, size_t n, uint32_t* qweight,
                                    void* scales_f16, void* stream) {
    if (!w_f16 || !qweight || !scales_f16) return fail(Y_B200_ERR_INVALID, "y_b200_int4_quantize: null pointer");
    if (k == 0 || k % 128 != 0 || n == 0 || n % 16 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_int4_quantize: need K %% 128 == 0 and N %% 16 == 0 (K=%zu N=%zu)", k, n);
    if (!aligned16(w_f16) || !aligned16(qweight) || !aligned16(scales_f16))
        return fail(Y_B200_ERR_ALIGN, "y_b200_int4_quantize: pointers must be 16-byte aligned");
    dim3 grid((unsigned)((n / 2 + 127) / 128), (unsigned)(k / 128));
    int4_quantize_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(w_f16), k, n, qweight, static_cast<__half*>(scales_f16));
    return check_cuda(cudaGetLastError(), "int4_quantize_kernel launch");
}

extern "C" size_t y_b200_int4_stream_bytes(size_t k, size_t n) {
    return (n / 16) * (k / 128) * (size_t)kBlkBytes;
}

extern "C" int y_b200_int4_repack(const uint32_t* qweight, const void* scales_f16, size_t k,
                                  size_t n, void* wstream, void* stream) {
    if (!qweight || !scales_f16 || !wstream) return fail(Y_B200_ERR_INVALID, "y_b200_int4_repack: null pointer");
    if (k == 0 || k % 128 != 0 || n == 0 || n % 16 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_int4_repack: need K %% 128 == 0 and N %% 16 == 0 (K=%zu N=%zu)", k, n);
    if (!aligned16(wstream)) return fail(Y_B200_ERR_ALIGN, "y_b200_int4_repack: wstream must be 16-byte aligned");
    const size_t words = y_b200_int4_stream_bytes(k, n) / 4;
    size_t blocks = (words + 255) / 256;
    const size_t cap = (size_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    int4_repack_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        qweight, static_cast<const uint16_t*>(scales_f16), k / 128, n, words,
        static_cast<uint32_t*>(wstream));
    return check_cuda(cudaGetLastError(), "int4_repack_kernel launch");
}

extern "C" int y_b200_gemm_int4_decode(const void* x_f16, const void* wstream, void* out_f16, int m,
                                       int n, int k, void* stream) {
    if (!x_f16 || !wstream || !out_f16) return fail(Y_B200_ERR_INVALID, "y_b200_gemm_int4_decode: null pointer");
    if (m < 1 || m > 32) return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_int4_decode: M=%d outside 1..32", m);
    if (k <= 0 || k % 128 != 0 || n <= 0 || n % 16 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_gemm_int4_decode: need K %% 128 == 0 and N %% 16 == 0 (K=%d N=%d)", k, n);
    if (!aligned16(x_f16) || !aligned16(wstream))
        return fail(Y_B200_ERR_ALIGN, "y_b200_gemm_int4_decode: x and wstream must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m <= 8) return launch_decode<1>(x_f16, wstream, out_f16, m, n, k, st);
    if (m <= 16) return launch_decode<2>(x_f16, wstream, out_f16, m, n, k, st);
    return launch_decode<4>(x_f16, wstream, out_f16, m, n, k, st);
}
