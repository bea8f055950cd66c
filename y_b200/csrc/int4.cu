// INT4 weight-only path: group quantise/pack, repack into the streaming layout,
// and the small-M decode GEMM.
//
// The decode GEMM is weight streaming (K*N/2 bytes of weights read exactly once),
// so it is built around having every SM's share of the stream requested from its
// first microsecond: the streaming layout makes each CTA's share one contiguous
// byte range cut into 1056-byte blocks (one 16-column tile x one 128-row group),
// each warp copies its own blocks into its own part of shared memory with
// per-thread 16-byte asynchronous copies, many blocks ahead, and dequantises in
// registers. Up to two tokens go through the FMA pipe; more go through
// mma.sync.m16n8k16 (f16 x f16 -> f32) with the weights as the 16-row operand
// and up to 32 tokens as 8-wide operands. The group scale multiplies each group's
// f32 partial sum, so the integer weights enter the arithmetic exactly. K is split
// across the warps of a CTA and reduced in shared memory in a fixed order: no
// atomics, results overwrite the output and are run-to-run identical. Nothing in
// the kernel waits on a barrier that another agent has to complete.
#include <type_traits>
#include <utility>

#include "common.cuh"

#include <algorithm>

namespace yb {
namespace {

// ---- quantise -----------------------------------------------------------------
// grid (ceil(N / 128), K / 128), 256 threads: one CTA quantises one 128-row group of 128
// columns. Thread (cv = tid % 16, rg = tid / 16) owns rows 8 rg .. 8 rg + 7 of the column
// vector cv (8 adjacent columns): eight 16-byte loads, 256 contiguous bytes per row across
// a half warp. The weights are read once and stay in registers between the column amax
// (partial maxima per row block through shared memory) and the packing: a packed word holds
// eight K-consecutive weights of one column, exactly the thread's eight rows, so every
// thread writes 32 contiguous bytes of qweight and a half warp 512. Measured at 4096 x 11008:
// rows held in registers, three CTAs per SM 43 us, four (64 registers) 39 us; four rows per
// thread in CTAs of 512 (halves of a word swapped by shuffle) 43 us; the tile staged in shared
// memory by cp.async (below: five CTAs per SM) 37.5 us with about 15 instructions per weight
// (conversion, amax, code with two range tests, clamp, bit-field packing: 19 us of issue time
// per SM); the code path described next needs about 9.
//
// The code of a weight is clamp(rint(v / s), -8, 7) with an IEEE division and ties to even. The
// division is not paid per element: v and s are f16 values, so the exact quotient is a ratio of
// two integers below 2048 times a power of two, and such a ratio is either exactly a half-integer
// or at least 1 / 4094 away from every half-integer. t = v * (1 / s) + 8 carries an error below
// 1e-6 for |v / s| < 7.4, so rint(t) - 8 is the code unless t sits within 1e-4 of a half-integer
// (then the quotient may BE that half-integer and the division settles the tie). The common path
// stays on the floating-point pipe and has no conversion, clamp or bit-field instruction:
//   y = t + 1.5 * 2^23 (y - 1.5 * 2^23 = rint(t), ties to even), d = t - rint(t),
//   word halves as floats, acc = acc * 16 + rint(t) over four rows (below 2^16: exact),
// and a word's eight rows are checked together afterwards: max |d| <= 0.4999 and no NaN in the
// accumulators. A column whose |amax / s| is not below 7.4 (a scale that rounded to a subnormal,
// an infinite weight) gets NaN for 1 / s, which sends its words down the same exact path; so
// every input gives the same code as the division. Stored nibbles are two's complement: the
// offset-binary digits rint(t) = q + 8 are flipped by one XOR per word.
// 16-byte asynchronous copy that writes zeros and reads nothing when `valid` is false.
__device__ __forceinline__ void cp_async_16_zfill_q(uint32_t dst_smem, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(bytes) : "memory");
}
// The definition, for the words the common path hands back.
__device__ __forceinline__ int int4_code_exact(float v, float s) {
    const int q = s > 0.0f ? __float2int_rn(__fdiv_rn(v, s)) : 0;
    return max(-8, min(7, q));
}

__global__ void __launch_bounds__(256, 5)
    int4_quantize_kernel(const __half* __restrict__ w, size_t K, size_t N,
                         uint32_t* __restrict__ qweight, __half* __restrict__ scales) {
    // The CTA's 128 x 128 tile waits in shared memory, not in registers: a thread copies its
    // eight 16-byte units there asynchronously and reads them back twice (amax, packing), so
    // five CTAs fit an SM and 160 KB per SM are in flight.
    __shared__ __align__(16) uint8_t tile[128][256];
    __shared__ float part[16][128];
    __shared__ __align__(16) float col_scale[128];
    __shared__ __align__(16) float col_rcp[128];
    const int cv = threadIdx.x & 15, rg = threadIdx.x >> 4;
    const size_t g = blockIdx.y;
    const size_t col = (size_t)blockIdx.x * 128 + (size_t)cv * 8;
    const bool live = col < N;  // N % 8 == 0: a column vector is wholly inside or outside
    {
        const __half* base = w + (g * 128 + (size_t)rg * 8) * N + (live ? col : 0);
        const uint32_t dst = smem_u32(&tile[rg * 8][cv * 16]);
#pragma unroll
        for (int r = 0; r < 8; ++r) cp_async_16_zfill_q(dst + r * 256, base + (size_t)r * N, live);
        asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    }
    const uint8_t* mine = &tile[rg * 8][cv * 16];  // this thread's own copies
    // Column maxima of |v| on f16 pairs (a NaN never wins a maximum, as with fmaxf).
    {
        __half2 m2[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) m2[j] = __float2half2_rn(0.0f);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const uint4 row = *reinterpret_cast<const uint4*>(mine + r * 256);
            const __half2* h = reinterpret_cast<const __half2*>(&row);
#pragma unroll
            for (int j = 0; j < 4; ++j) m2[j] = __hmax2(m2[j], __habs2(h[j]));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(m2[j]);
            part[rg][cv * 8 + 2 * j] = f.x;
            part[rg][cv * 8 + 2 * j + 1] = f.y;
        }
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        float a = part[0][threadIdx.x];
#pragma unroll
        for (int r = 1; r < 16; ++r) a = fmaxf(a, part[r][threadIdx.x]);
        const __half h = __float2half_rn(__fdiv_rn(a, 7.0f));
        const float sc = __half2float(h);
        const float rcp = sc > 0.0f ? __frcp_rn(sc) : 0.0f;
        col_scale[threadIdx.x] = sc;
        // NaN for a column the common path must not touch (see above)
        col_rcp[threadIdx.x] = __fmul_rn(a, rcp) < 7.4f ? rcp : __int_as_float(0x7fc00000);
        const size_t c = (size_t)blockIdx.x * 128 + threadIdx.x;
        if (c < N) scales[g * N + c] = h;
    }
    __syncthreads();
    if (!live) return;
    constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: t + kMagic has rint(t) in its low mantissa bits
    float rcp[8];
    {
        const float4 r0 = *reinterpret_cast<const float4*>(&col_rcp[cv * 8]);
        const float4 r1 = *reinterpret_cast<const float4*>(&col_rcp[cv * 8 + 4]);
        rcp[0] = r0.x; rcp[1] = r0.y; rcp[2] = r0.z; rcp[3] = r0.w;
        rcp[4] = r1.x; rcp[5] = r1.y; rcp[6] = r1.z; rcp[7] = r1.w;
    }
    float acc[8][2], dmax[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c][0] = acc[c][1] = dmax[c] = 0.0f;
#pragma unroll
    for (int r = 7; r >= 0; --r) {  // the highest nibble of each half word first
        const uint4 row = *reinterpret_cast<const uint4*>(mine + r * 256);
        const __half2* h = reinterpret_cast<const __half2*>(&row);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = 2 * j + e;
                const float tq = __fmaf_rn(e == 0 ? f.x : f.y, rcp[c], 8.0f);
                const float rt = __fsub_rn(__fadd_rn(tq, kMagic), kMagic);  // rint(tq)
                dmax[c] = fmaxf(dmax[c], fabsf(__fsub_rn(tq, rt)));
                acc[c][r >> 2] = __fmaf_rn(acc[c][r >> 2], 16.0f, rt);
            }
        }
    }
    uint32_t words[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        // 2^23 + n has the integer n < 2^16 in its low mantissa bits
        const uint32_t lo = __float_as_uint(__fadd_rn(acc[c][0], 8388608.0f));
        const uint32_t hi = __float_as_uint(__fadd_rn(acc[c][1], 8388608.0f));
        words[c] = __byte_perm(lo, hi, 0x5410) ^ 0x88888888u;
        const float chk = __fadd_rn(acc[c][0], acc[c][1]);
        if (!(dmax[c] <= 0.4999f) || !(chk == chk)) {  // a possible tie, a NaN, or a column off the common path
            const float sc = col_scale[cv * 8 + c];
            uint32_t wd = 0u;
#pragma unroll 1
            for (int r = 0; r < 8; ++r) {
                const float v = __half2float(*reinterpret_cast<const __half*>(mine + r * 256 + 2 * c));
                wd |= ((uint32_t)int4_code_exact(v, sc) & 0xfu) << (4 * r);
            }
            words[c] = wd;
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(qweight + (g * 16 + (size_t)rg) * N + col);
    dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
    dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
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
                       size_t ngroups, size_t N, size_t total_blocks,
                       uint32_t* __restrict__ stream) {
    // One warp per 1056-byte block. Its 256 source words are 16 packed rows of 16 adjacent
    // columns: a half warp reads one 64-byte row segment per load (eight loads per lane), the
    // words change places in shared memory (row pitch 17 words: both sides conflict-free) and
    // every lane writes its two 16-byte units of the block; lanes 0..7 copy the scale pairs. (One
    // output word per thread gathered its source with a stride of N words: 8x read
    // amplification, 27 us for 4096 x 11008 against 2 x 23 MB of traffic.)
    __shared__ uint32_t tile[8][16][17];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t(*t)[17] = tile[warp];
    const int rsel = lane >> 4, csel = lane & 15;
    const int gq = lane >> 2, c = lane & 3;
    for (size_t blk = (size_t)blockIdx.x * 8 + warp; blk < total_blocks; blk += (size_t)gridDim.x * 8) {
        const size_t tl = blk / ngroups, g = blk % ngroups;
        const uint32_t* src = qweight + (g * 16 + (size_t)rsel) * N + tl * 16 + csel;
#pragma unroll
        for (int r = 0; r < 8; ++r) t[2 * r + rsel][csel] = src[(size_t)(2 * r) * N];
        __syncwarp();
        uint32_t* dst = stream + blk * kBlkWords;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t v = t[4 * (2 * h + i / 2) + c][gq + 8 * (i % 2)] ^ 0x88888888u;
                // nibble positions 0,4,1,5,2,6,3,7 for logical elements 0..7
                o[i] = (v & 0xfu) | ((v >> 4) & 0xfu) << 16 | ((v >> 8) & 0xfu) << 4 | ((v >> 12) & 0xfu) << 20 |
                       ((v >> 16) & 0xfu) << 8 | ((v >> 20) & 0xfu) << 24 | ((v >> 24) & 0xfu) << 12 |
                       ((v >> 28) & 0xfu) << 28;
            }
            *reinterpret_cast<uint4*>(dst + h * 128 + lane * 4) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        if (lane < 8) {
            const uint16_t* sp = scales + g * N + tl * 16 + 2 * lane;
            dst[256 + lane] = (uint32_t)sp[0] | ((uint32_t)sp[1] << 16);
        }
        __syncwarp();  // the tile is reused by the warp's next block
    }
}

// ---- decode GEMM ------------------------------------------------------------------

// NT = 8-token operand tiles of the tensor path (M <= 8 * NT). round_tiles = 16-column
// weight tiles whose accumulators a warp keeps in registers at once. Every warp streams
// its own blocks: `depth` blocks (1056 bytes each) are in flight or waiting in the warp's
// private part of shared memory.
template <int NT>
struct DecodeCfg {
    // Warps = K groups worked on at once (one group per warp). 32-token launches keep 4x
    // the accumulators and activation fragments per thread, so they run 8 warps (more
    // registers per thread) instead of 16.
    static constexpr int warps = NT == 4 ? 8 : 16;
    static constexpr int threads = warps * 32;
    static constexpr int round_tiles = 5;
    // Ring depth, measured at K = 4096, N = 11008: 3 -> 4 slots takes 1.7 % off a launch at 1 to 8
    // tokens (5.98 -> 5.88 us at one token); deeper rings only delay the activations behind more
    // weight requests.
    static constexpr int depth = NT == 1 ? 4 : (NT == 2 ? 4 : 6);
    static constexpr int stage_bytes = warps * depth * kBlkBytes;
    static constexpr int red_floats = warps * round_tiles * NT * 128;
    static constexpr int smem_bytes = stage_bytes + red_floats * 4;
    static constexpr int unit_k = warps * 128;  // K covered by the warps of a CTA in one phase
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = a * b + c with c and d in different registers: the first MMA of a chain reads its start
// value where it lies (no copy into the accumulator first).
__device__ __forceinline__ void mma_16816_from(float (&d)[4], const float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
// d = a * b.
__device__ __forceinline__ void mma_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    mma_16816_from(d, zero, a0, a1, a2, a3, b0, b1);
}

// Dequantisation costs one logic instruction per f16 pair. With u = q + 8 the
// stored offset-binary nibble:
//   (w & 0x000F000F) | 0x6400  is the f16 pair 1024 + u = q + 1032   (ulp 1 at 1024)
//   (w & 0x00F000F0) | 0x5400  is the f16 pair   64 + u = q +   72   (ulp 1/16 at 64)
// The offsets are not subtracted per weight. They are the same for every weight
// column, so their contribution to a group's partial sum,
// 1032 * sum(x over the "lo" K slots) + 72 * sum(x over the "hi" K slots), is
// computed once per (group, token) and the group's accumulator starts at its
// negative. All products are exact in f32.
//
// (w & mask) | exponent is one LOP3 only if at most one of the two constants is an
// immediate. The compiler, knowing both, emitted two instructions per pair (the ncu
// opcode counts showed 66 LOP3 per block where 32 are needed), so the constants are
// read from constant memory into registers once per kernel and the LOP3 is written out.
__constant__ uint32_t kDeqConst[4] = {0x000f000fu, 0x64006400u, 0x00f000f0u, 0x54005400u};
struct DeqRegs {
    uint32_t mask_lo, exp_lo, mask_hi, exp_hi;
};
__device__ __forceinline__ uint32_t and_or(uint32_t w, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(w), "r"(mask), "r"(orv));  // (w & mask) | orv
    return d;
}
constexpr uint32_t kOffsetLo = 0x64086408u;  // f16 pair (1032, 1032)
constexpr uint32_t kOffsetHi = 0x54805480u;  // f16 pair (72, 72)

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
// 16-byte copy that writes zeros and reads nothing when `valid` is false.
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst_smem, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// f(integral_constant<int, 0>), ..., f(integral_constant<int, N - 1>): a loop whose index
// is a compile-time constant inside the body.
template <typename F, int... I>
__device__ __forceinline__ void static_for_impl(F&& f, std::integer_sequence<int, I...>) {
    (f(std::integral_constant<int, I>()), ...);
}
template <int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
    static_for_impl(f, std::make_integer_sequence<int, N>());
}

// The blocks one warp works through, in order: rounds of up to round_tiles tiles; within a
// round the warp's K groups (phase p -> group p * warps + warp); within a phase the tiles.
// `src` runs along with the position so that a step is one add in the common case.
struct BlockSeq {
    const uint8_t* src;
    int r0, rt, p, t;
    __device__ __forceinline__ bool live(int t_end) const { return r0 < t_end; }
};

// Up to 8 * NT tokens per launch. A one- or two-token FMA-pipe variant (fma.rn.f32.f16 on
// dequantised pairs, no tensor instructions) was built and measured: 240 instructions per
// block against 130 here, 7.2 us against 7.0 us at K = 4096, N = 11008, so it was dropped.
//
// Weights reach shared memory by per-thread 16-byte asynchronous copies: lane l copies
// exactly the two 16-byte units it will read back (plus, in lanes 0 and 1, the block's
// scales), `depth` blocks ahead. A whole CTA's share of a 4096 x 11008 matrix (157 KB) is
// requested in its first microsecond. (A single thread issuing 1-D bulk copies kept only
// about 25 KB per SM in flight at DRAM latency, which held the kernel at 3.2 TB/s.)
// The first copies are issued before griddepcontrol.wait: the weights do not depend on
// the kernel before this one, the activations do.
template <int NT>
__global__ void __launch_bounds__(DecodeCfg<NT>::threads, 1)
    int4_decode_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ wstream,
                       __half* __restrict__ out, int M, int N, int K, int share_q, int share_r) {
    using Cfg = DecodeCfg<NT>;
    constexpr int kRoundTiles = Cfg::round_tiles, kWarps = Cfg::warps, kDepth = Cfg::depth;
    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem + Cfg::stage_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const DeqRegs dq = {kDeqConst[0], kDeqConst[1], kDeqConst[2], kDeqConst[3]};
    uint8_t* stage = smem + (size_t)warp * kDepth * kBlkBytes;
    const uint32_t stage0 = smem_u32(stage);
    pdl_launch_dependents();

    const int ngroups = K / 128;
    const int my_phases = warp < ngroups ? (ngroups - warp + kWarps - 1) / kWarps : 0;
    // CTA b owns share_q tiles, the first share_r CTAs one more (both computed by the host: a
    // division is a long dependent subroutine at the very start of a kernel whose first
    // requests should go out at once).
    const int bid = (int)blockIdx.x;
    const int t_begin = bid * share_q + min(bid, share_r);
    const int t_end = t_begin + share_q + (bid < share_r ? 1 : 0);

    const size_t tile_stride = (size_t)ngroups * kBlkBytes;  // same group, next tile
    const uint8_t* const wmine = wstream + (size_t)warp * kBlkBytes;  // this warp's group of phase 0, tile 0
    BlockSeq ahead = {wmine + (size_t)t_begin * tile_stride, t_begin, min(kRoundTiles, t_end - t_begin), 0, 0};
    const bool streaming = my_phases > 0;
    // Requests the next block of the sequence into slot `slot` and steps the sequence. Every
    // call commits one group, empty when the sequence has ended, so that "all but the newest
    // kDepth - 1 groups are complete" always means "the oldest outstanding block has arrived".
    auto request = [&](int slot) {
        if (streaming && ahead.live(t_end)) {
            const uint32_t dst = stage0 + slot * kBlkBytes;
            cp_async_16(dst + lane * 16, ahead.src + lane * 16);
            cp_async_16(dst + 512 + lane * 16, ahead.src + 512 + lane * 16);
            if (lane < 2) cp_async_16(dst + 1024 + lane * 16, ahead.src + 1024 + lane * 16);
            ahead.src += tile_stride;
            if (++ahead.t == ahead.rt) {  // once per phase: recompute instead of stepping
                ahead.t = 0;
                if (++ahead.p == my_phases) {
                    ahead.p = 0;
                    ahead.r0 += kRoundTiles;
                    ahead.rt = min(kRoundTiles, t_end - ahead.r0);
                }
                ahead.src = wmine + (size_t)ahead.r0 * tile_stride + (size_t)ahead.p * (kWarps * kBlkBytes);
            }
        }
        cp_async_commit();
    };
#pragma unroll 1
    for (int i = 0; i < kDepth; ++i) request(i);
    int slot = 0;
    // The block in `slot` has arrived and every lane of the warp can read it.
    auto acquire = [&]() -> const uint8_t* {
        cp_async_wait<kDepth - 1>();
        __syncwarp();
        return stage + slot * kBlkBytes;
    };
    // Every lane is done with the block in `slot`: reuse the slot for the block kDepth ahead.
    auto release = [&]() {
        __syncwarp();
        request(slot);
        if (++slot == kDepth) slot = 0;
    };

    pdl_wait();  // earlier kernels' writes to x / reads of out are complete
    const int gq = lane >> 2, c = lane & 3;
    // ---- weights are the 16-row MMA operand, tokens the 8-wide one.
    // The common decode shape (K = 4096 with 16 warps: two K groups per warp; a CTA share of
    // four or five tiles: one round) runs as straight-line code: block b of the warp is
    // (group b / RT, tile b % RT), so its ring slot, its source and whether a block kDepth
    // ahead exists are all known at compile time. The blocks requested before the wait
    // above are the first kDepth of the same order. Against the loop below this saves about
    // a quarter of the instructions per block. (Only for up to 8 tokens: with wider token
    // tiles the second code path costs the loop below registers it does not have.)
    if constexpr (NT == 1) {
        const int share = t_end - t_begin;
        if (ngroups == 2 * kWarps && (share == kRoundTiles || share == kRoundTiles - 1)) {
            float acc[kRoundTiles][4];
            uint4 xf[4];       // activation fragments of the current group: token gq, k = 128g + 32pp + 8c + (0..7)
            float neg_off[4];  // minus the group's offset contribution (see the dequantisation note above)
#pragma unroll
            for (int t = 0; t < kRoundTiles; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
            auto group_offsets = [&]() {
                // four chains of two MMAs, not one of eight: every warp of the CTA runs this pass
                // at the same moment (right after the activations arrive), so nothing hides a
                // long chain's latency
                float o[4][4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    mma_16816_first(o[pp], kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[pp].x, xf[pp].y);
                    mma_16816(o[pp], kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[pp].z, xf[pp].w);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) neg_off[i] = -((o[0][i] + o[1][i]) + (o[2][i] + o[3][i]));
            };
            // One 16 x 128 block against the group's activations, added into `a`. `done_reading`
            // runs as soon as the block's bytes are in registers (it frees the ring slot).
            auto block_math = [&](const uint8_t* blk, auto&& done_reading, float (&a)[4]) {
                const uint4 u0 = *reinterpret_cast<const uint4*>(blk + lane * 16);
                const uint4 u1 = *reinterpret_cast<const uint4*>(blk + 512 + lane * 16);
                const __half* sc = reinterpret_cast<const __half*>(blk + 1024);
                const float s_lo = __half2float(sc[gq]);
                const float s_hi = __half2float(sc[gq + 8]);
                done_reading();
                const uint32_t wA[4] = {u0.x, u0.z, u1.x, u1.z};  // column gq
                const uint32_t wB[4] = {u0.y, u0.w, u1.y, u1.w};  // column gq + 8
                // two independent chains of four MMAs (even and odd 16-wide K slices); the first
                // starts from the negated offsets, the second from zero
                float t0[4], t1[4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    const uint32_t hA = wA[pp] >> 8, hB = wB[pp] >> 8;
                    const uint32_t a0 = and_or(wA[pp], dq.mask_lo, dq.exp_lo), a1 = and_or(wB[pp], dq.mask_lo, dq.exp_lo);
                    const uint32_t a2 = and_or(wA[pp], dq.mask_hi, dq.exp_hi), a3 = and_or(wB[pp], dq.mask_hi, dq.exp_hi);
                    const uint32_t e0 = and_or(hA, dq.mask_lo, dq.exp_lo), e1 = and_or(hB, dq.mask_lo, dq.exp_lo);
                    const uint32_t e2 = and_or(hA, dq.mask_hi, dq.exp_hi), e3 = and_or(hB, dq.mask_hi, dq.exp_hi);
                    if (pp == 0) {
                        mma_16816_from(t0, neg_off, a0, a1, a2, a3, xf[pp].x, xf[pp].y);
                        mma_16816_first(t1, e0, e1, e2, e3, xf[pp].z, xf[pp].w);
                    } else {
                        mma_16816(t0, a0, a1, a2, a3, xf[pp].x, xf[pp].y);
                        mma_16816(t1, e0, e1, e2, e3, xf[pp].z, xf[pp].w);
                    }
                }
                a[0] = fmaf(s_lo, t1[0], fmaf(s_lo, t0[0], a[0]));
                a[1] = fmaf(s_lo, t1[1], fmaf(s_lo, t0[1], a[1]));
                a[2] = fmaf(s_hi, t1[2], fmaf(s_hi, t0[2], a[2]));
                a[3] = fmaf(s_hi, t1[3], fmaf(s_hi, t0[3], a[3]));
            };
            float* const mine = red + (size_t)warp * (kRoundTiles * 128);
            auto straight_line = [&](auto rt_const) {
                constexpr int RT = decltype(rt_const)::value;
                static_assert(RT >= kDepth, "the second group's activations must land before its first block");
                // K is known on this path, so every source of the warp is s0 plus a constant
                constexpr size_t kTileStride = (size_t)2 * kWarps * kBlkBytes;
                const uint8_t* const s0 = wmine + (size_t)t_begin * kTileStride + lane * 16;
                const uint8_t* const s1 = s0 + (size_t)kWarps * kBlkBytes;
                const uint32_t d0 = stage0 + lane * 16;
                // First group's activations straight into registers.
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    xf[pp] = make_uint4(0, 0, 0, 0);
                    if (gq < M)
                        xf[pp] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)gq * K + (size_t)warp * 128 + pp * 32 + c * 8));
                }
                // The second group's travel with the first block request after the wait, into
                // this warp's part of the reduction area (unused until the round ends), so that
                // the switch of groups does not wait on a global load.
                {
                    const uint32_t xdst = smem_u32(mine) + lane * 16;
                    const __half* xsrc = x + (size_t)(gq < M ? gq : 0) * K + (size_t)(kWarps + warp) * 128 + c * 8;
#pragma unroll
                    for (int pp = 0; pp < 4; ++pp) cp_async_16_zfill(xdst + pp * 512, xsrc + pp * 32, gq < M);
                }
                group_offsets();
                static_for<2 * RT>([&](auto b_const) {
                    constexpr int b = decltype(b_const)::value;
                    cp_async_wait<kDepth - 1>();  // blocks 0..b and, from b = kDepth on, the activations
                    __syncwarp();
                    if constexpr (b == RT) {
#pragma unroll
                        for (int pp = 0; pp < 4; ++pp)
                            xf[pp] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(mine) + pp * 512 + lane * 16);
                        group_offsets();
                    }
                    block_math(stage + (b % kDepth) * kBlkBytes,
                               [&]() {
                                   __syncwarp();
                                   constexpr int nb = b + kDepth;
                                   if constexpr (nb < 2 * RT) {
                                       const uint8_t* src = (nb < RT ? s0 : s1) + (size_t)(nb % RT) * kTileStride;
                                       const uint32_t dst = d0 + (nb % kDepth) * kBlkBytes;
                                       cp_async_16(dst, src);
                                       cp_async_16(dst + 512, src + 512);
                                       if (lane < 2) cp_async_16(dst + 1024, src + 1024);
                                   }
                                   cp_async_commit();  // one group per block, empty or not
                               },
                               acc[b % RT]);
                });
            };
            if (share == kRoundTiles)
                straight_line(std::integral_constant<int, kRoundTiles>());
            else
                straight_line(std::integral_constant<int, kRoundTiles - 1>());
            cp_async_wait<0>();  // only empty groups are left
            // ---- cross-warp reduction in warp order, then store (as in the loop below) ----
#pragma unroll
            for (int t = 0; t < kRoundTiles; ++t)
                *reinterpret_cast<float4*>(mine + t * 128 + lane * 4) = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
            __syncthreads();
            // One pass: thread e4 sums the 16 warps' copies of one lane's four accumulators of
            // one tile (sixteen 16-byte reads issued together, then four chains of adds in
            // warp order). With one float per thread the 640 sums of a five-tile share took
            // two dependent rounds on the first four warps, 0.5 us at the end of every launch.
            if ((int)threadIdx.x < share * 32) {
                const int e4 = threadIdx.x;
                float4 p[kWarps];
#pragma unroll
                for (int w = 0; w < kWarps; ++w)
                    p[w] = *reinterpret_cast<const float4*>(red + w * (kRoundTiles * 128) + e4 * 4);
                float v[4] = {p[0].x, p[0].y, p[0].z, p[0].w};
#pragma unroll
                for (int w = 1; w < kWarps; ++w) {
                    v[0] += p[w].x;
                    v[1] += p[w].y;
                    v[2] += p[w].z;
                    v[3] += p[w].w;
                }
                const int t = e4 >> 5, l = e4 & 31;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int col = (t_begin + t) * 16 + (l >> 2) + 8 * (i >> 1);
                    const int tok = 2 * (l & 3) + (i & 1);
                    if (tok < M) out[(size_t)tok * N + col] = __float2half_rn(v[i]);
                }
            }
            return;
        }
    }
    for (int r0 = t_begin; r0 < t_end; r0 += kRoundTiles) {
        const int rt = min(kRoundTiles, t_end - r0);
        float acc[kRoundTiles][NT][4];
#pragma unroll
        for (int t = 0; t < kRoundTiles; ++t)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[t][j][i] = 0.0f;
        for (int p = 0; p < my_phases; ++p) {
            const int g = p * kWarps + warp;
            // Activation fragments of this warp's group: token gq + 8j,
            // k = 128g + 32pp + 8c + (0..7).
            uint4 xf[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int tok = gq + 8 * j;
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    xf[j][pp] = make_uint4(0, 0, 0, 0);
                    if (tok < M)
                        xf[j][pp] = __ldg(reinterpret_cast<const uint4*>(
                            x + (size_t)tok * K + (size_t)g * 128 + pp * 32 + c * 8));
                }
            }
            // Offset contribution of this group (see the dequantisation note above): identical for
            // all 16 weight columns, so one MMA pass with a constant operand.
            float neg_off[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float o[4][4];  // the same four chains and the same sum as the straight-line path
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    mma_16816_first(o[pp], kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[j][pp].x, xf[j][pp].y);
                    mma_16816(o[pp], kOffsetLo, kOffsetLo, kOffsetHi, kOffsetHi, xf[j][pp].z, xf[j][pp].w);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) neg_off[j][i] = -((o[0][i] + o[1][i]) + (o[2][i] + o[3][i]));
            }
            auto tile_step = [&](const int t) {
                const uint8_t* blk = acquire();
                const uint4 u0 = *reinterpret_cast<const uint4*>(blk + lane * 16);
                const uint4 u1 = *reinterpret_cast<const uint4*>(blk + 512 + lane * 16);
                const __half* sc = reinterpret_cast<const __half*>(blk + 1024);
                const float s_lo = __half2float(sc[gq]);
                const float s_hi = __half2float(sc[gq + 8]);
                release();
                const uint32_t wA[4] = {u0.x, u0.z, u1.x, u1.z};  // column gq
                const uint32_t wB[4] = {u0.y, u0.w, u1.y, u1.w};  // column gq + 8
                // The two chains of the straight-line path, one after the other (a thread of this path
                // has no registers for both at once): the same operations in the same order per
                // output, so a token's result does not depend on which path computed it.
                float ch[NT][4];
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    const uint32_t a0 = and_or(wA[pp], dq.mask_lo, dq.exp_lo), a1 = and_or(wB[pp], dq.mask_lo, dq.exp_lo);
                    const uint32_t a2 = and_or(wA[pp], dq.mask_hi, dq.exp_hi), a3 = and_or(wB[pp], dq.mask_hi, dq.exp_hi);
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        if (pp == 0)
                            mma_16816_from(ch[j], neg_off[j], a0, a1, a2, a3, xf[j][pp].x, xf[j][pp].y);
                        else
                            mma_16816(ch[j], a0, a1, a2, a3, xf[j][pp].x, xf[j][pp].y);
                    }
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    acc[t][j][0] = fmaf(s_lo, ch[j][0], acc[t][j][0]);
                    acc[t][j][1] = fmaf(s_lo, ch[j][1], acc[t][j][1]);
                    acc[t][j][2] = fmaf(s_hi, ch[j][2], acc[t][j][2]);
                    acc[t][j][3] = fmaf(s_hi, ch[j][3], acc[t][j][3]);
                }
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) {
                    const uint32_t hA = wA[pp] >> 8, hB = wB[pp] >> 8;
                    const uint32_t e0 = and_or(hA, dq.mask_lo, dq.exp_lo), e1 = and_or(hB, dq.mask_lo, dq.exp_lo);
                    const uint32_t e2 = and_or(hA, dq.mask_hi, dq.exp_hi), e3 = and_or(hB, dq.mask_hi, dq.exp_hi);
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        if (pp == 0)
                            mma_16816_first(ch[j], e0, e1, e2, e3, xf[j][pp].z, xf[j][pp].w);
                        else
                            mma_16816(ch[j], e0, e1, e2, e3, xf[j][pp].z, xf[j][pp].w);
                    }
                }
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    acc[t][j][0] = fmaf(s_lo, ch[j][0], acc[t][j][0]);
                    acc[t][j][1] = fmaf(s_lo, ch[j][1], acc[t][j][1]);
                    acc[t][j][2] = fmaf(s_hi, ch[j][2], acc[t][j][2]);
                    acc[t][j][3] = fmaf(s_hi, ch[j][3], acc[t][j][3]);
                }
            };
            if (rt == kRoundTiles) {
#pragma unroll
                for (int t = 0; t < kRoundTiles; ++t) tile_step(t);
            } else {
#pragma unroll
                for (int t = 0; t < kRoundTiles; ++t)
                    if (t < rt) tile_step(t);
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
        __syncthreads();
        // thread e4 sums the warps' copies of one lane's four accumulators of one (tile, token
        // tile): all reads issued together, then four chains of adds in warp order
        const int nout4 = rt * NT * 32;
        for (int e4 = threadIdx.x; e4 < nout4; e4 += kWarps * 32) {
            float4 p[kWarps];
#pragma unroll
            for (int w = 0; w < kWarps; ++w)
                p[w] = *reinterpret_cast<const float4*>(red + w * (kRoundTiles * NT * 128) + e4 * 4);
            float v[4] = {p[0].x, p[0].y, p[0].z, p[0].w};
#pragma unroll
            for (int w = 1; w < kWarps; ++w) {
                v[0] += p[w].x;
                v[1] += p[w].y;
                v[2] += p[w].z;
                v[3] += p[w].w;
            }
            const int t = e4 / (NT * 32), j = (e4 / 32) % NT, l = e4 & 31;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int col = (r0 + t) * 16 + (l >> 2) + 8 * (i >> 1);
                const int tok = 8 * j + 2 * (l & 3) + (i & 1);
                if (tok < M) out[(size_t)tok * N + col] = __float2half_rn(v[i]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();  // only empty groups can be left; nothing may be pending at exit
}

// CTAs of a launch: one per SM (fewer for fewer column tiles than SMs). The straight-line path
// (up to 8 tokens, K = 4096) wants four or five column tiles per CTA; a matrix too wide for
// that in one wave runs as whole waves of such CTAs when the tile count allows it (N = 22016:
// 296 CTAs instead of 148 with nine or ten tiles each on the loop path). A CTA of a later wave
// starts when one of an earlier wave exits and finds the launch before long complete.
int decode_grid(int nt, int n, int k) {
    const int tiles = n / 16, sms = sm_count();
    if (nt == 1 && k == 2 * DecodeCfg<1>::unit_k && tiles > 5 * sms) {
        const int g = (tiles + 5 * sms - 1) / (5 * sms) * sms;
        if (tiles / g >= 4 && (tiles + g - 1) / g <= 5) return g;
    }
    return tiles < sms ? tiles : sms;
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
    const int grid = decode_grid(NT, n, k);
    return check_cuda(launch_pdl(int4_decode_kernel<NT>, (unsigned)grid, (unsigned)Cfg::threads, Cfg::smem_bytes, st,
                                 static_cast<const __half*>(x), static_cast<const uint8_t*>(wstream),
                                 static_cast<__half*>(out), m, n, k, tiles / grid, tiles % grid),
                      "int4_decode_kernel launch");
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A measurement aid, not part of the path: what a launch that does nothing but read `n16`
// 16-byte units costs in the same kind of dependent chain as the decode GEMM (programmatic
// dependent launch, one CTA of 512 threads per multiprocessor, the first 128 KB per CTA
// requested before griddepcontrol.wait, one word that the launch before wrote read after
// it). The decode kernel's launch time is held against this as well as against the copy
// bandwidth: a chain of 23 MB launches cannot run at the bandwidth of a long copy.
constexpr int kProbeUnroll = 16;
__global__ void __launch_bounds__(512, 1)
    chain_read_probe_kernel(const uint4* __restrict__ w, size_t n16, uint32_t* __restrict__ link) {
    pdl_launch_dependents();
    const size_t per = (n16 + gridDim.x - 1) / gridDim.x;
    const size_t b0 = (size_t)blockIdx.x * per, b1 = b0 + per < n16 ? b0 + per : n16;
    uint32_t acc = 0;
    size_t i = b0 + threadIdx.x;
    uint4 v[kProbeUnroll];
#pragma unroll
    for (int u = 0; u < kProbeUnroll; ++u) {
        const size_t j = i + (size_t)u * 512;
        v[u] = j < b1 ? __ldcs(w + j) : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
    const uint32_t dep = link[threadIdx.x & 31];  // written by the launch before this one
    for (;;) {
#pragma unroll
        for (int u = 0; u < kProbeUnroll; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
        i += (size_t)kProbeUnroll * 512;
        if (i >= b1) break;
#pragma unroll
        for (int u = 0; u < kProbeUnroll; ++u) {
            const size_t j = i + (size_t)u * 512;
            v[u] = j < b1 ? __ldcs(w + j) : make_uint4(0, 0, 0, 0);
        }
    }
    // every CTA's sum feeds the word the next launch reads, so no load can be dropped
    if (threadIdx.x == 0 && blockIdx.x < 32) link[blockIdx.x] = (acc ^ dep) | 1u;
    else if (acc == 0x9e3779b9u) link[32 + (threadIdx.x & 31)] = acc;
}

}  // namespace

// Launch geometry of the decode kernel for the host launch API.
void decode_launch_geometry(int m, int n, int k, unsigned* grid, unsigned* block, unsigned* smem, int* slots,
                            int* unit_k) {
    *grid = n > 0 ? (unsigned)decode_grid(m <= 8 ? 1 : (m <= 16 ? 2 : 4), n, k) : 0u;
    if (m <= 8) { *block = DecodeCfg<1>::threads; *smem = DecodeCfg<1>::smem_bytes; *slots = DecodeCfg<1>::depth; *unit_k = DecodeCfg<1>::unit_k; }
    else if (m <= 16) { *block = DecodeCfg<2>::threads; *smem = DecodeCfg<2>::smem_bytes; *slots = DecodeCfg<2>::depth; *unit_k = DecodeCfg<2>::unit_k; }
    else { *block = DecodeCfg<4>::threads; *smem = DecodeCfg<4>::smem_bytes; *slots = DecodeCfg<4>::depth; *unit_k = DecodeCfg<4>::unit_k; }
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
    dim3 grid((unsigned)((n + 127) / 128), (unsigned)(k / 128));
    int4_quantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
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
    const size_t total_blocks = (n / 16) * (k / 128);  // 1056-byte blocks, one warp each
    size_t ctas = (total_blocks + 7) / 8;
    const size_t cap = (size_t)sm_count() * 16;
    if (ctas > cap) ctas = cap;
    int4_repack_kernel<<<(unsigned)ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        qweight, static_cast<const uint16_t*>(scales_f16), k / 128, n, total_blocks,
        static_cast<uint32_t*>(wstream));
    return check_cuda(cudaGetLastError(), "int4_repack_kernel launch");
}

extern "C" int y_b200_probe_chain_read(const void* const* bufs, int nbufs, size_t bytes, int launches,
                                       int reps, void* scratch_256, float* us_per_launch, void* stream) {
    if (!bufs || nbufs < 1 || !scratch_256 || !us_per_launch)
        return fail(Y_B200_ERR_INVALID, "y_b200_probe_chain_read: null pointer or no buffers");
    if (bytes < 16 || bytes % 16 != 0 || launches < 1 || reps < 1 || reps > 64)
        return fail(Y_B200_ERR_SHAPE, "y_b200_probe_chain_read: bytes %% 16 == 0, launches >= 1, 1 <= reps <= 64");
    for (int i = 0; i < nbufs; ++i)
        if (!bufs[i] || !aligned16(bufs[i])) return fail(Y_B200_ERR_ALIGN, "y_b200_probe_chain_read: buffer %d null or not 16-byte aligned", i);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* link = static_cast<uint32_t*>(scratch_256);
    YB_CUDA(cudaMemsetAsync(link, 0, 256, st));
    cudaEvent_t e0, e1;
    YB_CUDA(cudaEventCreate(&e0));
    YB_CUDA(cudaEventCreate(&e1));
    float sorted[64];
    cudaError_t err = cudaSuccess;
    for (int r = -1; r < reps && err == cudaSuccess; ++r) {  // r = -1: warm-up
        if (r >= 0) err = cudaEventRecord(e0, st);
        for (int i = 0; i < launches && err == cudaSuccess; ++i)
            err = launch_pdl(chain_read_probe_kernel, (unsigned)sm_count(), 512u, 0, st,
                             static_cast<const uint4*>(bufs[i % nbufs]), bytes / 16, link);
        if (r >= 0 && err == cudaSuccess) {
            err = cudaEventRecord(e1, st);
            if (err == cudaSuccess) err = cudaEventSynchronize(e1);
            float ms = 0.0f;
            if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
            sorted[r] = ms * 1000.0f / (float)launches;
        }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (err != cudaSuccess) return check_cuda(err, "y_b200_probe_chain_read");
    std::sort(sorted, sorted + reps);
    *us_per_launch = sorted[reps / 2];
    return Y_B200_OK;
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
