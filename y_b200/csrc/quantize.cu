// HBM-bound kernels of the FP8 path: abs-max reduce, e4m3 quantise (plain and
// transposed), RMSNorm -> e4m3 prologue, and the device-side input generator.
// All global traffic is 128-bit per thread; reductions are warp-shuffle plus
// one atomic per CTA on the f32 bit pattern (non-negative floats order like
// unsigned integers, so max needs no floating-point atomics and is exact).
#include "common.cuh"

namespace yb {
namespace {

constexpr int kThreads = 256;

// ---- loads of 8 elements as f32 ---------------------------------------------
template <int KIND>
struct Elem;
template <>
struct Elem<Y_B200_F16> {
    __device__ static void load8(const void* p, size_t i, float (&v)[8]) {
        uint4 u = *reinterpret_cast<const uint4*>(static_cast<const __half*>(p) + i);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    }
    __device__ static float load1(const void* p, size_t i) {
        return __half2float(static_cast<const __half*>(p)[i]);
    }
};
template <>
struct Elem<Y_B200_BF16> {
    __device__ static void load8(const void* p, size_t i, float (&v)[8]) {
        uint4 u = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + i);
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
    __device__ static float load1(const void* p, size_t i) {
        return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    }
};
template <>
struct Elem<Y_B200_F32> {
    __device__ static void load8(const void* p, size_t i, float (&v)[8]) {
        const float4* q = reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
        float4 a = q[0], b = q[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    __device__ static float load1(const void* p, size_t i) {
        return static_cast<const float*>(p)[i];
    }
};

// Eight 16-bit elements held in a uint4 -> f32 (KIND is F16 or BF16).
template <int KIND>
__device__ __forceinline__ void unpack8(const uint4& u, float (&v)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (KIND == Y_B200_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        } else {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

__device__ __forceinline__ void block_atomic_max(float local, unsigned int* out) {
    __shared__ unsigned int warp_max[kThreads / 32];
    unsigned int bits = __float_as_uint(local);  // local >= 0
    bits = warp_max_u32(bits);
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = bits;
    __syncthreads();
    if (threadIdx.x < 32) {
        unsigned int v = threadIdx.x < kThreads / 32 ? warp_max[threadIdx.x] : 0u;
        v = warp_max_u32(v);
        if (threadIdx.x == 0 && v != 0u) atomicMax(out, v);
    }
}

// ---- amax ----------------------------------------------------------------------
// n8 = number of aligned 8-element vectors; the scalar tail [n8*8, n) is folded
// in by the first threads of block 0.
template <int KIND>
__global__ void __launch_bounds__(kThreads) amax_kernel(const void* __restrict__ x, size_t n,
                                                        unsigned int* __restrict__ out) {
    pdl_wait();
    const size_t n8 = n / 8;
    float m = 0.0f;
    // four independent vectors per trip, so a thread has 64 bytes (128 for f32) in flight
    const size_t stride = (size_t)gridDim.x * kThreads;
    size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (; v + 3 * stride < n8; v += 4 * stride) {
        float f[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) Elem<KIND>::load8(x, (v + u * stride) * 8, f[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[u][j]));
    }
    for (; v < n8; v += stride) {
        float f[8];
        Elem<KIND>::load8(x, v * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    }
    if (blockIdx.x == 0) {
        size_t i = n8 * 8 + threadIdx.x;
        if (i < n) m = fmaxf(m, fabsf(Elem<KIND>::load1(x, i)));
    }
    pdl_launch_dependents();
    block_atomic_max(m, out);
}

__global__ void scale_from_amax_kernel(const float* amax, float* scale) {
    pdl_wait();
    scale[0] = scale_from_amax(amax[0]);
}

// ---- quantise --------------------------------------------------------------------
// SCALE_IS_AMAX: `s` points at an amax; the scale is derived on the fly and
// thread 0 publishes it to scale_out.
template <int KIND, bool SCALE_IS_AMAX>
__global__ void __launch_bounds__(kThreads)
    quantize_kernel(const void* __restrict__ x, size_t n, const float* __restrict__ s, float s_val,
                    uint8_t* __restrict__ q, float* __restrict__ scale_out) {
    pdl_wait();
    pdl_launch_dependents();
    const float scale = s == nullptr ? s_val : (SCALE_IS_AMAX ? scale_from_amax(s[0]) : s[0]);
    const float inv = inv_scale(scale);
    if (SCALE_IS_AMAX && scale_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0)
        scale_out[0] = scale;
    const size_t n16 = n / 16;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n16;
         i += (size_t)gridDim.x * kThreads) {
        // After an amax pass over the same tensor (first to last) the end of it is what L2 still
        // holds: walk it last to first.
        const size_t v = SCALE_IS_AMAX ? n16 - 1 - i : i;
        float a[8], b[8];
        Elem<KIND>::load8(x, v * 16, a);
        Elem<KIND>::load8(x, v * 16 + 8, b);
        uint4 o;
        o.x = cvt_e4m3x4(__fmul_rn(a[0], inv), __fmul_rn(a[1], inv), __fmul_rn(a[2], inv),
                         __fmul_rn(a[3], inv));
        o.y = cvt_e4m3x4(__fmul_rn(a[4], inv), __fmul_rn(a[5], inv), __fmul_rn(a[6], inv),
                         __fmul_rn(a[7], inv));
        o.z = cvt_e4m3x4(__fmul_rn(b[0], inv), __fmul_rn(b[1], inv), __fmul_rn(b[2], inv),
                         __fmul_rn(b[3], inv));
        o.w = cvt_e4m3x4(__fmul_rn(b[4], inv), __fmul_rn(b[5], inv), __fmul_rn(b[6], inv),
                         __fmul_rn(b[7], inv));
        *reinterpret_cast<uint4*>(q + v * 16) = o;
    }
    if (blockIdx.x == 0) {
        size_t i = n16 * 16 + threadIdx.x;
        if (i < n) q[i] = (uint8_t)(cvt_e4m3x2(__fmul_rn(Elem<KIND>::load1(x, i), inv), 0.0f) & 0xff);
    }
}

// ---- transposed quantise -----------------------------------------------------------
// x [rows, cols] -> q [cols, rows]. One CTA moves a 128(row) x 64(col) tile
// through shared memory so both the reads (along cols) and the writes (along
// rows) are contiguous. A thread converts 4 rows x 8 columns and stores, per
// column, one 32-bit word holding its 4 row bytes; the word index within a
// tile row is XORed with 4 * (column / 8), which spreads the 32 lanes of a warp
// over the 32 banks and keeps every aligned group of 4 words together for the
// 16-byte reads of the second phase. Edges are handled element-wise.
constexpr int kTR = 128, kTC = 64;
template <int KIND, bool SCALE_IS_AMAX>
__global__ void __launch_bounds__(kThreads)
    quantize_transpose_kernel(const void* __restrict__ x, size_t rows, size_t cols,
                              const float* __restrict__ s, float s_val, uint8_t* __restrict__ q,
                              float* __restrict__ scale_out) {
    __shared__ __align__(16) uint32_t tile[kTC][kTR / 4];
    pdl_wait();
    pdl_launch_dependents();
    const float scale = s == nullptr ? s_val : (SCALE_IS_AMAX ? scale_from_amax(s[0]) : s[0]);
    const float inv = inv_scale(scale);
    if (SCALE_IS_AMAX && scale_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 &&
        threadIdx.x == 0)
        scale_out[0] = scale;
    const size_t r0 = (size_t)blockIdx.y * kTR, c0 = (size_t)blockIdx.x * kTC;
    const bool vec_in = (cols % 8 == 0);
    {
        // 32 row quads x 8 column vectors = 256 slots, one per thread.
        const int rq = threadIdx.x / 8, cv = threadIdx.x % 8;
        const size_t gc = c0 + (size_t)cv * 8;
        float f[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const size_t gr = r0 + (size_t)rq * 4 + i;
            if (gr < rows && vec_in && gc + 8 <= cols) {
                Elem<KIND>::load8(x, gr * cols + gc, f[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    f[i][j] = (gr < rows && gc + j < cols) ? Elem<KIND>::load1(x, gr * cols + gc + j) : 0.0f;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            tile[cv * 8 + j][rq ^ (cv * 4)] =
                cvt_e4m3x4(__fmul_rn(f[0][j], inv), __fmul_rn(f[1][j], inv), __fmul_rn(f[2][j], inv),
                           __fmul_rn(f[3][j], inv));
    }
    __syncthreads();
    // 64 output rows x 8 sixteen-byte vectors = 512 slots, 2 per thread.
    const bool vec_out = (rows % 16 == 0);
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int slot = it * kThreads + threadIdx.x;
        const int c = slot / 8, rv = slot % 8;
        const size_t gc = c0 + c, gr = r0 + (size_t)rv * 16;
        if (gc >= cols) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(&tile[c][(rv ^ (c / 8)) * 4]);
        if (vec_out && gr + 16 <= rows) {
            *reinterpret_cast<uint4*>(q + gc * rows + gr) = v;
        } else {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            for (int j = 0; j < 16; ++j)
                if (gr + j < rows) q[gc * rows + gr + j] = (uint8_t)(w[j / 4] >> (8 * (j % 4)));
        }
    }
}

// Full-tile, 16-bit-input variant: a CTA walks a strip of row tiles of one 64-column
// band. The next tile's loads are issued before the current tile is converted, and the
// shared-memory tile is double-buffered, so a CTA always has 16 KB of loads in flight and
// synchronises once per tile. Same tile layout and swizzle as above.
template <int KIND, bool SCALE_IS_AMAX>
__global__ void __launch_bounds__(kThreads)
    quantize_transpose_strip_kernel(const uint16_t* __restrict__ x, size_t rows, size_t cols,
                                    const float* __restrict__ s, float s_val, uint8_t* __restrict__ q,
                                    float* __restrict__ scale_out, int tiles_per_cta) {
    __shared__ __align__(16) uint32_t tile[2][kTC][kTR / 4];
    pdl_wait();
    pdl_launch_dependents();
    const float scale = s == nullptr ? s_val : (SCALE_IS_AMAX ? scale_from_amax(s[0]) : s[0]);
    const float inv = inv_scale(scale);
    if (SCALE_IS_AMAX && scale_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 &&
        threadIdx.x == 0)
        scale_out[0] = scale;
    const size_t c0 = (size_t)blockIdx.x * kTC;
    const int row_tiles = (int)(rows / kTR);
    // after an amax pass the last rows are what L2 still holds: the strips that start first take those
    const int strip = SCALE_IS_AMAX ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
    const int rt0 = strip * tiles_per_cta, rt1 = min(rt0 + tiles_per_cta, row_tiles);
    const int rq = threadIdx.x / 8, cv = threadIdx.x % 8;
    const uint16_t* xin = x + c0 + (size_t)cv * 8 + (size_t)rq * 4 * cols;  // row rq*4 of tile 0
    const int oc0 = threadIdx.x / 8, orv = threadIdx.x % 8;                // write-out slots
    uint4 cur[4], nxt[4];
    auto load_tile = [&](int rt, uint4 (&dst)[4]) {
        const uint16_t* p = xin + (size_t)rt * kTR * cols;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = *reinterpret_cast<const uint4*>(p + (size_t)i * cols);
    };
    if (rt0 < rt1) load_tile(rt0, cur);
    int b = 0;
    for (int rt = rt0; rt < rt1; ++rt, b ^= 1) {
        if (rt + 1 < rt1) load_tile(rt + 1, nxt);
        float f[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) unpack8<KIND>(cur[i], f[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            tile[b][cv * 8 + j][rq ^ (cv * 4)] =
                cvt_e4m3x4(__fmul_rn(f[0][j], inv), __fmul_rn(f[1][j], inv), __fmul_rn(f[2][j], inv),
                           __fmul_rn(f[3][j], inv));
        __syncthreads();
        const size_t r0 = (size_t)rt * kTR;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int c = oc0 + it * 32;
            *reinterpret_cast<uint4*>(q + (c0 + c) * rows + r0 + (size_t)orv * 16) =
                *reinterpret_cast<const uint4*>(&tile[b][c][(orv ^ (c / 8)) * 4]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
    }
}

// ---- RMSNorm -> e4m3 ------------------------------------------------------------------
// One 256-thread CTA per row. The sum of squares follows a FIXED order so the
// result can be reproduced bit for bit on a CPU: thread t folds the 8-element
// vectors t, t+256, ... with fma(x, x, acc); each warp adds its 32 partials by
// butterfly (xor 16, 8, 4, 2, 1); the eight warp totals are added in warp
// order; mean = total / hidden; rstd = 1 / sqrt(mean + eps) with correctly
// rounded division and square root. y = (x * rstd) * gamma.
// Adds the thread's partial sums in the fixed order described above. `warp_tot` is
// the caller's eight-float scratch; callers that loop alternate between two of them.
__device__ __forceinline__ float rms_rstd_from_partial(float acc, size_t hidden, float eps, float* warp_tot) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = warp_tot[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total = __fadd_rn(total, warp_tot[w]);
    const float mean = __fdiv_rn(total, (float)hidden);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

// acc = fma(a, a, acc) for both f16 halves of `w`, low half first: the product of
// two f16 values is exact in f32, so this is the f32 fma on the converted values
// without the conversions.
__device__ __forceinline__ float fma_sq_f16x2(uint32_t w, float acc) {
    const unsigned short lo = (unsigned short)(w & 0xffffu), hi = (unsigned short)(w >> 16);
    asm("fma.rn.f32.f16 %0, %1, %1, %0;" : "+f"(acc) : "h"(lo));
    asm("fma.rn.f32.f16 %0, %1, %1, %0;" : "+f"(acc) : "h"(hi));
    return acc;
}

// Any row length: one CTA per row, the row is read twice (the second time from L1/L2).
__global__ void __launch_bounds__(kThreads)
    rmsnorm_stats_long_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma,
                              size_t hidden, float eps, float* __restrict__ rstd_out,
                              unsigned int* __restrict__ amax_out) {
    __shared__ float warp_tot[8];
    pdl_wait();
    const __half* xr = x + (size_t)blockIdx.x * hidden;
    const size_t nvec = hidden / 8;
    float acc = 0.0f;
    for (size_t v = threadIdx.x; v < nvec; v += kThreads) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + v * 8);
        acc = fma_sq_f16x2(u.x, acc);
        acc = fma_sq_f16x2(u.y, acc);
        acc = fma_sq_f16x2(u.z, acc);
        acc = fma_sq_f16x2(u.w, acc);
    }
    const float rstd = rms_rstd_from_partial(acc, hidden, eps, warp_tot);
    if (threadIdx.x == 0) rstd_out[blockIdx.x] = rstd;
    float m = 0.0f;
    for (size_t v = threadIdx.x; v < nvec; v += kThreads) {
        float f[8], g[8];
        Elem<Y_B200_F16>::load8(xr, v * 8, f);
        Elem<Y_B200_F16>::load8(gamma, v * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(f[j], rstd), g[j])));
    }
    block_atomic_max(m, amax_out);
}

// Rows of at most VPT * 256 vectors: persistent CTAs walk the rows; gamma sits in
// shared memory as f32 (converted once per CTA); a row is read once and stays in
// registers between the sum of squares and the amax, and the next row's loads are
// issued before the current row is worked on, so DRAM latency overlaps the arithmetic.
template <int VPT>
struct RowRegs {
    uint4 v[VPT];
};

template <int VPT>
__device__ __forceinline__ void stats_load_row(const uint4* __restrict__ xv, size_t row, uint32_t nvec,
                                               RowRegs<VPT>& r) {
    const uint4* p = xv + row * nvec + threadIdx.x;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
        r.v[i] = threadIdx.x + i * kThreads < nvec ? p[i * kThreads] : make_uint4(0u, 0u, 0u, 0u);
}

template <int VPT>
__device__ __forceinline__ float stats_row(const RowRegs<VPT>& r, uint32_t nvec, size_t hidden, float eps,
                                           const float* gamma_s, float* warp_tot, float* rstd_slot, float m) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {  // absent vectors are zeros: fma(0, 0, acc) = acc
        acc = fma_sq_f16x2(r.v[i].x, acc);
        acc = fma_sq_f16x2(r.v[i].y, acc);
        acc = fma_sq_f16x2(r.v[i].z, acc);
        acc = fma_sq_f16x2(r.v[i].w, acc);
    }
    const float rstd = rms_rstd_from_partial(acc, hidden, eps, warp_tot);
    if (threadIdx.x == 0) *rstd_slot = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const uint32_t v = threadIdx.x + i * kThreads;
        if (v >= nvec) continue;
        const float4* gs = reinterpret_cast<const float4*>(gamma_s) + 2 * v;
        const float4 g0 = gs[0], g1 = gs[1];
        const __half2* h = reinterpret_cast<const __half2*>(&r.v[i]);
        const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        const float2 c = __half22float2(h[2]), d = __half22float2(h[3]);
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(a.x, rstd), g0.x)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(a.y, rstd), g0.y)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(b.x, rstd), g0.z)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(b.y, rstd), g0.w)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(c.x, rstd), g1.x)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(c.y, rstd), g1.y)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(d.x, rstd), g1.z)));
        m = fmaxf(m, fabsf(__fmul_rn(__fmul_rn(d.y, rstd), g1.w)));
    }
    return m;
}

template <int VPT>
__global__ void __launch_bounds__(kThreads, 4)
    rmsnorm_stats_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma, size_t rows,
                         size_t hidden, float eps, float* __restrict__ rstd_out,
                         unsigned int* __restrict__ amax_out) {
    extern __shared__ __align__(16) float gamma_s[];
    // Two reduction scratch arrays used in turn: a warp that is already in the next row
    // writes the other one while a slower warp still reads this one.
    __shared__ float warp_tot[2][8];
    pdl_wait();
    const uint32_t nvec = (uint32_t)(hidden / 8);
    for (uint32_t v = threadIdx.x; v < nvec; v += kThreads) {
        float g[8];
        Elem<Y_B200_F16>::load8(gamma, (size_t)v * 8, g);
        float4* d = reinterpret_cast<float4*>(gamma_s) + 2 * v;
        d[0] = make_float4(g[0], g[1], g[2], g[3]);
        d[1] = make_float4(g[4], g[5], g[6], g[7]);
    }
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    const size_t stride = gridDim.x;
    RowRegs<VPT> ra, rb;
    size_t row = blockIdx.x;
    if (row < rows) stats_load_row<VPT>(xv, row, nvec, ra);
    __syncthreads();
    float m = 0.0f;
    while (row < rows) {
        const size_t row1 = row + stride;
        if (row1 < rows) stats_load_row<VPT>(xv, row1, nvec, rb);
        m = stats_row<VPT>(ra, nvec, hidden, eps, gamma_s, warp_tot[0], rstd_out + row, m);
        if (row1 >= rows) break;
        row = row1 + stride;
        if (row < rows) stats_load_row<VPT>(xv, row, nvec, ra);
        m = stats_row<VPT>(rb, nvec, hidden, eps, gamma_s, warp_tot[1], rstd_out + row1, m);
    }
    // Only now: dependents that become resident early and sit in their wait slow this
    // kernel down (measured: +10 us at 8192 x 8192 when triggered at the top).
    pdl_launch_dependents();
    block_atomic_max(m, amax_out);
}

__global__ void __launch_bounds__(kThreads)
    rmsnorm_quantize_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma,
                            size_t hidden, const float* __restrict__ rstd_in,
                            const float* __restrict__ amax, uint8_t* __restrict__ q,
                            float* __restrict__ scale_out) {
    pdl_wait();  // the statistics kernel has finished: amax and rstd are final
    pdl_launch_dependents();
    const float scale = scale_from_amax(amax[0]);
    const float inv = inv_scale(scale);
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out != nullptr) scale_out[0] = scale;
    // Rows are taken last to first: the statistics kernel ran first to last, so the
    // rows it touched most recently, which L2 still holds, are read first.
    const size_t row = gridDim.x - 1 - blockIdx.x;
    const __half* xr = x + row * hidden;
    uint8_t* qr = q + row * hidden;
    const float rstd = rstd_in[row];
    const size_t nvec = hidden / 8;
    for (size_t v = threadIdx.x; v < nvec; v += kThreads) {
        float f[8], g[8];
        Elem<Y_B200_F16>::load8(xr, v * 8, f);
        Elem<Y_B200_F16>::load8(gamma, v * 8, g);
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = __fmul_rn(__fmul_rn(__fmul_rn(f[j], rstd), g[j]), inv);
        uint2 o;
        o.x = cvt_e4m3x4(y[0], y[1], y[2], y[3]);
        o.y = cvt_e4m3x4(y[4], y[5], y[6], y[7]);
        *reinterpret_cast<uint2*>(qr + v * 8) = o;
    }
}

// ---- fused add + RMSNorm with the residual stream (f16 in, f16 out) ------------------------
// h = x + residual in f32; total = sum(h^2) in the fixed order above; mean = total * (1/hidden);
// out = f16((h * rstd) * w); new_residual = f16(h). One 256-thread CTA per row. VPT > 0: the
// row (at most VPT * 256 vectors) lives in registers as f32 between the two phases, so x and
// residual are read once; VPT == 0: any length, the second phase re-reads them.
__device__ __forceinline__ void add8_f16(const uint4& a, const uint4& b, float (&h)[8]) {
    float fa[8], fb[8];
    unpack8<Y_B200_F16>(a, fa);
    unpack8<Y_B200_F16>(b, fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = __fadd_rn(fa[j], fb[j]);
}

__device__ __forceinline__ uint4 pack8_f16(const float (&v)[8]) {
    return make_uint4(pack_f16x2(v[0], v[1]), pack_f16x2(v[2], v[3]), pack_f16x2(v[4], v[5]),
                      pack_f16x2(v[6], v[7]));
}

template <int VPT>
__global__ void __launch_bounds__(kThreads)
    rmsnorm_residual_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
                            const __half* __restrict__ weight, size_t hidden, float eps,
                            __half* __restrict__ out, __half* __restrict__ new_residual) {
    __shared__ float warp_tot[8];
    pdl_wait();
    pdl_launch_dependents();
    const size_t row0 = (size_t)blockIdx.x * hidden;
    const uint4* xv = reinterpret_cast<const uint4*>(x + row0);
    const uint4* rv = reinterpret_cast<const uint4*>(residual + row0);
    const uint4* wv = reinterpret_cast<const uint4*>(weight);
    uint4* ov = reinterpret_cast<uint4*>(out + row0);
    uint4* nv = reinterpret_cast<uint4*>(new_residual + row0);
    const uint32_t nvec = (uint32_t)(hidden / 8);
    const float inv_hidden = __fdiv_rn(1.0f, (float)hidden);
    float acc = 0.0f;
    if constexpr (VPT > 0) {
        float h[VPT][8];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const uint32_t v = threadIdx.x + i * kThreads;
            if (v < nvec) {
                add8_f16(xv[v], rv[v], h[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) h[i][j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = __fmaf_rn(h[i][j], h[i][j], acc);
        }
        // Same reduction order as the prologue kernels; the mean is total * (1 / hidden)
        // here (a multiply, as in the reference kernel), not a division.
        float total;
        {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
            if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = acc;
            __syncthreads();
            total = warp_tot[0];
#pragma unroll
            for (int w = 1; w < 8; ++w) total = __fadd_rn(total, warp_tot[w]);
        }
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(total, inv_hidden), eps)));
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const uint32_t v = threadIdx.x + i * kThreads;
            if (v >= nvec) continue;
            float g[8], y[8];
            unpack8<Y_B200_F16>(wv[v], g);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = __fmul_rn(__fmul_rn(h[i][j], rstd), g[j]);
            ov[v] = pack8_f16(y);
            nv[v] = pack8_f16(h[i]);
        }
    } else {
        for (uint32_t v = threadIdx.x; v < nvec; v += kThreads) {
            float h[8];
            add8_f16(xv[v], rv[v], h);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = __fmaf_rn(h[j], h[j], acc);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
        if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = acc;
        __syncthreads();
        float total = warp_tot[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) total = __fadd_rn(total, warp_tot[w]);
        const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(total, inv_hidden), eps)));
        for (uint32_t v = threadIdx.x; v < nvec; v += kThreads) {
            float h[8], g[8], y[8];
            add8_f16(xv[v], rv[v], h);
            unpack8<Y_B200_F16>(wv[v], g);
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = __fmul_rn(__fmul_rn(h[j], rstd), g[j]);
            ov[v] = pack8_f16(y);
            nv[v] = pack8_f16(h);
        }
    }
}

// ---- rotary position embedding (interleaved pairs), f16 in and out ---------------------------
// A row is one token's query or key vector of one head.
// inv_freq comes in as a kernel parameter (the host computes base^(-2i/head_dim) in double
// precision once per call), theta = f32(pos) * inv_freq[i], and sin/cos are taken after a
// two-term Cody-Waite reduction to [-pi, pi] so the fast units stay accurate at positions
// in the thousands.
constexpr int kRopeMaxPairs = 128;  // head_dim <= 256
struct RopeTable {
    float inv_freq[kRopeMaxPairs];
};

__device__ __forceinline__ void sincos_reduced(float theta, float& s, float& c) {
    const float n = rintf(__fmul_rn(theta, 0.15915494309189535f));  // theta / 2pi
    float r = __fmaf_rn(-n, 6.28318548202514648f, theta);           // 2pi = hi + lo
    r = __fmaf_rn(-n, -1.74845553146951715e-7f, r);
    s = __sinf(r);
    c = __cosf(r);
}

// A warp works on spans of 128 consecutive pairs (512 bytes: one row of head 256, two of
// head 128, four of head 64), lane L on the four pairs [4L, 4L + 3] of the span, so every
// load and store is 16 bytes whatever the head size. Four spans are loaded before the first
// is rotated, which keeps 64 bytes per lane in flight.
constexpr int kRopeSpansPerWarp = 4;

template <int HEAD_DIM>
__global__ void __launch_bounds__(kThreads)
    rope_kernel(const __half* __restrict__ x, const int* __restrict__ positions, __half* __restrict__ out,
                size_t rows, const __grid_constant__ RopeTable table) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int pairs_per_row = HEAD_DIM / 2, rows_per_span = 128 / pairs_per_row, S = kRopeSpansPerWarp;
    // The table goes to shared memory once per CTA: lanes index it differently, and a
    // constant-bank load with 16 distinct addresses per warp is replayed 16 times (the
    // MIO-throttle stalls ncu showed at head 128).
    __shared__ __align__(16) float s_inv[kRopeMaxPairs];
    if (threadIdx.x < pairs_per_row) s_inv[threadIdx.x] = table.inv_freq[threadIdx.x];
    __syncthreads();
    const size_t spans = (rows + rows_per_span - 1) / rows_per_span;
    const size_t span0 = ((size_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5)) * S;
    if (span0 >= spans) return;
    const int lane = threadIdx.x & 31;
    const int row_in_span = (lane * 4) / pairs_per_row, pair0 = (lane * 4) % pairs_per_row;
    uint4 w[S];
    float pos[S];
    bool live[S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        const size_t row = (span0 + s) * rows_per_span + row_in_span;
        live[s] = row < rows;
        if (live[s]) {
            pos[s] = (float)positions[row];
            w[s] = *reinterpret_cast<const uint4*>(x + row * HEAD_DIM + pair0 * 2);
        }
    }
    const float4 fr = *reinterpret_cast<const float4*>(s_inv + pair0);
    const float inv_freq[4] = {fr.x, fr.y, fr.z, fr.w};
#pragma unroll
    for (int s = 0; s < S; ++s) {
        if (!live[s]) continue;
        uint32_t v[4] = {w[s].x, w[s].y, w[s].z, w[s].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float theta = __fmul_rn(pos[s], inv_freq[j]);
            float sn, cs;
            sincos_reduced(theta, sn, cs);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[j]));
            const float o0 = __fsub_rn(__fmul_rn(f.x, cs), __fmul_rn(f.y, sn));
            const float o1 = __fadd_rn(__fmul_rn(f.x, sn), __fmul_rn(f.y, cs));
            v[j] = pack_f16x2(o0, o1);
        }
        const size_t row = (span0 + s) * rows_per_span + row_in_span;
        *reinterpret_cast<uint4*>(out + row * HEAD_DIM + pair0 * 2) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// ---- input generator --------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t index, uint64_t seed) {
    uint64_t z = index * 0x9E3779B97F4A7C15ull + seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__global__ void fill_random_f16_kernel(uint16_t* out, size_t n, uint64_t index0, uint64_t seed) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        uint64_t z = splitmix64(index0 + i, seed);
        uint16_t sign = (uint16_t)((z >> 63) & 1u);
        uint16_t exp = (uint16_t)(12u + (uint16_t)((z >> 40) & 0x3u) % 3u);
        out[i] = (uint16_t)((sign << 15) | (exp << 10) | (uint16_t)(z & 0x3ffu));
    }
}

int grid_for(size_t work_items) {
    size_t want = (work_items + kThreads - 1) / kThreads;
    size_t cap = (size_t)sm_count() * 8;
    if (want < 1) want = 1;
    return (int)(want < cap ? want : cap);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int kind_ok(int kind) { return kind == Y_B200_F32 || kind == Y_B200_F16 || kind == Y_B200_BF16; }

template <bool IS_AMAX>
int launch_quantize(const void* x, int kind, size_t n, const float* s, float s_val, void* q, float* scale_out,
                    cudaStream_t st) {
    int grid = grid_for(n / 16 + 1);
    uint8_t* qq = static_cast<uint8_t*>(q);
    switch (kind) {
        case Y_B200_F16:
            YB_CUDA(launch_pdl(quantize_kernel<Y_B200_F16, IS_AMAX>, grid, kThreads, 0, st, x, n, s, s_val, qq, scale_out));
            break;
        case Y_B200_BF16:
            YB_CUDA(launch_pdl(quantize_kernel<Y_B200_BF16, IS_AMAX>, grid, kThreads, 0, st, x, n, s, s_val, qq, scale_out));
            break;
        default:
            YB_CUDA(launch_pdl(quantize_kernel<Y_B200_F32, IS_AMAX>, grid, kThreads, 0, st, x, n, s, s_val, qq, scale_out));
            break;
    }
    return check_cuda(cudaGetLastError(), "quantize_kernel launch");
}

template <bool IS_AMAX>
int launch_quantize_t(const void* x, int kind, size_t rows, size_t cols, const float* s, float s_val, void* q,
                      float* scale_out, cudaStream_t st) {
    dim3 grid((unsigned)((cols + kTC - 1) / kTC), (unsigned)((rows + kTR - 1) / kTR));
    uint8_t* qq = static_cast<uint8_t*>(q);
    if ((kind == Y_B200_F16 || kind == Y_B200_BF16) && rows % kTR == 0 && cols % kTC == 0 &&
        (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q) & 15u) == 0) {
        // Strips of up to 8 row tiles; enough CTAs to fill the GPU several times over.
        const int row_tiles = (int)(rows / kTR);
        int tpc = 8;
        while (tpc > 1 && (cols / kTC) * (size_t)((row_tiles + tpc - 1) / tpc) < (size_t)sm_count() * 8) tpc /= 2;
        dim3 sgrid((unsigned)(cols / kTC), (unsigned)((row_tiles + tpc - 1) / tpc));
        const uint16_t* xs = static_cast<const uint16_t*>(x);
        if (kind == Y_B200_F16)
            YB_CUDA(launch_pdl(quantize_transpose_strip_kernel<Y_B200_F16, IS_AMAX>, sgrid, kThreads, 0, st, xs, rows, cols, s, s_val, qq, scale_out, tpc));
        else
            YB_CUDA(launch_pdl(quantize_transpose_strip_kernel<Y_B200_BF16, IS_AMAX>, sgrid, kThreads, 0, st, xs, rows, cols, s, s_val, qq, scale_out, tpc));
        return check_cuda(cudaGetLastError(), "quantize_transpose_strip_kernel launch");
    }
    switch (kind) {
        case Y_B200_F16:
            YB_CUDA(launch_pdl(quantize_transpose_kernel<Y_B200_F16, IS_AMAX>, grid, kThreads, 0, st, x, rows, cols, s, s_val, qq, scale_out));
            break;
        case Y_B200_BF16:
            YB_CUDA(launch_pdl(quantize_transpose_kernel<Y_B200_BF16, IS_AMAX>, grid, kThreads, 0, st, x, rows, cols, s, s_val, qq, scale_out));
            break;
        default:
            YB_CUDA(launch_pdl(quantize_transpose_kernel<Y_B200_F32, IS_AMAX>, grid, kThreads, 0, st, x, rows, cols, s, s_val, qq, scale_out));
            break;
    }
    return check_cuda(cudaGetLastError(), "quantize_transpose_kernel launch");
}

int launch_amax(const void* x, int kind, size_t n, float* amax_out, cudaStream_t st) {
    YB_CUDA(cudaMemsetAsync(amax_out, 0, sizeof(float), st));
    int grid = grid_for(n / 8 + 1);
    unsigned int* out = reinterpret_cast<unsigned int*>(amax_out);
    switch (kind) {
        case Y_B200_F16: YB_CUDA(launch_pdl(amax_kernel<Y_B200_F16>, grid, kThreads, 0, st, x, n, out)); break;
        case Y_B200_BF16: YB_CUDA(launch_pdl(amax_kernel<Y_B200_BF16>, grid, kThreads, 0, st, x, n, out)); break;
        default: YB_CUDA(launch_pdl(amax_kernel<Y_B200_F32>, grid, kThreads, 0, st, x, n, out)); break;
    }
    return check_cuda(cudaGetLastError(), "amax_kernel launch");
}

}  // namespace

// Internal entry used by the f32 drop-in GEMM. The host's scale travels as a kernel
// argument, not through a device word: a copy from the caller's stack would leave a
// dangling host address in a captured graph.
int quantize_with_host_scale(const void* x, int kind, size_t rows, size_t cols, bool transpose,
                             float scale, void* q, cudaStream_t st) {
    if (transpose) return launch_quantize_t<false>(x, kind, rows, cols, nullptr, scale, q, nullptr, st);
    return launch_quantize<false>(x, kind, rows * cols, nullptr, scale, q, nullptr, st);
}

// Internal: requantise with the scale derived from an amax word.
int quantize_from_amax(const void* x, int kind, size_t n, const float* amax, void* q,
                       float* scale_out, cudaStream_t st) {
    return launch_quantize<true>(x, kind, n, amax, 0.0f, q, scale_out, st);
}

}  // namespace yb

using namespace yb;

extern "C" int y_b200_amax(const void* x, int x_kind, size_t n, float* amax_out, void* stream) {
    if (!x || !amax_out) return fail(Y_B200_ERR_INVALID, "y_b200_amax: null pointer");
    if (!kind_ok(x_kind)) return fail(Y_B200_ERR_INVALID, "y_b200_amax: bad element kind %d", x_kind);
    if (!aligned16(x)) return fail(Y_B200_ERR_ALIGN, "y_b200_amax: x must be 16-byte aligned");
    return launch_amax(x, x_kind, n, amax_out, static_cast<cudaStream_t>(stream));
}

extern "C" int y_b200_scale_from_amax(const float* amax, float* scale_out, void* stream) {
    if (!amax || !scale_out) return fail(Y_B200_ERR_INVALID, "y_b200_scale_from_amax: null pointer");
    YB_CUDA(launch_pdl(scale_from_amax_kernel, 1, 1, 0, static_cast<cudaStream_t>(stream), static_cast<const float*>(amax), scale_out));
    return check_cuda(cudaGetLastError(), "scale_from_amax_kernel launch");
}

extern "C" int y_b200_quantize_fp8(const void* x, int x_kind, size_t n, const float* scale, void* q,
                                   void* stream) {
    if (!x || !scale || !q) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8: null pointer");
    if (!kind_ok(x_kind)) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8: bad element kind %d", x_kind);
    if (!aligned16(x) || !aligned16(q))
        return fail(Y_B200_ERR_ALIGN, "y_b200_quantize_fp8: x and q must be 16-byte aligned");
    return launch_quantize<false>(x, x_kind, n, scale, 0.0f, q, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int y_b200_quantize_fp8_transpose(const void* x, int x_kind, size_t rows, size_t cols,
                                             const float* scale, void* q, void* stream) {
    if (!x || !scale || !q) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8_transpose: null pointer");
    if (!kind_ok(x_kind)) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8_transpose: bad element kind %d", x_kind);
    if (rows == 0 || cols == 0) return Y_B200_OK;
    if (!aligned16(x) || !aligned16(q))
        return fail(Y_B200_ERR_ALIGN, "y_b200_quantize_fp8_transpose: x and q must be 16-byte aligned");
    return launch_quantize_t<false>(x, x_kind, rows, cols, scale, 0.0f, q, nullptr,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int y_b200_quantize_fp8_dynamic(const void* x, int x_kind, size_t rows, size_t cols,
                                           int transpose, void* q, float* scale_out, void* stream) {
    if (!x || !q || !scale_out) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8_dynamic: null pointer");
    if (!kind_ok(x_kind)) return fail(Y_B200_ERR_INVALID, "y_b200_quantize_fp8_dynamic: bad element kind %d", x_kind);
    if (!aligned16(x) || !aligned16(q))
        return fail(Y_B200_ERR_ALIGN, "y_b200_quantize_fp8_dynamic: x and q must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // scale_out holds the amax while the quantise kernel runs (every CTA reads
    // it, none writes it); a last one-thread kernel turns it into the scale.
    int rc = launch_amax(x, x_kind, rows * cols, scale_out, st);
    if (rc) return rc;
    if (transpose && rows != 0 && cols != 0)
        rc = launch_quantize_t<true>(x, x_kind, rows, cols, scale_out, 0.0f, q, nullptr, st);
    else
        rc = launch_quantize<true>(x, x_kind, rows * cols, scale_out, 0.0f, q, nullptr, st);
    if (rc) return rc;
    YB_CUDA(launch_pdl(scale_from_amax_kernel, 1, 1, 0, st, static_cast<const float*>(scale_out), scale_out));
    return check_cuda(cudaGetLastError(), "scale_from_amax_kernel launch");
}

extern "C" size_t y_b200_rmsnorm_workspace_bytes(size_t rows) { return rows * sizeof(float) + 256; }

extern "C" int y_b200_rmsnorm_quantize_fp8(const void* x_f16, const void* gamma_f16, size_t rows,
                                           size_t hidden, float eps, void* q, float* scale_out,
                                           void* workspace, size_t workspace_bytes, void* stream) {
    if (!x_f16 || !gamma_f16 || !q || !scale_out)
        return fail(Y_B200_ERR_INVALID, "y_b200_rmsnorm_quantize_fp8: null pointer");
    if (hidden == 0 || hidden % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_rmsnorm_quantize_fp8: hidden=%zu must be a positive multiple of 8", hidden);
    if (!workspace || workspace_bytes < y_b200_rmsnorm_workspace_bytes(rows))
        return fail(Y_B200_ERR_WORKSPACE, "y_b200_rmsnorm_quantize_fp8: workspace needs %zu bytes",
                    y_b200_rmsnorm_workspace_bytes(rows));
    if (!aligned16(x_f16) || !aligned16(gamma_f16) || !aligned16(q) || !aligned16(workspace))
        return fail(Y_B200_ERR_ALIGN, "y_b200_rmsnorm_quantize_fp8: pointers must be 16-byte aligned");
    if (rows == 0) return Y_B200_OK;
    if (rows > 0x7fffffffu) return fail(Y_B200_ERR_SHAPE, "y_b200_rmsnorm_quantize_fp8: too many rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // workspace: [0,256) amax word, then rows floats of rstd.
    unsigned int* amax = static_cast<unsigned int*>(workspace);
    float* rstd = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
    YB_CUDA(cudaMemsetAsync(amax, 0, sizeof(unsigned int), st));
    const __half* xh = static_cast<const __half*>(x_f16);
    const __half* gh = static_cast<const __half*>(gamma_f16);
    const size_t nvec = hidden / 8;
    if (nvec <= 4 * kThreads) {
        // Four CTAs of up to 64 registers per thread fit an SM; each keeps gamma as f32.
        const unsigned smem = (unsigned)(hidden * sizeof(float));
        const size_t want = (size_t)sm_count() * 4;
        const unsigned grid = (unsigned)(rows < want ? rows : want);
        if (nvec <= kThreads)
            YB_CUDA(launch_pdl(rmsnorm_stats_kernel<1>, grid, kThreads, smem, st, xh, gh, rows, hidden, eps, rstd, amax));
        else if (nvec <= 2 * kThreads)
            YB_CUDA(launch_pdl(rmsnorm_stats_kernel<2>, grid, kThreads, smem, st, xh, gh, rows, hidden, eps, rstd, amax));
        else
            YB_CUDA(launch_pdl(rmsnorm_stats_kernel<4>, grid, kThreads, smem, st, xh, gh, rows, hidden, eps, rstd, amax));
    } else {
        YB_CUDA(launch_pdl(rmsnorm_stats_long_kernel, (unsigned)rows, kThreads, 0, st, xh, gh, hidden, eps, rstd, amax));
    }
    YB_CUDA(cudaGetLastError());
    YB_CUDA(launch_pdl(rmsnorm_quantize_kernel, (unsigned)rows, kThreads, 0, st, xh, gh, hidden, rstd,
                       reinterpret_cast<const float*>(amax), static_cast<uint8_t*>(q), scale_out));
    return check_cuda(cudaGetLastError(), "rmsnorm_quantize_kernel launch");
}

extern "C" int y_b200_rmsnorm_residual(const void* x_f16, const void* residual_f16, const void* weight_f16,
                                       size_t rows, size_t hidden, float eps, void* out_f16,
                                       void* new_residual_f16, void* stream) {
    if (!x_f16 || !residual_f16 || !weight_f16 || !out_f16 || !new_residual_f16)
        return fail(Y_B200_ERR_INVALID, "y_b200_rmsnorm_residual: null pointer");
    if (hidden == 0 || hidden % 8 != 0)
        return fail(Y_B200_ERR_SHAPE, "y_b200_rmsnorm_residual: hidden=%zu must be a positive multiple of 8", hidden);
    if (!aligned16(x_f16) || !aligned16(residual_f16) || !aligned16(weight_f16) || !aligned16(out_f16) ||
        !aligned16(new_residual_f16))
        return fail(Y_B200_ERR_ALIGN, "y_b200_rmsnorm_residual: pointers must be 16-byte aligned");
    if (rows == 0) return Y_B200_OK;
    if (rows > 0x7fffffffu) return fail(Y_B200_ERR_SHAPE, "y_b200_rmsnorm_residual: too many rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xh = static_cast<const __half*>(x_f16);
    const __half* rh = static_cast<const __half*>(residual_f16);
    const __half* wh = static_cast<const __half*>(weight_f16);
    __half* oh = static_cast<__half*>(out_f16);
    __half* nh = static_cast<__half*>(new_residual_f16);
    const size_t nvec = hidden / 8;
    const unsigned grid = (unsigned)rows;
    cudaError_t e;
    if (nvec <= kThreads) e = launch_pdl(rmsnorm_residual_kernel<1>, grid, kThreads, 0, st, xh, rh, wh, hidden, eps, oh, nh);
    else if (nvec <= 2 * kThreads) e = launch_pdl(rmsnorm_residual_kernel<2>, grid, kThreads, 0, st, xh, rh, wh, hidden, eps, oh, nh);
    else if (nvec <= 4 * kThreads) e = launch_pdl(rmsnorm_residual_kernel<4>, grid, kThreads, 0, st, xh, rh, wh, hidden, eps, oh, nh);
    else e = launch_pdl(rmsnorm_residual_kernel<0>, grid, kThreads, 0, st, xh, rh, wh, hidden, eps, oh, nh);
    return check_cuda(e, "rmsnorm_residual_kernel launch");
}

extern "C" int y_b200_rope(const void* x_f16, const int32_t* positions, void* out_f16, size_t rows, int head_dim,
                           float base, void* stream) {
    if (!x_f16 || !positions || !out_f16) return fail(Y_B200_ERR_INVALID, "y_b200_rope: null pointer");
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        return fail(Y_B200_ERR_SHAPE, "y_b200_rope: head_dim=%d must be 64, 128 or 256", head_dim);
    if (!(base > 1.0f)) return fail(Y_B200_ERR_INVALID, "y_b200_rope: base must be greater than 1");
    if (!aligned16(x_f16) || !aligned16(out_f16) || (reinterpret_cast<uintptr_t>(positions) & 3u))
        return fail(Y_B200_ERR_ALIGN, "y_b200_rope: x and out need 16-byte, positions 4-byte alignment");
    if (rows == 0) return Y_B200_OK;
    RopeTable table;
    for (int i = 0; i < head_dim / 2; ++i)
        table.inv_freq[i] = (float)pow((double)base, -2.0 * (double)i / (double)head_dim);
    for (int i = head_dim / 2; i < kRopeMaxPairs; ++i) table.inv_freq[i] = 0.0f;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half* xh = static_cast<const __half*>(x_f16);
    __half* oh = static_cast<__half*>(out_f16);
    const size_t rows_per_span = 128 / (size_t)(head_dim / 2);
    const size_t spans = (rows + rows_per_span - 1) / rows_per_span;
    const size_t spans_per_cta = (size_t)(kThreads / 32) * kRopeSpansPerWarp;
    const size_t ctas = (spans + spans_per_cta - 1) / spans_per_cta;
    if (ctas > 0x7fffffffu) return fail(Y_B200_ERR_SHAPE, "y_b200_rope: too many rows");
    const unsigned grid = (unsigned)ctas;
    cudaError_t e;
    if (head_dim == 256) e = launch_pdl(rope_kernel<256>, grid, kThreads, 0, st, xh, positions, oh, rows, table);
    else if (head_dim == 128) e = launch_pdl(rope_kernel<128>, grid, kThreads, 0, st, xh, positions, oh, rows, table);
    else e = launch_pdl(rope_kernel<64>, grid, kThreads, 0, st, xh, positions, oh, rows, table);
    return check_cuda(e, "rope_kernel launch");
}

extern "C" int y_b200_fill_random_f16(void* out_f16, size_t n, uint64_t index0, uint64_t seed,
                                      void* stream) {
    if (!out_f16) return fail(Y_B200_ERR_INVALID, "y_b200_fill_random_f16: null pointer");
    if (n == 0) return Y_B200_OK;
    fill_random_f16_kernel<<<grid_for(n), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t*>(out_f16), n, index0, seed);
    return check_cuda(cudaGetLastError(), "fill_random_f16_kernel launch");
}
