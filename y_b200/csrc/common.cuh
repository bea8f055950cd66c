// Shared device helpers for the sm_100a kernels: error plumbing, bounded
// mbarrier waits, TMA and tcgen05 PTX wrappers, small conversion helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/y_b200.h"

namespace yb {

// ---- host-side error plumbing ---------------------------------------------
// Every extern "C" entry returns 0 or a negative Y_B200_ERR_* code and leaves
// a message retrievable through y_b200_last_error() (thread local).
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

#define YB_CUDA(call)                                         \
    do {                                                      \
        int _rc = ::yb::check_cuda((call), #call);            \
        if (_rc != 0) return _rc;                             \
    } while (0)

int sm_count();  // multiprocessors of the current device (cached per device)

// ---- device status word ------------------------------------------------------
// Kernels that wait on mbarriers never spin without a limit: a wait that runs
// out records where it gave up in this word and the kernel unwinds. The host
// reads it with y_b200_device_status().
struct DeviceStatus {
    unsigned int code;   // 0 = ok, else Y_B200_DEV_* reason
    unsigned int where;  // role / barrier index that gave up
    unsigned int block;  // blockIdx.x of the reporting CTA
    unsigned int extra;
};
DeviceStatus* device_status_ptr();  // per-device, allocated on first use
DeviceStatus* static_entry_status_ptr();  // status word of the allocation-free GEMM entry; null until it has run

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Cycle budget of one wait (about two seconds at 2 GHz). Far above any legal
// wait inside these kernels, far below the watchdog of a shared machine.
constexpr long long kWaitCycles = 4000000000LL;

// Bounded wait. Returns false when the budget ran out or when another role of
// this CTA already raised `abort_flag` (a word in shared memory).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag, long long budget = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ffu) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > budget) return false;
        }
    }
    return true;
}

__device__ __forceinline__ void report_timeout(DeviceStatus* st, volatile uint32_t* abort_flag,
                                               unsigned int where, unsigned int extra) {
    *abort_flag = 1u;
    if (st != nullptr && atomicCAS(&st->code, 0u, (unsigned int)Y_B200_DEV_WAIT_TIMEOUT) == 0u) {
        st->where = where;
        st->block = blockIdx.x;
        st->extra = extra;
    }
}

// ---- TMA ----------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load into this CTA's shared memory; completion is counted in bytes
// on `bar`. x is the innermost coordinate (elements); x * elemsize must be a
// multiple of 16. No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}


// ---- tcgen05 / TMEM --------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// The mbarrier gets one arrival once every tcgen05.mma this thread issued so
// far has finished (implies fence::before_thread_sync).
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same for 16-bit operands (f16 x f16 -> f32): K = 16 elements per instruction, i.e. the
// same 32 bytes of K as kind::f8f6f4, so operand tiles and descriptors are laid out alike.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---- CTA pairs (cta_group::2) --------------------------------------------------------
// Two CTAs of a cluster share one MMA: the even-ranked CTA issues it, each CTA holds its
// half of both operands in its own shared memory and its half of the accumulator rows
// in its own tensor memory.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the cluster's CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this offset in every CTA of `cta_mask`, once all MMAs
// issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}
// Tiled 2-D load into THIS CTA's shared memory whose completion bytes are counted on
// the barrier at the same offset in the pair's even-ranked CTA (bit 24 of a shared
// cluster address selects the odd CTA of a pair).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar,
                                                 int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar & 0xFEFFFFFFu), "r"(x), "r"(y)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives
// lane (base_lane + t), registers r[0..31] are columns col .. col+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are one
// 128-byte swizzle span wide (the layout a SWIZZLE_128B tensor-map box lands
// in): 8-row groups 1024 bytes apart, descriptor version 1, 128-byte swizzle.
// The tile base must be 1024-byte aligned; advancing along K inside the span
// adds the byte offset to the start address.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);  // start address, 16-byte units
    d |= (uint64_t)0 << 16;                        // leading byte offset: unused here
    d |= (uint64_t)(1024u >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f8f6f4 / kind::f16, dense, f32 accumulate,
// both operands K-major. a_fmt/b_fmt: f8f6f4 0 = e4m3, 1 = e5m2; f16 kind
// 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                  uint32_t b_fmt) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- small conversion helpers -------------------------------------------------
// Two f32 -> two e4m3 codes (round to nearest even, saturate to +-448):
// `lo` lands in bits 0..7, `hi` in bits 8..15.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
    return cvt_e4m3x2(a, b) | (cvt_e4m3x2(c, d) << 16);
}

// scale = max(amax / 448, 1e-12), inv = 1 / scale; both correctly rounded.
__device__ __forceinline__ float scale_from_amax(float amax) {
    return fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
}
__device__ __forceinline__ float inv_scale(float scale) { return __fdiv_rn(1.0f, scale); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
    return __reduce_max_sync(0xffffffffu, v);
}

#endif  // __CUDACC__

// ---- programmatic dependent launch ------------------------------------------------
// A kernel launched with launch_pdl may start while the kernel before it in the
// stream is still running (once every CTA of that kernel has called
// pdl_launch_dependents or exited). It must call pdl_wait before it touches anything
// an earlier kernel may write or still read; after pdl_wait the earlier kernel has
// completed and its writes are visible. Both calls are no-ops in a kernel that was
// launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace yb
