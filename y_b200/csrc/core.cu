// Library-wide plumbing: thread-local error text, per-device cached properties
// and the device status word that bounded waits report into.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace yb {
namespace {

thread_local char g_error[1024] = "";

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
int g_sm_count[kMaxDevices] = {};
DeviceStatus* g_status[kMaxDevices] = {};

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    return (dev >= 0 && dev < kMaxDevices) ? dev : -1;
}

}  // namespace

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    return fail(Y_B200_ERR_CUDA, "%s failed: %s (cudaError %d)", what, cudaGetErrorString(e), (int)e);
}

int sm_count() {
    const int dev = current_device();
    if (dev < 0) return 148;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 148;  // B200
        }
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

DeviceStatus* device_status_ptr() {
    const int dev = current_device();
    if (dev < 0) return nullptr;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status[dev] == nullptr) {
        void* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess || cudaMemset(p, 0, 256) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_status[dev] = static_cast<DeviceStatus*>(p);
    }
    return g_status[dev];
}

}  // namespace yb

using namespace yb;

extern "C" const char* y_b200_last_error(void) { return g_error; }

extern "C" const char* y_b200_version(void) { return "y_b200 0.1 (sm_100a)"; }

extern "C" int y_b200_device_status(void* stream) {
    DeviceStatus* dptr = device_status_ptr();
    if (!dptr) return fail(Y_B200_ERR_CUDA, "y_b200_device_status: no CUDA device");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Two words: the one every workspace-taking entry reports into, and the one inside the
    // allocation-free entry's built-in scratch (present once that entry has run here).
    DeviceStatus* words[2] = {dptr, static_entry_status_ptr()};
    DeviceStatus h[2] = {};
    for (int i = 0; i < 2; ++i)
        if (words[i]) YB_CUDA(cudaMemcpyAsync(&h[i], words[i], sizeof h[i], cudaMemcpyDeviceToHost, st));
    YB_CUDA(cudaStreamSynchronize(st));
    if (h[0].code == 0 && h[1].code == 0) return 0;
    for (int i = 0; i < 2; ++i)
        if (h[i].code != 0) YB_CUDA(cudaMemsetAsync(words[i], 0, sizeof h[i], st));
    YB_CUDA(cudaStreamSynchronize(st));
    const int w = h[0].code != 0 ? 0 : 1;
    return fail(Y_B200_ERR_DEVICE,
                "device wait ran out%s: code %u at role/barrier 0x%x, CTA %u, detail %u",
                w == 1 ? " in y_b200_gemm_fp8_f32_static" : "", h[w].code, h[w].where, h[w].block, h[w].extra);
}

// ---- peer memory (CUDA IPC) -----------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) == Y_B200_PEER_HANDLE_BYTES, "the exported handle is a cudaIpcMemHandle_t");

extern "C" int y_b200_peer_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return yb::fail(Y_B200_ERR_INVALID, "y_b200_peer_alloc: null output or zero size");
    *ptr = nullptr;
    return yb::check_cuda(cudaMalloc(ptr, bytes), "cudaMalloc(peer buffer)");
}

extern "C" int y_b200_peer_free(void* ptr) {
    if (!ptr) return 0;
    return yb::check_cuda(cudaFree(ptr), "cudaFree(peer buffer)");
}

extern "C" int y_b200_peer_export(const void* ptr, unsigned char handle[Y_B200_PEER_HANDLE_BYTES]) {
    if (!ptr || !handle) return yb::fail(Y_B200_ERR_INVALID, "y_b200_peer_export: null argument");
    cudaIpcMemHandle_t h;
    int rc = yb::check_cuda(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)), "cudaIpcGetMemHandle");
    if (rc) return rc;
    memcpy(handle, &h, sizeof h);
    return 0;
}

extern "C" int y_b200_peer_open(const unsigned char handle[Y_B200_PEER_HANDLE_BYTES], void** peer_ptr) {
    if (!handle || !peer_ptr) return yb::fail(Y_B200_ERR_INVALID, "y_b200_peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    *peer_ptr = nullptr;
    return yb::check_cuda(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

extern "C" int y_b200_peer_close(void* peer_ptr) {
    if (!peer_ptr) return 0;
    return yb::check_cuda(cudaIpcCloseMemHandle(peer_ptr), "cudaIpcCloseMemHandle");
}

extern "C" int y_b200_peer_read(void* host_dst, const void* device_src, size_t bytes) {
    if (!host_dst || !device_src) return yb::fail(Y_B200_ERR_INVALID, "y_b200_peer_read: null pointer");
    return yb::check_cuda(cudaMemcpy(host_dst, device_src, bytes, cudaMemcpyDeviceToHost), "cudaMemcpy(device to host)");
}

// ---- self-test of the bounded-wait path ---------------------------------------------------------
// One CTA, two warps. Warp 0 waits on an mbarrier that nothing will ever complete, with a
// budget of `cycles`; when the budget runs out it records the timeout exactly as the GEMM's
// roles do. Warp 1 plays a second role of the CTA: it watches the abort flag (bounded too)
// and leaves when it is raised. The kernel always returns; the context stays usable.
namespace yb {
namespace {
__global__ void bounded_wait_selftest_kernel(DeviceStatus* status, long long cycles) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!mbar_wait(smem_u32(&bar), 0u, abort_flag, cycles)) report_timeout(status, abort_flag, 0x7e57u, 0u);
    } else if (threadIdx.x == 32) {
        const long long t0 = clock64();
        while (*abort_flag == 0 && clock64() - t0 < 4 * cycles + 1000000) {
        }
    }
}
}  // namespace
}  // namespace yb

extern "C" int y_b200_selftest_bounded_wait(unsigned long long cycles, void* stream) {
    if (cycles == 0 || cycles > 2000000000ull)
        return yb::fail(Y_B200_ERR_INVALID, "y_b200_selftest_bounded_wait: cycles must be in 1..2e9 (about one second)");
    yb::DeviceStatus* st = yb::device_status_ptr();
    if (!st) return yb::fail(Y_B200_ERR_CUDA, "y_b200_selftest_bounded_wait: no CUDA device");
    yb::bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(st, (long long)cycles);
    return yb::check_cuda(cudaGetLastError(), "bounded_wait_selftest_kernel launch");
}
