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
    DeviceStatus h;
    YB_CUDA(cudaMemcpyAsync(&h, dptr, sizeof h, cudaMemcpyDeviceToHost, st));
    YB_CUDA(cudaStreamSynchronize(st));
    if (h.code == 0) return 0;
    YB_CUDA(cudaMemsetAsync(dptr, 0, sizeof h, st));
    YB_CUDA(cudaStreamSynchronize(st));
    return fail(Y_B200_ERR_DEVICE,
                "device wait ran out: code %u at role/barrier 0x%x, CTA %u, detail %u", h.code,
                h.where, h.block, h.extra);
}
