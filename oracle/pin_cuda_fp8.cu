// Host-side e4m3 conversions from NVIDIA's cuda_fp8.h, exported so the tests
// can pin the oracle's encoder/decoder against an independent implementation.
// TEST INFRASTRUCTURE ONLY; contains no device code.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

extern "C" unsigned char pin_nv_e4m3_encode(float x) {
    return (unsigned char)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

extern "C" float pin_nv_e4m3_decode(unsigned char code) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
    return __half2float(__half(h));
}
