"""Host launch API: Python face of the C-ABI mirror of the reference's
`CudaContext` / `DeviceBuffer` / `KernelModule` (src/cuda_runtime.rs:243-630),
plus the `c_api.rs` helpers. Same names, argument meaning and error behaviour:
`CudaContext.new()` returns None when there is no device; range errors and
launch errors raise with the library's message; nothing is computed on the CPU.
"""
from __future__ import annotations

import ctypes as C
import json

from . import _lib
from ._lib import ARG_F32, ARG_I32, ARG_PTR, Arg, LaunchInfo, YB200Error, lib, take_string

CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE = 38  # src/empirical_autotune.rs:396


class DeviceBuffer:
    def __init__(self, handle):
        self._h = handle

    def device_ptr(self) -> int:
        return lib.y_buf_device_ptr(self._h)

    def len_bytes(self) -> int:
        return lib.y_buf_len_bytes(self._h)

    def free(self) -> None:
        if self._h:
            lib.y_buf_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:  # at interpreter exit the library binding may be gone already
            pass


class KernelModule:
    def __init__(self, handle):
        self._h = handle

    def set_max_dynamic_smem(self, nbytes: int) -> None:
        _lib.check(lib.y_kernel_set_max_dynamic_smem(self._h, nbytes))

    def launch_info(self) -> LaunchInfo:
        info = LaunchInfo()
        _lib.check(lib.y_kernel_launch_info(self._h, C.byref(info)))
        return info

    def free(self) -> None:
        if self._h:
            lib.y_kernel_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:  # at interpreter exit the library binding may be gone already
            pass


def _args(values) -> C.Array:
    """ints that are device pointers -> PTR, python floats -> F32, ('i32', v) -> I32."""
    arr = (Arg * len(values))()
    for i, v in enumerate(values):
        if isinstance(v, tuple) and v[0] == "i32":
            arr[i].kind, arr[i].v.i32 = ARG_I32, int(v[1])
        elif isinstance(v, float):
            arr[i].kind, arr[i].v.f32 = ARG_F32, v
        elif isinstance(v, DeviceBuffer):
            arr[i].kind, arr[i].v.ptr = ARG_PTR, v.device_ptr()
        else:
            arr[i].kind, arr[i].v.ptr = ARG_PTR, int(v)
    return arr


def _dim3(t):
    if t is None:
        return None
    return (C.c_uint * 3)(*t)


class CudaContext:
    def __init__(self, handle):
        self._h = handle

    @staticmethod
    def new() -> "CudaContext | None":
        h = lib.y_ctx_create()
        return CudaContext(h) if h else None

    def device_name(self) -> str:
        return lib.y_ctx_device_name(self._h).decode()

    def device_attribute(self, attrib: int) -> int | None:
        v = C.c_int()
        return v.value if lib.y_ctx_device_attribute(self._h, attrib, C.byref(v)) == 0 else None

    def alloc(self, len_bytes: int) -> DeviceBuffer:
        h = lib.y_ctx_alloc(self._h, len_bytes)
        if not h:
            raise YB200Error(_lib.ERR_CUDA, _lib.last_error())
        return DeviceBuffer(h)

    def memset_u8(self, buf: DeviceBuffer, value: int) -> None:
        _lib.check(lib.y_ctx_memset_u8(self._h, buf._h, value))

    def memcpy_htod_at(self, buf: DeviceBuffer, offset_bytes: int, src: bytes) -> None:
        _lib.check(lib.y_ctx_memcpy_htod_at(self._h, buf._h, offset_bytes, src, len(src)))

    def memcpy_dtoh_at(self, nbytes: int, buf: DeviceBuffer, offset_bytes: int) -> bytes:
        dst = C.create_string_buffer(nbytes)
        _lib.check(lib.y_ctx_memcpy_dtoh_at(self._h, dst, nbytes, buf._h, offset_bytes))
        return dst.raw

    def memcpy_dtod(self, dst: DeviceBuffer, src: DeviceBuffer) -> None:
        _lib.check(lib.y_ctx_memcpy_dtod(self._h, dst._h, src._h))

    def mem_info(self):
        f, t = C.c_size_t(), C.c_size_t()
        return (f.value, t.value) if lib.y_ctx_mem_info(self._h, C.byref(f), C.byref(t)) == 0 else None

    def synchronize(self) -> None:
        _lib.check(lib.y_ctx_synchronize(self._h))

    def load_module(self, image: str | None, entry: str) -> KernelModule:
        """`image` is the descriptor text from compile_to_ptx, or None for the
        runtime-shape entries (`y_fp8_gemm`, `y_int4_decode_gemm`)."""
        h = lib.y_ctx_load_module(self._h, image.encode() if image is not None else None, entry.encode())
        if not h:
            raise YB200Error(_lib.ERR_UNSUPPORTED, _lib.last_error())
        return KernelModule(h)

    def launch(self, kernel: KernelModule, grid, block, shared_bytes: int, args) -> None:
        arr = _args(args)
        _lib.check(lib.y_ctx_launch(self._h, kernel._h, _dim3(grid), _dim3(block), shared_bytes, arr, len(args)))

    def time_launches(self, kernel: KernelModule, grid, block, shared_bytes: int, arg_sets, iters: int) -> float:
        """Mean microseconds per launch over `iters` back-to-back launches; launch i
        uses arg_sets[i % len(arg_sets)]."""
        if iters == 0:
            raise YB200Error(_lib.ERR_INVALID, "time_launches called with iters = 0")
        if not arg_sets:
            raise YB200Error(_lib.ERR_INVALID, "time_launches called with no argument sets")
        nargs = len(arg_sets[0])
        flat = _args([v for s in arg_sets for v in s])
        out = C.c_double()
        _lib.check(lib.y_ctx_time_launches(self._h, kernel._h, _dim3(grid), _dim3(block), shared_bytes, flat,
                                           len(arg_sets), nargs, iters, C.byref(out)))
        return out.value

    def close(self) -> None:
        if self._h:
            lib.y_ctx_destroy(self._h)
            self._h = None


# ---- c_api.rs -------------------------------------------------------------------
def compile_to_ptx(source: str, target_sm: str = "sm_100a") -> str:
    err = C.c_void_p()
    out = lib.y_compile_to_ptx(source.encode() if source is not None else None,
                               target_sm.encode() if target_sm is not None else None, C.byref(err))
    msg = take_string(err.value)
    text = take_string(out)
    if text is None:
        raise ValueError(msg or "compile failed")
    return text


def autotune_search_space(m: int, n: int, k: int, is_fp8: bool):
    return json.loads(take_string(lib.y_autotune_search_space_json(m, n, k, bool(is_fp8))))


def autotune_select_config(m: int, n: int, k: int, is_fp8: bool):
    return json.loads(take_string(lib.y_autotune_select_config_json(m, n, k, bool(is_fp8))))


def block_cdiv(a: int, b: int) -> int:
    return lib.y_block_cdiv(a, b)
