"""ctypes binding of liby_b200.so (the C ABI declared in include/y_b200.h).

The library is the product; this module only loads it and declares the
argument types. There is no fallback: if the shared library is missing the
import fails with instructions to build it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liby_b200.so")

OK = 0
ERR_INVALID, ERR_SHAPE, ERR_ALIGN, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE, ERR_UNSUPPORTED = (
    -1, -2, -3, -4, -5, -6, -7)
F32, F16, BF16, E4M3 = 0, 1, 2, 3
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_SWIGLU, EPI_BIAS_GELU, EPI_BIAS_SILU = 0, 1, 2, 3, 4, 5


class YB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"liby_b200 error {code}: {message}")
        self.code = code
        self.message = message


class GemmFp8Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("bt", C.c_void_p), ("c", C.c_void_p),
        ("m", C.c_int), ("n", C.c_int), ("k", C.c_int),
        ("scale_a", C.c_float), ("scale_b", C.c_float),
        ("scale_a_dev", C.c_void_p), ("scale_b_dev", C.c_void_p),
        ("bias", C.c_void_p), ("bias_kind", C.c_int),
        ("epilogue", C.c_int), ("out_kind", C.c_int),
        ("amax_out", C.c_void_p),
        ("cta_n", C.c_int), ("max_ctas", C.c_int), ("cta_m", C.c_int),
        ("c_replicas", C.c_void_p * 7), ("c_replica_count", C.c_int),
    ]


class GemmF16Args(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("bt", C.c_void_p), ("c", C.c_void_p),
        ("m", C.c_int), ("n", C.c_int), ("k", C.c_int),
        ("alpha", C.c_float),
        ("bias", C.c_void_p), ("bias_kind", C.c_int),
        ("epilogue", C.c_int), ("out_kind", C.c_int),
        ("cta_n", C.c_int), ("max_ctas", C.c_int), ("cta_m", C.c_int),
    ]


class LaunchInfo(C.Structure):
    _fields_ = [
        ("grid", C.c_uint * 3), ("block", C.c_uint * 3), ("cluster", C.c_uint * 3),
        ("dyn_smem_bytes", C.c_uint), ("workspace_bytes", C.c_size_t),
        ("cta_m", C.c_int), ("cta_n", C.c_int), ("cta_k", C.c_int), ("stages", C.c_int),
        ("fused_epilogues", C.c_int),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python y_b200/build.py` (needs nvcc); "
            "this package has no CPU or PyTorch fallback")
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _sz, _i, _f, _u32, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint32, C.c_uint64

# name -> (restype, argtypes); every symbol include/y_b200.h declares.
SIGNATURES = {
    "y_b200_last_error": (C.c_char_p, []),
    "y_b200_version": (C.c_char_p, []),
    "y_b200_device_status": (_i, [_vp]),
    "y_b200_selftest_bounded_wait": (_i, [_u64, _vp]),
    "y_b200_amax": (_i, [_vp, _i, _sz, _vp, _vp]),
    "y_b200_scale_from_amax": (_i, [_vp, _vp, _vp]),
    "y_b200_quantize_fp8": (_i, [_vp, _i, _sz, _vp, _vp, _vp]),
    "y_b200_quantize_fp8_transpose": (_i, [_vp, _i, _sz, _sz, _vp, _vp, _vp]),
    "y_b200_quantize_fp8_dynamic": (_i, [_vp, _i, _sz, _sz, _i, _vp, _vp, _vp]),
    "y_b200_rmsnorm_workspace_bytes": (_sz, [_sz]),
    "y_b200_rmsnorm_quantize_fp8": (_i, [_vp, _vp, _sz, _sz, _f, _vp, _vp, _vp, _sz, _vp]),
    "y_b200_gemm_fp8": (_i, [C.POINTER(GemmFp8Args), _vp]),
    "y_b200_gemm_fp8_launch_info": (_i, [_i, _i, _i, _i, C.POINTER(LaunchInfo)]),
    "y_b200_gemm_fp8_f32_workspace_bytes": (_sz, [_i, _i, _i]),
    "y_b200_gemm_fp8_f32": (_i, [_vp, _vp, _f, _f, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "y_b200_gemm_fp8_f32_static": (_i, [_vp, _vp, _f, _f, _vp, _i, _i, _i, _vp]),
    "y_b200_gemm_f16": (_i, [C.POINTER(GemmF16Args), _vp]),
    "y_b200_gemm_f16_rowmajor_workspace_bytes": (_sz, [_i, _i]),
    "y_b200_gemm_f16_rowmajor": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _i, _vp, _sz, _vp]),
    "y_b200_gemm_f16_swiglu_workspace_bytes": (_sz, [_i, _i]),
    "y_b200_gemm_f16_swiglu": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "y_b200_gemm_f16_decode": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp]),
    "y_b200_gemm_f16_splitk_workspace": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "y_b200_splitk_reduction": (_i, [_vp, _vp, _sz, _i, _i, _i, _vp]),
    "y_b200_swiglu_workspace_bytes": (_sz, [_i, _i]),
    "y_b200_gemm_fp8_swiglu_requant": (_i, [C.POINTER(GemmFp8Args), _vp, _vp, _vp, _sz, _vp]),
    "y_b200_mlp_workspace_bytes": (_sz, [_i, _i]),
    "y_b200_mlp_swiglu_fp8": (_i, [_vp, C.c_float, _vp, _vp, C.c_float, _vp, C.c_float, _vp, _i, _i, _i, _i, _i,
                               _vp, _sz, _vp]),
    "y_b200_int4_quantize": (_i, [_vp, _sz, _sz, _vp, _vp, _vp]),
    "y_b200_int4_stream_bytes": (_sz, [_sz, _sz]),
    "y_b200_int4_repack": (_i, [_vp, _vp, _sz, _sz, _vp, _vp]),
    "y_b200_gemm_int4_decode": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp]),
    "y_b200_probe_chain_read": (_i, [C.POINTER(_vp), _i, _sz, _i, _i, _vp, C.POINTER(C.c_float), _vp]),
    "y_b200_rmsnorm_residual": (_i, [_vp, _vp, _vp, _sz, _sz, C.c_float, _vp, _vp, _vp]),
    "y_b200_rope": (_i, [_vp, _vp, _vp, _sz, _i, C.c_float, _vp]),
    "y_b200_paged_decode_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "y_b200_paged_decode_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "y_b200_peer_alloc": (_i, [_sz, C.POINTER(_vp)]),
    "y_b200_peer_free": (_i, [_vp]),
    "y_b200_peer_export": (_i, [_vp, C.c_char_p]),
    "y_b200_peer_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "y_b200_peer_close": (_i, [_vp]),
    "y_b200_peer_read": (_i, [_vp, _vp, _sz]),
    "y_b200_fill_random_f16": (_i, [_vp, _sz, _u64, _u64, _vp]),
    "y_compile_to_ptx": (_vp, [C.c_char_p, C.c_char_p, C.POINTER(_vp)]),
    "y_autotune_search_space_json": (_vp, [_u32, _u32, _u32, C.c_bool]),
    "y_autotune_select_config_json": (_vp, [_u32, _u32, _u32, C.c_bool]),
    "y_interpret_kernel": (C.c_int32, [C.c_char_p, C.POINTER(_vp)]),
    "y_block_cdiv": (_u32, [_u32, _u32]),
    "y_free_string": (None, [_vp]),
}



class Arg(C.Structure):
    class _V(C.Union):
        _fields_ = [("ptr", C.c_uint64), ("f32", C.c_float), ("i32", C.c_int32)]

    _fields_ = [("kind", C.c_int), ("v", _V)]


ARG_PTR, ARG_F32, ARG_I32 = 0, 1, 2
_u3 = C.POINTER(C.c_uint)
_u32p = C.POINTER(C.c_uint32)

# include/y_b200_runtime.h
SIGNATURES.update({
    "y_ctx_create": (_vp, []),
    "y_ctx_destroy": (None, [_vp]),
    "y_ctx_device_name": (C.c_char_p, [_vp]),
    "y_ctx_device_attribute": (_i, [_vp, _i, C.POINTER(C.c_int)]),
    "y_ctx_mem_info": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "y_ctx_synchronize": (_i, [_vp]),
    "y_ctx_alloc": (_vp, [_vp, _sz]),
    "y_buf_free": (None, [_vp]),
    "y_buf_device_ptr": (_u64, [_vp]),
    "y_buf_len_bytes": (_sz, [_vp]),
    "y_ctx_memset_u8": (_i, [_vp, _vp, C.c_uint8]),
    "y_ctx_memcpy_htod_at": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "y_ctx_memcpy_dtoh_at": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "y_ctx_memcpy_dtod": (_i, [_vp, _vp, _vp]),
    "y_ctx_load_module": (_vp, [_vp, C.c_char_p, C.c_char_p]),
    "y_kernel_free": (None, [_vp]),
    "y_kernel_set_max_dynamic_smem": (_i, [_vp, C.c_uint]),
    "y_kernel_launch_info": (_i, [_vp, C.POINTER(LaunchInfo)]),
    "y_ctx_launch": (_i, [_vp, _vp, _u3, _u3, C.c_uint, C.POINTER(Arg), _i]),
    "y_ctx_time_launches": (_i, [_vp, _vp, _u3, _u3, C.c_uint, C.POINTER(Arg), _i, _i, C.c_uint,
                                 C.POINTER(C.c_double)]),
    "y_colpar_create": (_vp, [_vp, _vp, _vp, C.c_float, _i, _i, _i, _i]),
    "y_colpar_destroy": (None, [_vp]),
    "y_colpar_forward": (_i, [_vp, _vp, _vp, _i, _vp]),
    "y_colpar_submit_host": (_i, [_vp, _vp, _vp, _vp]),
    "y_colpar_drain": (_i, [_vp, _vp]),
    "y_colpar_synchronize": (_i, [_vp]),
    "y_colpar_host_bytes_per_step": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "y_autotune_persist_key": (_vp, [_u32, _u32, _u32, _i, C.c_char_p]),
    "y_autotune_parse_persisted": (_i, [C.c_char_p, _u32p]),
    "y_autotune_set_profile_path": (None, [C.c_char_p]),
    "y_autotune_store": (_i, [_u32, _u32, _u32, _i, C.c_char_p, _u32p]),
    "y_autotune_lookup": (_i, [_u32, _u32, _u32, _i, C.c_char_p, _u32p, _u32p]),
    "y_autotune_set_mode": (None, [_i]),
    "y_autotune_clear_cache": (None, []),
    "y_autotune_is_launchable": (_i, [_u32p, _u32, _i]),
    "y_autotune_score": (C.c_double, [_u32p, _u32, _u32, _u32, _i]),
    "y_autotune_tied": (_i, [C.c_double, C.c_double, C.c_double, C.c_double]),
    "y_autotune_select_winner": (_sz, [C.POINTER(C.c_double), _sz]),
    "y_autotune_plan_weight_replicas": (_sz, [_sz, _sz, _sz, _sz, _sz]),
    "y_autotune_measure_fp8_json": (_vp, [_u32, _u32, _u32]),
    "y_parse_launch_config": (_i, [C.c_char_p, _u32, _u32, _u32p]),
})

for _name, (_res, _args) in SIGNATURES.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError:
        raise ImportError(f"{LIB_PATH} is older than this package (no symbol {_name}): rebuild it with "
                          "`python y_b200/build.py`") from None
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.y_b200_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise YB200Error(rc, last_error())


def take_string(ptr) -> str | None:
    """Copies a library-owned C string and frees it with y_free_string."""
    if not ptr:
        return None
    s = C.string_at(ptr).decode("utf-8", "replace")
    lib.y_free_string(ptr)
    return s
