"""ctypes front end of the CPU oracle (`liboracle.so`, built by `oracle/Makefile`).

TEST INFRASTRUCTURE ONLY. Only the tests, the smoke check and the CPU-baseline
leg of the benchmark import this package; the shipped library never does.
Arrays are numpy: f16 and bf16 tensors travel as `uint16` bit patterns, e4m3
tensors as `uint8` codes.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_SWIGLU, EPI_BIAS_GELU, EPI_BIAS_SILU = 0, 1, 2, 3, 4, 5
OUT_F32, OUT_F16, OUT_BF16 = 0, 1, 2
BIAS_NONE, BIAS_F16, BIAS_F32 = 0, 1, 2

SEED_A = 0xA5A5_1234_5678_9ABC  # src/empirical_autotune.rs:106
SEED_B = 0xB1B1_0FED_CBA9_8765  # src/empirical_autotune.rs:107


def build(force: bool = False) -> None:
    """Compile the oracle libraries if they are missing (needs gcc and nvcc)."""
    need = force or not all(
        os.path.exists(os.path.join(_HERE, n)) for n in ("liboracle.so", "libpin_fp8.so")
    )
    if need:
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True,
                       stdout=subprocess.DEVNULL)


def _stale(name: str, sources) -> bool:
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    return any(os.path.getmtime(os.path.join(_HERE, s)) > built for s in sources
               if os.path.exists(os.path.join(_HERE, s)))


def _load(name: str, sources=()) -> C.CDLL:
    if _stale(name, sources):  # missing, or older than its sources: make rebuilds what changed
        subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
    return C.CDLL(os.path.join(_HERE, name))


_lib = _load("liboracle.so", ("oracle.c", "oracle.h"))

_u8p = C.POINTER(C.c_uint8)
_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_f32p = C.POINTER(C.c_float)


def _sig(name, restype, *argtypes):
    fn = getattr(_lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_f16_to_f32 = _sig("orc_f16_bits_to_f32", C.c_float, C.c_uint16)
_f32_to_f16 = _sig("orc_f32_to_f16_bits", C.c_uint16, C.c_float)
_f32_to_bf16 = _sig("orc_f32_to_bf16_bits", C.c_uint16, C.c_float)
_e4m3_enc = _sig("orc_e4m3_encode", C.c_uint8, C.c_float)
_e4m3_dec = _sig("orc_e4m3_decode", C.c_float, C.c_uint8)
_splitmix = _sig("orc_splitmix64", C.c_uint64, C.c_uint64, C.c_uint64)
_rand_f16 = _sig("orc_random_f16_bits", C.c_uint16, C.c_uint64, C.c_uint64)
_fill_rand = _sig("orc_fill_random_f16", None, _u16p, C.c_size_t, C.c_uint64)
_fill_norm = _sig("orc_fill_normal_f16", None, _u16p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_float)
_fill_unif = _sig("orc_fill_uniform_f16", None, _u16p, C.c_size_t, C.c_uint64, C.c_uint64,
                  C.c_float, C.c_float)
_cdiv = _sig("orc_block_cdiv", C.c_uint32, C.c_uint32, C.c_uint32)
_swz = _sig("orc_grid_swizzle", None, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
            C.POINTER(C.c_uint32), C.POINTER(C.c_uint32))
_amax16 = _sig("orc_amax_f16", C.c_float, _u16p, C.c_size_t)
_amax32 = _sig("orc_amax_f32", C.c_float, _f32p, C.c_size_t)
_scale = _sig("orc_scale_from_amax", C.c_float, C.c_float)
_q16 = _sig("orc_quantize_fp8_f16", None, _u16p, C.c_size_t, C.c_float, _u8p)
_q32 = _sig("orc_quantize_fp8_f32", None, _f32p, C.c_size_t, C.c_float, _u8p)
_q16t = _sig("orc_quantize_fp8_f16_transpose", None, _u16p, C.c_size_t, C.c_size_t, C.c_float, _u8p)
_rms = _sig("orc_rmsnorm_f16", C.c_float, _u16p, _u16p, C.c_size_t, C.c_size_t, C.c_float, _f32p, _f32p)
_rmsres = _sig("orc_rmsnorm_residual_f16", None, _u16p, _u16p, _u16p, C.c_size_t, C.c_size_t, C.c_float, _u16p, _u16p)
_rope = _sig("orc_rope_f16", None, _u16p, C.POINTER(C.c_int32), C.c_size_t, C.c_int, C.c_float, _u16p)
_i32p = C.POINTER(C.c_int32)
_attn = _sig("orc_paged_decode_attention", None, _u16p, _u16p, _u16p, _i32p, _i32p, C.c_int, C.c_int, C.c_int,
             C.c_int, C.c_int, C.c_int, _u16p)
_rmsq = _sig("orc_rmsnorm_quantize_fp8", None, _u16p, _u16p, C.c_size_t, C.c_size_t, C.c_float,
             _u8p, _f32p)
_gemm8 = _sig("orc_gemm_fp8", None, _u8p, _u8p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float,
              C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t)
_dec8 = _sig("orc_decode_e4m3", None, _u8p, C.c_size_t, _f32p)
_gemm8d = _sig("orc_gemm_fp8_decoded", None, _u8p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float,
               C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t)
_gemm16 = _sig("orc_gemm_f16", None, _u16p, _u16p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p,
               C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t)
_requant = _sig("orc_requant_bf16_fp8", None, _u16p, C.c_size_t, _u8p, _f32p)
_i4q = _sig("orc_int4_quantize", None, _u16p, C.c_size_t, C.c_size_t, C.c_size_t, _u32p, _u16p)
_i4bytes = _sig("orc_int4_stream_bytes", C.c_size_t, C.c_size_t, C.c_size_t)
_i4pack = _sig("orc_int4_repack", None, _u32p, _u16p, C.c_size_t, C.c_size_t, _u8p)
_i4gemm = _sig("orc_gemm_int4_decode", None, _u16p, _u32p, _u16p, C.c_size_t, C.c_size_t,
               C.c_size_t, C.c_size_t, _u16p)
num_threads = _sig("orc_num_threads", C.c_int)


def _p(a: np.ndarray, ty):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ty)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---- scalars ---------------------------------------------------------------
def f16_bits_to_f32(h: int) -> float:
    return float(_f16_to_f32(h))


def f32_to_f16_bits(x: float) -> int:
    return int(_f32_to_f16(x))


def f32_to_bf16_bits(x: float) -> int:
    return int(_f32_to_bf16(x))


def e4m3_encode(x: float) -> int:
    return int(_e4m3_enc(x))


def e4m3_decode(code: int) -> float:
    return float(_e4m3_dec(code))


def splitmix64(index: int, seed: int) -> int:
    return int(_splitmix(index, seed))


def random_f16_bits(index: int, seed: int) -> int:
    return int(_rand_f16(index, seed))


def block_cdiv(a: int, b: int) -> int:
    return int(_cdiv(a, b))


def grid_swizzle(bx: int, by: int, gx: int, gy: int, group: int):
    n, m = C.c_uint32(), C.c_uint32()
    _swz(bx, by, gx, gy, group, C.byref(n), C.byref(m))
    return n.value, m.value


# ---- inputs ----------------------------------------------------------------
def fill_random_f16(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, np.uint16)
    _fill_rand(_p(out, _u16p), n, seed)
    return out


def fill_normal_f16(n: int, seed: int, std: float = 1.0, index0: int = 0) -> np.ndarray:
    out = np.empty(n, np.uint16)
    _fill_norm(_p(out, _u16p), n, index0, seed, std)
    return out


def fill_uniform_f16(n: int, seed: int, lo: float, hi: float, index0: int = 0) -> np.ndarray:
    out = np.empty(n, np.uint16)
    _fill_unif(_p(out, _u16p), n, index0, seed, lo, hi)
    return out


# ---- FP8 -------------------------------------------------------------------
def amax_f16(x: np.ndarray) -> float:
    x = _c(x, np.uint16)
    return float(_amax16(_p(x, _u16p), x.size))


def amax_f32(x: np.ndarray) -> float:
    x = _c(x, np.float32)
    return float(_amax32(_p(x, _f32p), x.size))


def scale_from_amax(amax: float) -> float:
    return float(_scale(amax))


def quantize_fp8_f16(x: np.ndarray, scale: float) -> np.ndarray:
    x = _c(x, np.uint16)
    q = np.empty(x.shape, np.uint8)
    _q16(_p(x, _u16p), x.size, scale, _p(q, _u8p))
    return q


def quantize_fp8_f32(x: np.ndarray, scale: float) -> np.ndarray:
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    _q32(_p(x, _f32p), x.size, scale, _p(q, _u8p))
    return q


def quantize_fp8_f16_transpose(x: np.ndarray, scale: float) -> np.ndarray:
    x = _c(x, np.uint16)
    rows, cols = x.shape
    q = np.empty((cols, rows), np.uint8)
    _q16t(_p(x, _u16p), rows, cols, scale, _p(q, _u8p))
    return q


def e4m3_decode_array(q: np.ndarray) -> np.ndarray:
    lut = np.array([e4m3_decode(i) for i in range(256)], np.float32)
    return lut[q]


def rmsnorm_f16(x: np.ndarray, gamma: np.ndarray, eps: float):
    """Returns (y f32 [rows, hidden], rstd f32 [rows], amax)."""
    x, gamma = _c(x, np.uint16), _c(gamma, np.uint16)
    rows, hidden = x.shape
    y = np.empty((rows, hidden), np.float32)
    rstd = np.empty(rows, np.float32)
    amax = _rms(_p(x, _u16p), _p(gamma, _u16p), rows, hidden, eps, _p(y, _f32p), _p(rstd, _f32p))
    return y, rstd, float(amax)


def rmsnorm_residual_f16(x: np.ndarray, residual: np.ndarray, weight: np.ndarray, eps: float):
    """Fused add + RMSNorm on f16 bit patterns. Returns (out, new_residual), both uint16 [rows, hidden]."""
    x, residual, weight = _c(x, np.uint16), _c(residual, np.uint16), _c(weight, np.uint16)
    rows, hidden = x.shape
    out = np.empty((rows, hidden), np.uint16)
    new_res = np.empty((rows, hidden), np.uint16)
    _rmsres(_p(x, _u16p), _p(residual, _u16p), _p(weight, _u16p), rows, hidden, eps, _p(out, _u16p), _p(new_res, _u16p))
    return out, new_res


def rope_f16(x: np.ndarray, positions: np.ndarray, base: float = 10000.0) -> np.ndarray:
    """Interleaved-pair rotary embedding on f16 bit patterns [rows, head_dim]; positions int32 [rows]."""
    x, positions = _c(x, np.uint16), _c(positions, np.int32)
    rows, head_dim = x.shape
    out = np.empty((rows, head_dim), np.uint16)
    _rope(_p(x, _u16p), positions.ctypes.data_as(C.POINTER(C.c_int32)), rows, head_dim, base, _p(out, _u16p))
    return out


def paged_decode_attention(q: np.ndarray, kcache: np.ndarray, vcache: np.ndarray, page_table: np.ndarray,
                           seq_lens: np.ndarray) -> np.ndarray:
    """q [S, Hq, D], caches [pages, page, Hkv, D] as f16 bit patterns; int32 page_table [S, max_pages],
    seq_lens [S]. Returns out [S, Hq, D] f16 bit patterns."""
    q, kcache, vcache = _c(q, np.uint16), _c(kcache, np.uint16), _c(vcache, np.uint16)
    page_table, seq_lens = _c(page_table, np.int32), _c(seq_lens, np.int32)
    s, hq, d = q.shape
    _, page, hkv, _ = kcache.shape
    out = np.empty((s, hq, d), np.uint16)
    _attn(_p(q, _u16p), _p(kcache, _u16p), _p(vcache, _u16p), page_table.ctypes.data_as(_i32p),
          seq_lens.ctypes.data_as(_i32p), s, hq, hkv, d, page, page_table.shape[1], _p(out, _u16p))
    return out


def rmsnorm_quantize_fp8(x: np.ndarray, gamma: np.ndarray, eps: float):
    """Returns (codes u8 [rows, hidden], scale)."""
    x, gamma = _c(x, np.uint16), _c(gamma, np.uint16)
    rows, hidden = x.shape
    q = np.empty((rows, hidden), np.uint8)
    s = C.c_float()
    _rmsq(_p(x, _u16p), _p(gamma, _u16p), rows, hidden, eps, _p(q, _u8p), C.byref(s))
    return q, float(s.value)


def _out_array(rows: int, cols: int, out_kind: int) -> np.ndarray:
    return np.empty((rows, cols), np.float32 if out_kind == OUT_F32 else np.uint16)


def _bias_args(bias):
    if bias is None:
        return None, BIAS_NONE, None
    if bias.dtype == np.float32:
        b = _c(bias, np.float32)
        return b.ctypes.data_as(C.c_void_p), BIAS_F32, b
    b = _c(bias, np.uint16)
    return b.ctypes.data_as(C.c_void_p), BIAS_F16, b


def gemm_fp8(aq, bqt, scale_a, scale_b, bias=None, epilogue=EPI_NONE, out_kind=OUT_F32,
             row_begin=0, row_count=None) -> np.ndarray:
    """aq [M, K] codes, bqt [N, K] codes (B stored K-major)."""
    aq, bqt = _c(aq, np.uint8), _c(bqt, np.uint8)
    (M, K), (N, K2) = aq.shape, bqt.shape
    assert K == K2
    row_count = M - row_begin if row_count is None else row_count
    out = _out_array(row_count, N // 2 if epilogue == EPI_SWIGLU else N, out_kind)
    bptr, bkind, keep = _bias_args(bias)
    _gemm8(_p(aq, _u8p), _p(bqt, _u8p), M, N, K, scale_a, scale_b, bptr, bkind, epilogue,
           out_kind, out.ctypes.data_as(C.c_void_p), row_begin, row_count)
    del keep
    return out


def decode_e4m3(q: np.ndarray) -> np.ndarray:
    q = _c(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    _dec8(_p(q, _u8p), q.size, _p(out, _f32p))
    return out


def gemm_fp8_decoded(aq, bf, scale_a, scale_b, out_kind=OUT_F32) -> np.ndarray:
    """gemm_fp8 with the weight operand already decoded by `decode_e4m3` ([N, K] f32)."""
    aq, bf = _c(aq, np.uint8), _c(bf, np.float32)
    (M, K), (N, _) = aq.shape, bf.shape
    out = _out_array(M, N, out_kind)
    _gemm8d(_p(aq, _u8p), _p(bf, _f32p), M, N, K, scale_a, scale_b, None, BIAS_NONE, EPI_NONE, out_kind,
            out.ctypes.data_as(C.c_void_p), 0, M)
    return out


def gemm_f16(a, bt, bias=None, epilogue=EPI_NONE, out_kind=OUT_F32, row_begin=0,
             row_count=None) -> np.ndarray:
    a, bt = _c(a, np.uint16), _c(bt, np.uint16)
    (M, K), (N, K2) = a.shape, bt.shape
    assert K == K2
    row_count = M - row_begin if row_count is None else row_count
    out = _out_array(row_count, N // 2 if epilogue == EPI_SWIGLU else N, out_kind)
    bptr, bkind, keep = _bias_args(bias)
    _gemm16(_p(a, _u16p), _p(bt, _u16p), M, N, K, bptr, bkind, epilogue, out_kind,
            out.ctypes.data_as(C.c_void_p), row_begin, row_count)
    del keep
    return out


def requant_bf16_fp8(h: np.ndarray):
    h = _c(h, np.uint16)
    q = np.empty(h.shape, np.uint8)
    s = C.c_float()
    _requant(_p(h, _u16p), h.size, _p(q, _u8p), C.byref(s))
    return q, float(s.value)


# ---- INT4 ------------------------------------------------------------------
def int4_quantize(w: np.ndarray, group: int = 128):
    """w [K, N] f16 bits -> (qweight u32 [K/8, N], scales f16 bits [K/group, N])."""
    w = _c(w, np.uint16)
    K, N = w.shape
    qw = np.empty((K // 8, N), np.uint32)
    sc = np.empty((K // group, N), np.uint16)
    _i4q(_p(w, _u16p), K, N, group, _p(qw, _u32p), _p(sc, _u16p))
    return qw, sc


def int4_stream_bytes(K: int, N: int) -> int:
    return int(_i4bytes(K, N))


def int4_repack(qweight: np.ndarray, scales: np.ndarray) -> np.ndarray:
    qweight, scales = _c(qweight, np.uint32), _c(scales, np.uint16)
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    out = np.empty(int4_stream_bytes(K, N), np.uint8)
    _i4pack(_p(qweight, _u32p), _p(scales, _u16p), K, N, _p(out, _u8p))
    return out


def gemm_int4_decode(x, qweight, scales, group: int = 128) -> np.ndarray:
    x, qweight, scales = _c(x, np.uint16), _c(qweight, np.uint32), _c(scales, np.uint16)
    M, K = x.shape
    N = qweight.shape[1]
    out = np.empty((M, N), np.uint16)
    _i4gemm(_p(x, _u16p), _p(qweight, _u32p), _p(scales, _u16p), M, N, K, group, _p(out, _u16p))
    return out


# ---- pin library (cuda_fp8.h host conversions) -----------------------------
def load_pin():
    lib = _load("libpin_fp8.so")
    lib.pin_nv_e4m3_encode.restype = C.c_uint8
    lib.pin_nv_e4m3_encode.argtypes = [C.c_float]
    lib.pin_nv_e4m3_decode.restype = C.c_float
    lib.pin_nv_e4m3_decode.argtypes = [C.c_uint8]
    return lib
