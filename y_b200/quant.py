"""Operator layer of the quantised-inference path on torch CUDA tensors.

Mirrors the operator API the reference documents for `y_lang.ops.quant`
(docs/y_language_documentation.md:4349-4354: `fp8_gemm(a, b, scale_a, scale_b)`,
`int4_weight_only_gemm(x, w_q4, scales, zeros)`) and adds the pieces the
B200 path is made of (amax, quantise, RMSNorm prologue, fused epilogues).
Every function is a thin call into liby_b200.so; torch only supplies device
memory and the current stream. Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import (BF16, E4M3, EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RELU, EPI_BIAS_SILU, EPI_NONE, EPI_SWIGLU, F16, F32,
                   GemmF16Args, GemmFp8Args, LaunchInfo, check, lib)

_KIND = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
_OUT_DTYPE = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _kind(t: torch.Tensor, name: str) -> int:
    try:
        return _KIND[t.dtype]
    except KeyError:
        raise ValueError(f"{name}: unsupported dtype {t.dtype}") from None


def device_status() -> None:
    """Raises if a kernel reported a bounded wait that ran out."""
    check(lib.y_b200_device_status(_stream()))


# ---- FP8 quantisation --------------------------------------------------------
def amax(x: torch.Tensor) -> torch.Tensor:
    """max|x| as a 1-element f32 device tensor."""
    _dev(x, "x")
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    check(lib.y_b200_amax(x.data_ptr(), _kind(x, "x"), x.numel(), out.data_ptr(), _stream()))
    return out


def scale_from_amax(a: torch.Tensor) -> torch.Tensor:
    out = torch.empty(1, dtype=torch.float32, device=a.device)
    check(lib.y_b200_scale_from_amax(a.data_ptr(), out.data_ptr(), _stream()))
    return out


def quantize_fp8(x: torch.Tensor, scale: torch.Tensor, transpose: bool = False) -> torch.Tensor:
    """e4m3 codes (uint8) of x / scale; `transpose` writes [cols, rows]."""
    _dev(x, "x"), _dev(scale, "scale")
    if transpose:
        rows, cols = x.shape
        q = torch.empty((cols, rows), dtype=torch.uint8, device=x.device)
        check(lib.y_b200_quantize_fp8_transpose(x.data_ptr(), _kind(x, "x"), rows, cols,
                                                scale.data_ptr(), q.data_ptr(), _stream()))
    else:
        q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        check(lib.y_b200_quantize_fp8(x.data_ptr(), _kind(x, "x"), x.numel(), scale.data_ptr(),
                                      q.data_ptr(), _stream()))
    return q


def quantize_fp8_dynamic(x: torch.Tensor, transpose: bool = False, out: torch.Tensor | None = None,
                         scale_out: torch.Tensor | None = None):
    """Per-tensor dynamic quantisation: returns (codes, scale) with
    scale = max(amax/448, 1e-12) computed on the device."""
    _dev(x, "x")
    rows = x.shape[0] if x.dim() == 2 else 1
    cols = x.shape[1] if x.dim() == 2 else x.numel()
    if transpose and x.dim() != 2:
        raise ValueError("transpose needs a 2-D tensor")
    shape = (cols, rows) if transpose else tuple(x.shape)
    q = out if out is not None else torch.empty(shape, dtype=torch.uint8, device=x.device)
    s = scale_out if scale_out is not None else torch.empty(1, dtype=torch.float32, device=x.device)
    check(lib.y_b200_quantize_fp8_dynamic(x.data_ptr(), _kind(x, "x"), rows, cols, int(transpose),
                                          q.data_ptr(), s.data_ptr(), _stream()))
    return q, s


def rmsnorm_quantize_fp8(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6,
                         workspace: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """y = x * rsqrt(mean(x^2) + eps) * gamma, quantised to e4m3 with a fresh
    per-tensor scale. x [rows, hidden] f16, gamma [hidden] f16. Returns (codes, scale);
    `out` (uint8 [rows, hidden]) receives the codes if given."""
    _dev(x, "x"), _dev(gamma, "gamma")
    if x.dtype != torch.float16 or gamma.dtype != torch.float16:
        raise ValueError("rmsnorm_quantize_fp8 takes f16 inputs")
    rows, hidden = x.shape
    need = lib.y_b200_rmsnorm_workspace_bytes(rows)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x.device)
    q = out if out is not None else torch.empty((rows, hidden), dtype=torch.uint8, device=x.device)
    if out is not None and (_dev(out, "out").shape != (rows, hidden) or out.dtype != torch.uint8):
        raise ValueError("rmsnorm_quantize_fp8: out must be uint8 [rows, hidden]")
    s = torch.empty(1, dtype=torch.float32, device=x.device)
    check(lib.y_b200_rmsnorm_quantize_fp8(x.data_ptr(), gamma.data_ptr(), rows, hidden, eps,
                                          q.data_ptr(), s.data_ptr(), ws.data_ptr(), ws.numel(),
                                          _stream()))
    return q, s


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5,
                      out: torch.Tensor | None = None, new_residual: torch.Tensor | None = None):
    """h = x + residual; returns (rmsnorm(h) * weight, h), both f16 [rows, hidden]
    (the reference's rmsnorm_residual_<H> kernel; `new_residual` may alias `residual`)."""
    _dev(x, "x"), _dev(residual, "residual"), _dev(weight, "weight")
    if x.dtype != torch.float16 or residual.dtype != torch.float16 or weight.dtype != torch.float16:
        raise ValueError("fused_add_rmsnorm takes f16 tensors")
    if x.shape != residual.shape or weight.shape != (x.shape[1],):
        raise ValueError("fused_add_rmsnorm: x and residual [rows, hidden], weight [hidden]")
    rows, hidden = x.shape
    o = out if out is not None else torch.empty_like(x)
    nr = new_residual if new_residual is not None else torch.empty_like(x)
    check(lib.y_b200_rmsnorm_residual(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), rows, hidden, eps,
                                      o.data_ptr(), nr.data_ptr(), _stream()))
    return o, nr


def rope(x: torch.Tensor, positions: torch.Tensor, base: float = 10000.0, out: torch.Tensor | None = None):
    """Interleaved-pair rotary embedding. x [rows, head_dim] f16 (a row is one token's query
    or key vector of one head), positions [rows] int32; `out` may be x itself."""
    _dev(x, "x"), _dev(positions, "positions")
    if x.dtype != torch.float16 or positions.dtype != torch.int32:
        raise ValueError("rope takes f16 x and int32 positions")
    rows, head_dim = x.shape
    if positions.shape != (rows,):
        raise ValueError("rope: one position per row")
    o = out if out is not None else torch.empty_like(x)
    check(lib.y_b200_rope(x.data_ptr(), positions.data_ptr(), o.data_ptr(), rows, head_dim, float(base), _stream()))
    return o


def paged_decode_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, page_table: torch.Tensor,
                           seq_lens: torch.Tensor, out: torch.Tensor | None = None,
                           workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Decode attention over a paged f16 KV cache. q [S, Hq, D]; kcache, vcache
    [pages, page_size, Hkv, D]; page_table [S, max_pages] int32; seq_lens [S] int32."""
    for t, name in ((q, "q"), (kcache, "kcache"), (vcache, "vcache"), (page_table, "page_table"), (seq_lens, "seq_lens")):
        _dev(t, name)
    if q.dtype != torch.float16 or kcache.dtype != torch.float16 or vcache.dtype != torch.float16:
        raise ValueError("paged_decode_attention takes f16 q and caches")
    if page_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise ValueError("paged_decode_attention takes int32 page_table and seq_lens")
    s, hq, d = q.shape
    _, page_size, hkv, d2 = kcache.shape
    if d2 != d or vcache.shape != kcache.shape or page_table.shape[0] != s or seq_lens.shape != (s,):
        raise ValueError("paged_decode_attention: inconsistent shapes")
    o = out if out is not None else torch.empty_like(q)
    need = lib.y_b200_paged_decode_attention_workspace_bytes(s, hq, hkv, d)
    ws = workspace if workspace is not None else torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    check(lib.y_b200_paged_decode_attention(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), page_table.data_ptr(),
                                            seq_lens.data_ptr(), o.data_ptr(), s, hq, hkv, d, page_size,
                                            page_table.shape[1], ws.data_ptr(), ws.numel(), _stream()))
    return o


# ---- FP8 GEMM -----------------------------------------------------------------
def _scale_fields(args: GemmFp8Args, name: str, s) -> None:
    if isinstance(s, torch.Tensor):
        _dev(s, name)
        if s.dtype != torch.float32:
            raise ValueError(f"{name} must be f32")
        setattr(args, name + "_dev", s.data_ptr())
        setattr(args, name, 1.0)
    else:
        setattr(args, name + "_dev", None)
        setattr(args, name, float(s))


def gemm_fp8_launch_info(m: int, n: int, k: int, cta_n: int = 0) -> LaunchInfo:
    """Grid, block, cluster, shared memory and tile the library would use for this shape."""
    info = LaunchInfo()
    check(lib.y_b200_gemm_fp8_launch_info(m, n, k, cta_n, C.byref(info)))
    return info


def gemm_fp8_codes(aq: torch.Tensor, bqt: torch.Tensor, scale_a, scale_b, *, bias=None,
                   epilogue: int = EPI_NONE, out_dtype=torch.float32, out: torch.Tensor | None = None,
                   amax_out: torch.Tensor | None = None, cta_n: int = 0, max_ctas: int = 0,
                   cta_m: int = 0, replicas=()):
    """C = epilogue((sa*sb) * aq @ bqt^T). aq [M, K], bqt [N, K] e4m3 codes
    (uint8 or float8_e4m3fn). Scales are floats or 1-element f32 device tensors.
    cta_m / cta_n force a tile (cta_m 256 = the CTA-pair kernel); 0 asks the tile table."""
    _dev(aq, "aq"), _dev(bqt, "bqt")
    (m, k), (n, k2) = aq.shape, bqt.shape
    if k != k2:
        raise ValueError(f"K mismatch: {k} vs {k2}")
    out_kind = {v: kk for kk, v in _OUT_DTYPE.items()}[out_dtype]
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    c = out if out is not None else torch.empty((m, n_out), dtype=out_dtype, device=aq.device)
    args = GemmFp8Args()
    args.a, args.bt, args.c = aq.data_ptr(), bqt.data_ptr(), c.data_ptr()
    args.m, args.n, args.k = m, n, k
    _scale_fields(args, "scale_a", scale_a)
    _scale_fields(args, "scale_b", scale_b)
    if bias is not None:
        _dev(bias, "bias")
        args.bias, args.bias_kind = bias.data_ptr(), _kind(bias, "bias")
    args.epilogue, args.out_kind = epilogue, out_kind
    args.amax_out = amax_out.data_ptr() if amax_out is not None else None
    args.cta_n, args.max_ctas, args.cta_m = cta_n, max_ctas, cta_m
    # replicas: device addresses (ints) or tensors laid out like c; every output element is also stored there
    args.c_replica_count = len(replicas)
    for i, r in enumerate(replicas):
        args.c_replicas[i] = r.data_ptr() if isinstance(r, torch.Tensor) else int(r)
    check(lib.y_b200_gemm_fp8(C.byref(args), _stream()))
    return c


def fp8_gemm(a: torch.Tensor, b: torch.Tensor, scale_a, scale_b, out_dtype=torch.float32):
    """The reference's documented operator: a [M, K], b [K, N] in f32/f16/bf16 are
    quantised to e4m3 with the given per-tensor scales, multiplied on the tensor
    cores, and dequantised by scale_a * scale_b. Pre-quantised `float8_e4m3fn`
    inputs are used as they are (b then must already be [N, K], K-major)."""
    if a.dtype == torch.float8_e4m3fn:
        return gemm_fp8_codes(a.view(torch.uint8), b.view(torch.uint8), scale_a, scale_b,
                              out_dtype=out_dtype)
    sa = scale_a if isinstance(scale_a, torch.Tensor) else torch.tensor(
        [scale_a], dtype=torch.float32, device=a.device)
    sb = scale_b if isinstance(scale_b, torch.Tensor) else torch.tensor(
        [scale_b], dtype=torch.float32, device=a.device)
    aq = quantize_fp8(a, sa)
    bqt = quantize_fp8(b, sb, transpose=True)
    return gemm_fp8_codes(aq, bqt, sa, sb, out_dtype=out_dtype)


def gemm_fp8_f32(a: torch.Tensor, b: torch.Tensor, scale_a: float, scale_b: float,
                 workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Drop-in for the reference entry gemm_fp8_<tag>(A, B, scale_a, scale_b, C):
    f32 A [M, K], f32 B [K, N], f32 C."""
    _dev(a, "a"), _dev(b, "b")
    (m, k), (k2, n) = a.shape, b.shape
    if k != k2 or a.dtype != torch.float32 or b.dtype != torch.float32:
        raise ValueError("gemm_fp8_f32 takes f32 A [M, K] and B [K, N]")
    need = lib.y_b200_gemm_fp8_f32_workspace_bytes(m, n, k)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=a.device)
    c = torch.empty((m, n), dtype=torch.float32, device=a.device)
    check(lib.y_b200_gemm_fp8_f32(a.data_ptr(), b.data_ptr(), scale_a, scale_b, c.data_ptr(), m, n,
                                  k, ws.data_ptr(), ws.numel(), _stream()))
    return c


# ---- F16 GEMM family -------------------------------------------------------------
def gemm_f16_kmajor(a: torch.Tensor, bt: torch.Tensor, *, bias=None, epilogue: int = EPI_NONE,
                    out_dtype=torch.float32, out: torch.Tensor | None = None, cta_n: int = 0, cta_m: int = 0):
    """C = epilogue(a @ bt^T) on the tensor cores (kind::f16): a [M, K], bt [N, K], both f16,
    K-major. EPI_SWIGLU: bt rows gate|up interleaved, C [M, N/2] f32 or bf16."""
    _dev(a, "a"), _dev(bt, "bt")
    (m, k), (n, k2) = a.shape, bt.shape
    if k != k2 or a.dtype != torch.float16 or bt.dtype != torch.float16:
        raise ValueError("gemm_f16_kmajor takes f16 a [M, K] and bt [N, K]")
    n_out = n // 2 if epilogue == EPI_SWIGLU else n
    c = out if out is not None else torch.empty((m, n_out), dtype=out_dtype, device=a.device)
    args = GemmF16Args()
    args.a, args.bt, args.c = a.data_ptr(), bt.data_ptr(), c.data_ptr()
    args.m, args.n, args.k = m, n, k
    if bias is not None:
        _dev(bias, "bias")
        args.bias, args.bias_kind = bias.data_ptr(), _kind(bias, "bias")
    args.epilogue, args.out_kind = epilogue, {v: kk for kk, v in _OUT_DTYPE.items()}[out_dtype]
    args.cta_n, args.cta_m = cta_n, cta_m
    check(lib.y_b200_gemm_f16(C.byref(args), _stream()))
    return c


def gemm_f16(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, relu: bool = False,
             out_dtype=torch.float32, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Drop-in for gemm_f16_<tag>(A, B, C) / gemm_f16_bias_relu_<tag>(A, B, Bias, C): f16 A [M, K],
    f16 B [K, N] row-major, C [M, N] f32 (or f16)."""
    _dev(a, "a"), _dev(b, "b")
    (m, k), (k2, n) = a.shape, b.shape
    if k != k2 or a.dtype != torch.float16 or b.dtype != torch.float16:
        raise ValueError("gemm_f16 takes f16 A [M, K] and B [K, N]")
    need = lib.y_b200_gemm_f16_rowmajor_workspace_bytes(n, k)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=a.device)
    c = torch.empty((m, n), dtype=out_dtype, device=a.device)
    check(lib.y_b200_gemm_f16_rowmajor(a.data_ptr(), b.data_ptr(), bias.data_ptr() if bias is not None else None,
                                       _kind(bias, "bias") if bias is not None else 0, int(relu), c.data_ptr(),
                                       {v: kk for kk, v in _OUT_DTYPE.items()}[out_dtype], m, n, k, ws.data_ptr(),
                                       ws.numel(), _stream()))
    return c


def gemm_f16_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor,
                    workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Drop-in for gemm_f16_swiglu_<tag>(X, Wgate, Wup, Out): Out [M, N] f32 = silu(X @ Wgate) * (X @ Wup)."""
    _dev(x, "x"), _dev(w_gate, "w_gate"), _dev(w_up, "w_up")
    (m, k), (k2, n) = x.shape, w_gate.shape
    if k != k2 or w_up.shape != w_gate.shape or any(t.dtype != torch.float16 for t in (x, w_gate, w_up)):
        raise ValueError("gemm_f16_swiglu takes f16 X [M, K] and Wgate, Wup [K, N]")
    need = lib.y_b200_gemm_f16_swiglu_workspace_bytes(n, k)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=x.device)
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    check(lib.y_b200_gemm_f16_swiglu(x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), out.data_ptr(), m, n, k,
                                     ws.data_ptr(), ws.numel(), _stream()))
    return out


def gemm_f16_decode(x: torch.Tensor, w: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """Small-M GEMM with f16 weights streamed once, row-major [K, N] (the reference's
    gemm_f16_decode_m<M> entries): out [M, N] = x [M, K] @ w, 1 <= M <= 32."""
    _dev(x, "x"), _dev(w, "w")
    (m, k), (k2, n) = x.shape, w.shape
    if k != k2 or x.dtype != torch.float16 or w.dtype != torch.float16:
        raise ValueError("gemm_f16_decode takes f16 x [M, K] and w [K, N]")
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    check(lib.y_b200_gemm_f16_decode(x.data_ptr(), k, w.data_ptr(), out.data_ptr(), F32 if out_dtype == torch.float32 else F16,
                                     m, n, k, _stream()))
    return out


def gemm_fp8_swiglu_requant(aq: torch.Tensor, bqt: torch.Tensor, scale_a, scale_b,
                            workspace: torch.Tensor | None = None, cta_n: int = 0, cta_m: int = 0):
    """silu(gate) * up on interleaved gate|up columns, re-quantised to e4m3 with
    a fresh per-tensor scale. Returns (codes [M, N/2], scale, h_bf16 view)."""
    _dev(aq, "aq"), _dev(bqt, "bqt")
    (m, k), (n, _) = aq.shape, bqt.shape
    need = lib.y_b200_swiglu_workspace_bytes(m, n)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=aq.device)
    q = torch.empty((m, n // 2), dtype=torch.uint8, device=aq.device)
    s = torch.empty(1, dtype=torch.float32, device=aq.device)
    args = GemmFp8Args()
    args.a, args.bt, args.c = aq.data_ptr(), bqt.data_ptr(), None
    args.m, args.n, args.k = m, n, k
    _scale_fields(args, "scale_a", scale_a)
    _scale_fields(args, "scale_b", scale_b)
    args.cta_n, args.cta_m = cta_n, cta_m
    args.c = ws.data_ptr()  # replaced by the library; must be non-null for validation
    check(lib.y_b200_gemm_fp8_swiglu_requant(C.byref(args), q.data_ptr(), s.data_ptr(),
                                             ws.data_ptr(), ws.numel(), _stream()))
    h = ws[256:256 + m * (n // 2) * 2].view(torch.bfloat16).view(m, n // 2)
    return q, s, h


def mlp_swiglu_fp8(aq: torch.Tensor, scale_a, w_gate_up_t: torch.Tensor, scale_gate_up: float,
                   w_down_t: torch.Tensor, scale_down: float, out_dtype=torch.bfloat16,
                   out: torch.Tensor | None = None, workspace: torch.Tensor | None = None):
    """out = (silu(A Wg) * (A Wu)) Wdown on e4m3 operands: SwiGLU GEMM, re-quantisation of
    the hidden tensor with a fresh per-tensor scale, down projection; no host sync inside.
    aq [M, K]; w_gate_up_t [2I, K] (gate|up rows interleaved); w_down_t [N_out, I]."""
    _dev(aq, "aq"), _dev(w_gate_up_t, "w_gate_up_t"), _dev(w_down_t, "w_down_t")
    (m, k), (n2, k2), (n_out, inter) = aq.shape, w_gate_up_t.shape, w_down_t.shape
    if k != k2 or n2 != 2 * inter:
        raise ValueError(f"shape mismatch: A {tuple(aq.shape)}, gate|up {tuple(w_gate_up_t.shape)}, "
                         f"down {tuple(w_down_t.shape)}")
    need = lib.y_b200_mlp_workspace_bytes(m, inter)
    ws = workspace if workspace is not None else torch.empty(need, dtype=torch.uint8, device=aq.device)
    o = out if out is not None else torch.empty((m, n_out), dtype=out_dtype, device=aq.device)
    out_kind = {v: kk for kk, v in _OUT_DTYPE.items()}[o.dtype]
    if isinstance(scale_a, torch.Tensor):
        sa, sa_dev = 1.0, _dev(scale_a, "scale_a").data_ptr()
    else:
        sa, sa_dev = float(scale_a), None
    check(lib.y_b200_mlp_swiglu_fp8(aq.data_ptr(), sa, sa_dev, w_gate_up_t.data_ptr(), float(scale_gate_up),
                                    w_down_t.data_ptr(), float(scale_down), o.data_ptr(), out_kind, m, k, inter,
                                    n_out, ws.data_ptr(), ws.numel(), _stream()))
    return o


# ---- INT4 weight-only ------------------------------------------------------------
def int4_quantize(w: torch.Tensor):
    """w [K, N] f16 -> (qweight int32 [K/8, N], scales f16 [K/128, N])."""
    _dev(w, "w")
    if w.dtype != torch.float16:
        raise ValueError("int4_quantize takes f16 weights")
    k, n = w.shape
    qw = torch.empty((k // 8, n), dtype=torch.int32, device=w.device)
    sc = torch.empty((k // 128, n), dtype=torch.float16, device=w.device)
    check(lib.y_b200_int4_quantize(w.data_ptr(), k, n, qw.data_ptr(), sc.data_ptr(), _stream()))
    return qw, sc


def int4_repack(qweight: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Canonical (qweight, scales) -> the streaming buffer the decode kernel reads."""
    _dev(qweight, "qweight"), _dev(scales, "scales")
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    out = torch.empty(lib.y_b200_int4_stream_bytes(k, n), dtype=torch.uint8, device=qweight.device)
    check(lib.y_b200_int4_repack(qweight.data_ptr(), scales.data_ptr(), k, n, out.data_ptr(), _stream()))
    return out


def gemm_int4_decode(x: torch.Tensor, wstream: torch.Tensor, n: int,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """out [M, N] f16 = x [M, K] f16 @ dequant(W), W given as the streaming buffer."""
    _dev(x, "x"), _dev(wstream, "wstream")
    m, k = x.shape
    o = out if out is not None else torch.empty((m, n), dtype=torch.float16, device=x.device)
    check(lib.y_b200_gemm_int4_decode(x.data_ptr(), wstream.data_ptr(), o.data_ptr(), m, n, k, _stream()))
    return o


def probe_chain_read(buffers, nbytes: int, launches: int = 200, reps: int = 7) -> float:
    """Microseconds per launch of a kernel that only reads `nbytes` from each of `buffers` in turn,
    in a chain of programmatic dependent launches (see y_b200_probe_chain_read): the floor a
    weight-streaming launch of that size is held against."""
    import ctypes as C

    for b in buffers:
        _dev(b, "buffer")
    ptrs = (C.c_void_p * len(buffers))(*[b.data_ptr() for b in buffers])
    scratch = torch.zeros(64, dtype=torch.int32, device=buffers[0].device)
    us = C.c_float(0.0)
    check(lib.y_b200_probe_chain_read(ptrs, len(buffers), nbytes, launches, reps, scratch.data_ptr(),
                                      C.byref(us), _stream()))
    return float(us.value)


def int4_weight_only_gemm(x: torch.Tensor, w_q4: torch.Tensor, scales: torch.Tensor, zeros=None):
    """The reference's documented W4A16 operator. `w_q4` is either the canonical
    [K/8, N] int32 packing (repacked on the fly) or a streaming buffer from
    `int4_repack`. The format is symmetric: `zeros` must be None."""
    if zeros is not None:
        raise ValueError("this build's INT4 format is symmetric (no zero-points); pass zeros=None")
    if w_q4.dtype == torch.uint8:
        return gemm_int4_decode(x, w_q4, scales.shape[1])
    return gemm_int4_decode(x, int4_repack(w_q4, scales), w_q4.shape[1])


def fill_random_f16(n: int, seed: int, index0: int = 0, device="cuda") -> torch.Tensor:
    out = torch.empty(n, dtype=torch.float16, device=device)
    check(lib.y_b200_fill_random_f16(out.data_ptr(), n, index0, seed, _stream()))
    return out
