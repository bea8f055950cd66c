"""Shared helpers of the GPU parity tests: oracle inputs to device tensors and the
GEMM acceptance criteria."""
import numpy as np
import torch

import oracle

# GEMM outputs: max-abs-err <= 1e-2 * ||row||_inf and mean relative error <= 2e-3
# against the oracle on identical quantised inputs.
ROW_TOL = 1e-2
MEAN_REL_TOL = 2e-3


def dev(a: np.ndarray) -> torch.Tensor:
    """numpy -> cuda; uint16 bit patterns travel as int16 and are viewed by the caller."""
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32).copy()).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def f16_dev(bits: np.ndarray) -> torch.Tensor:
    return dev(bits).view(torch.float16)


def host_bits(t: torch.Tensor) -> np.ndarray:
    """f16/bf16 cuda tensor -> uint16 bit patterns."""
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def to_f64(arr: np.ndarray, kind: int) -> np.ndarray:
    if kind == oracle.OUT_F32:
        return arr.astype(np.float64)
    if kind == oracle.OUT_F16:
        return arr.view(np.float16).astype(np.float64)
    return (arr.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def assert_gemm_close(got: np.ndarray, ref: np.ndarray, what: str = ""):
    got, ref = got.astype(np.float64), ref.astype(np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    row_inf = np.abs(ref).max(axis=1, keepdims=True)
    err = np.abs(got - ref)
    worst = (err - ROW_TOL * row_inf).max()
    assert worst <= 0, f"{what}: max-abs-err exceeds 1e-2*||row||inf by {worst}"
    mean_rel = err.mean() / max(np.abs(ref).mean(), 1e-30)
    assert mean_rel <= MEAN_REL_TOL, f"{what}: mean relative error {mean_rel}"


def quantised_operands(m, n, k, seed_a=oracle.SEED_A, seed_b=oracle.SEED_B):
    """Seeded N(0,1) f16 A [M,K], B [K,N] and their oracle quantisation."""
    a = oracle.fill_normal_f16(m * k, seed_a).reshape(m, k)
    b = oracle.fill_normal_f16(k * n, seed_b).reshape(k, n)
    sa = oracle.scale_from_amax(oracle.amax_f16(a))
    sb = oracle.scale_from_amax(oracle.amax_f16(b))
    return a, b, sa, sb, oracle.quantize_fp8_f16(a, sa), oracle.quantize_fp8_f16_transpose(b, sb)
