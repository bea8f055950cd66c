"""Generates the golden fixtures in this directory.

Run from the repository root:  python tests/golden/make_golden.py

Two kinds of vectors:
  * e4m3_torch.npz - f32 inputs and the e4m3 codes torch's CPU conversion
    (`tensor.to(torch.float8_e4m3fn)`) gives for them: an implementation that is
    independent of the oracle. Covers every representable value, every rounding
    midpoint and its two neighbours, and random values.
  * path_small.npz - small seeded cases of every step of the path (quantise,
    transposed quantise, RMSNorm prologue, INT4 pack/repack, FP8 GEMM with each
    epilogue, INT4 decode GEMM) as computed by the oracle when this file was
    made. They guard the oracle against drift and are what the GPU kernels
    are compared with bit for bit (codes) or within tolerance (GEMM outputs).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def e4m3_vectors():
    dec = [oracle.e4m3_decode(c) for c in range(0x7F)]
    vals = []
    for lo, hi in zip(dec[:-1], dec[1:]):
        lo, hi = np.float32(lo), np.float32(hi)
        mid = np.float32((lo + hi) / np.float32(2))
        for v in (lo, hi, mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1e9))):
            vals += [v, -v]
    rng = np.random.default_rng(1234)
    vals += list((rng.standard_normal(20000) * 120).astype(np.float32))
    vals += list((rng.standard_normal(10000) * 0.03).astype(np.float32))
    x = np.array(vals, np.float32)
    x = x[np.abs(x) < 464.0]  # beyond the last midpoint torch gives NaN, hardware saturates
    codes = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.savez_compressed(os.path.join(HERE, "e4m3_torch.npz"), x=x, codes=codes, decode_table=table)


def path_vectors():
    out = {}
    M, N, K = 48, 40, 128
    a = oracle.fill_normal_f16(M * K, oracle.SEED_A).reshape(M, K)
    b = oracle.fill_normal_f16(K * N, oracle.SEED_B).reshape(K, N)
    sa = oracle.scale_from_amax(oracle.amax_f16(a))
    sb = oracle.scale_from_amax(oracle.amax_f16(b))
    aq = oracle.quantize_fp8_f16(a, sa)
    bqt = oracle.quantize_fp8_f16_transpose(b, sb)
    bias = oracle.fill_normal_f16(N, oracle.SEED_B + 1, 0.1)
    out.update(gemm_shape=np.array([M, N, K]), scale_a=np.float32(sa), scale_b=np.float32(sb),
               aq=aq, bqt=bqt,
               c_f32=oracle.gemm_fp8(aq, bqt, sa, sb),
               c_bias_relu_bf16=oracle.gemm_fp8(aq, bqt, sa, sb, bias=bias,
                                                epilogue=oracle.EPI_BIAS_RELU, out_kind=oracle.OUT_BF16),
               h_swiglu_bf16=oracle.gemm_fp8(aq, bqt, sa, sb, epilogue=oracle.EPI_SWIGLU,
                                             out_kind=oracle.OUT_BF16))
    q, s = oracle.requant_bf16_fp8(out["h_swiglu_bf16"])
    out.update(swiglu_q=q, swiglu_scale=np.float32(s))
    # RMSNorm prologue
    R, H = 6, 512
    x = oracle.fill_normal_f16(R * H, oracle.SEED_A + 7).reshape(R, H)
    g = oracle.fill_uniform_f16(H, oracle.SEED_A + 2, 0.5, 1.5)
    rq, rs = oracle.rmsnorm_quantize_fp8(x, g, 1e-6)
    out.update(rms_shape=np.array([R, H]), rms_q=rq, rms_scale=np.float32(rs))
    # INT4
    K4, N4, M4 = 256, 32, 5
    w = oracle.fill_normal_f16(K4 * N4, oracle.SEED_B + 3, 1.0 / 16.0).reshape(K4, N4)
    xw = oracle.fill_normal_f16(M4 * K4, oracle.SEED_A + 3).reshape(M4, K4)
    qw, sc = oracle.int4_quantize(w)
    out.update(int4_shape=np.array([M4, N4, K4]), int4_qweight=qw, int4_scales=sc,
               int4_stream=oracle.int4_repack(qw, sc),
               int4_out=oracle.gemm_int4_decode(xw, qw, sc))
    np.savez_compressed(os.path.join(HERE, "path_small.npz"), **out)


if __name__ == "__main__":
    e4m3_vectors()
    path_vectors()
    for f in ("e4m3_torch.npz", "path_small.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
