"""INT4 weight-only path on the GPU: quantise/pack and repack are bit-exact against
the oracle; the decode GEMM meets the GEMM acceptance criteria."""
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, dev, f16_dev, host_bits, to_f64

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


@pytest.mark.parametrize("k,n", [(128, 16), (256, 32), (1024, 176), (4096, 1376), (4096, 11008)])
def test_quantise_and_repack_bit_exact(q, k, n):
    w = oracle.fill_normal_f16(k * n, oracle.SEED_B + 3, 1.0 / 16.0).reshape(k, n)
    if k >= 256:
        w[128:256, 5] = 0  # an all-zero group: scale 0, codes 0
    qw, sc = q.int4_quantize(f16_dev(w))
    rq, rs = oracle.int4_quantize(w)
    assert np.array_equal(qw.cpu().numpy().view(np.uint32), rq)
    assert np.array_equal(host_bits(sc), rs)
    stream = q.int4_repack(qw, sc)
    assert np.array_equal(stream.cpu().numpy(), oracle.int4_repack(rq, rs))


def test_quantise_ties_and_near_ties_bit_exact(q):
    # The kernel replaces the per-element division by a multiplication with 1 / s and takes the
    # division only near half-integers. Columns whose quotients are EXACT half-integers (ties go
    # to even), columns of every f16 value of a binade against an awkward scale, subnormal
    # weights and a subnormal scale must still give the oracle's codes.
    k, n = 256, 64
    w = np.zeros((k, n), np.float32)
    rng = np.random.default_rng(17)
    for c in range(n):
        s0 = 2.0 ** -(c % 12)                     # group amax = 7 s0 -> scale exactly s0
        half = (rng.integers(-7, 7, size=k) + 0.5) * s0     # -6.5 .. 6.5 times s0
        w[:, c] = half
        w[0, c] = 7.0 * s0
        w[128, c] = -7.0 * s0
    wh = w.astype(np.float16)
    # awkward scales: amax values whose seventh is not a power of two; all f16 values of [1, 2)
    wh[:128, 40:48] = np.arange(0x3C00, 0x3C00 + 128 * 8, dtype=np.uint16).view(np.float16).reshape(128, 8)
    wh[128:, 40:48] = (np.arange(0x3C00 + 1024 - 128 * 8, 0x3C00 + 1024, dtype=np.uint16).view(np.float16).reshape(128, 8) * np.float16(-1))
    wh[:128, 48:52] = np.arange(1, 1 + 128 * 4, dtype=np.uint16).view(np.float16).reshape(128, 4)   # subnormals only: subnormal scale
    bits = wh.view(np.uint16)
    qw, sc = q.int4_quantize(f16_dev(bits))
    rq, rs = oracle.int4_quantize(bits)
    assert np.array_equal(host_bits(sc), rs)
    assert np.array_equal(qw.cpu().numpy().view(np.uint32), rq)


@pytest.mark.parametrize("m", [1, 2, 4, 7, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("k,n", [(256, 32), (1024, 2368), (4096, 1376)])
def test_decode_gemm_matches_oracle(q, m, k, n):
    w = oracle.fill_normal_f16(k * n, oracle.SEED_B + 3, 1.0 / np.sqrt(k)).reshape(k, n)
    x = oracle.fill_normal_f16(m * k, oracle.SEED_A + 3).reshape(m, k)
    rq, rs = oracle.int4_quantize(w)
    stream = dev(oracle.int4_repack(rq, rs))
    out = q.gemm_int4_decode(f16_dev(x), stream, n)
    q.device_status()
    ref = oracle.gemm_int4_decode(x, rq, rs)
    assert_gemm_close(to_f64(host_bits(out), oracle.OUT_F16), to_f64(ref, oracle.OUT_F16), f"M={m}")


def test_decode_exact_integers_and_determinism(q):
    # integer activations and unit scales: every partial sum is exact, so the
    # result must equal the integer matmul bit for bit
    m, k, n = 8, 1152, 208   # 9 groups: exercises the partial last ring slot
    rng = np.random.default_rng(9)
    qv = rng.integers(-8, 8, size=(k, n)).astype(np.int32)
    xv = rng.integers(-4, 5, size=(m, k)).astype(np.float32)
    nib = (qv & 0xF).astype(np.uint32).reshape(k // 8, 8, n)
    qw = np.zeros((k // 8, n), np.uint32)
    for j in range(8):
        qw |= nib[:, j, :] << np.uint32(4 * j)
    sc = np.full((k // 128, n), np.float16(1.0)).view(np.uint16)
    stream = dev(oracle.int4_repack(qw, sc))
    xd = torch.from_numpy(xv).cuda().to(torch.float16)
    out = q.gemm_int4_decode(xd, stream, n)
    q.device_status()
    ref = xv.astype(np.float64) @ qv.astype(np.float64)
    assert np.array_equal(out.float().cpu().numpy().astype(np.float64), ref.astype(np.float16).astype(np.float64))
    for _ in range(20):
        assert torch.equal(q.gemm_int4_decode(xd, stream, n), out)


def test_decode_config_shape_full(q, golden_dir):
    # K=4096, N=11008 (the decode config), every M of the config
    k, n = 4096, 11008
    w = (torch.randn(k, n, device="cuda") / 64).to(torch.float16)
    qw, sc = q.int4_quantize(w)
    stream = q.int4_repack(qw, sc)
    qw_h, sc_h = qw.cpu().numpy().view(np.uint32), host_bits(sc)
    # pack -> unpack round trip on the device data
    nib = np.stack([(qw_h >> (4 * j)) & 0xF for j in range(8)], axis=1).reshape(k, n).astype(np.int32)
    qint = np.where(nib >= 8, nib - 16, nib)
    wd = qint * np.repeat(sc_h.view(np.float16).astype(np.float32), 128, axis=0)
    assert np.abs(wd - w.float().cpu().numpy()).max() <= np.abs(w.float().cpu().numpy()).max() / 7 * 0.51 + 1e-6
    for m in (1, 3, 4, 8, 32):
        x = torch.randn(m, k, device="cuda", dtype=torch.float16)
        out = q.gemm_int4_decode(x, stream, n)
        q.device_status()
        ref = oracle.gemm_int4_decode(host_bits(x), qw_h, sc_h)
        assert_gemm_close(to_f64(host_bits(out), oracle.OUT_F16), to_f64(ref, oracle.OUT_F16), f"M={m}")
    # up to 8 tokens this shape takes the kernel's straight-line path, 9 tokens its loop: the
    # same sums in the same order, so the first 8 rows must agree bit for bit
    x9 = torch.randn(9, k, device="cuda", dtype=torch.float16)
    assert torch.equal(q.gemm_int4_decode(x9[:8].contiguous(), stream, n), q.gemm_int4_decode(x9, stream, n)[:8])
    g = np.load(os.path.join(golden_dir, "path_small.npz"))
    M4, N4, K4 = g["int4_shape"]
    xw = oracle.fill_normal_f16(M4 * K4, oracle.SEED_A + 3).reshape(M4, K4)
    out = q.gemm_int4_decode(f16_dev(xw), dev(g["int4_stream"]), int(N4))
    assert_gemm_close(to_f64(host_bits(out), oracle.OUT_F16), to_f64(g["int4_out"], oracle.OUT_F16))
    out2 = q.int4_weight_only_gemm(f16_dev(xw), dev(g["int4_qweight"]), f16_dev(g["int4_scales"]))
    assert torch.equal(out, out2)


def test_decode_preconditions(q):
    from y_b200._lib import YB200Error, ERR_SHAPE
    x = torch.zeros(33, 128, dtype=torch.float16, device="cuda")
    s = torch.zeros(1056, dtype=torch.uint8, device="cuda")
    with pytest.raises(YB200Error) as e:
        q.gemm_int4_decode(x, s, 16)
    assert e.value.code == ERR_SHAPE
    with pytest.raises(YB200Error):
        q.gemm_int4_decode(x[:4, :100].contiguous(), s, 16)


@pytest.mark.parametrize("tiles", [592, 740, 800, 149, 1376])
def test_decode_both_paths_on_mixed_shares(q, tiles):
    # K = 4096 with 592 / 740 column tiles: every CTA owns 4 / 5 tiles (straight-line path);
    # 800: shares of 5 and 6 (both paths in one launch); 149: shares of 1 and 2 (loop only);
    # 1376 (N = 22016): up to 8 tokens run as two waves of CTAs with 4 or 5 tiles each
    k, n = 4096, 16 * tiles
    w = oracle.fill_normal_f16(k * n, oracle.SEED_B + 11, 1.0 / 64.0).reshape(k, n)
    rq, rs = oracle.int4_quantize(w)
    stream = dev(oracle.int4_repack(rq, rs))
    x = oracle.fill_normal_f16(9 * k, oracle.SEED_A + 11).reshape(9, k)
    xd = f16_dev(x)
    out9 = q.gemm_int4_decode(xd, stream, n)          # 9 tokens: the loop path everywhere
    for m in (1, 5, 8):
        out = q.gemm_int4_decode(xd[:m].contiguous(), stream, n)
        assert torch.equal(out, out9[:m]), m
    q.device_status()
    ref = oracle.gemm_int4_decode(x[:8], rq, rs)
    assert_gemm_close(to_f64(host_bits(out), oracle.OUT_F16), to_f64(ref, oracle.OUT_F16))


def test_chain_read_probe_reports_a_launch_time(q):
    # the measurement aid bench.py holds the decode kernel against: a plain reader in a chain of
    # programmatic dependent launches; the time must be positive and below a millisecond here
    bufs = [torch.full((1 << 22,), i + 1, dtype=torch.uint8, device="cuda") for i in range(4)]
    us = q.probe_chain_read(bufs, 1 << 22, launches=20, reps=3)
    q.device_status()
    assert 0.5 < us < 1000.0
