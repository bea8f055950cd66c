"""Parity of the tcgen05 FP8 GEMM and its fused epilogues with the oracle, through
the C ABI. Exact-integer operands make any layout or descriptor mistake an exact
mismatch; seeded N(0,1) operands are held to the path's acceptance criteria."""
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, dev, f16_dev, host_bits, quantised_operands, to_f64

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


def _int_codes(shape, seed, lo=-8, hi=8):
    """Small integers as e4m3 codes: products and sums up to K=4096 are exact in f32."""
    rng = np.random.default_rng(seed)
    v = rng.integers(lo, hi + 1, size=shape).astype(np.float32)
    return np.array([oracle.e4m3_encode(float(t)) for t in v.ravel()], np.uint8).reshape(shape), v


@pytest.mark.parametrize("m,n,k,cta_n", [
    (128, 256, 128, 256), (128, 64, 128, 64), (128, 128, 128, 128),   # one tile, one k-block
    (128, 256, 512, 256), (256, 512, 256, 256), (384, 320, 384, 128),  # several tiles / k-blocks
    (17, 9, 64, 64), (33, 17, 128, 64), (130, 130, 192, 128), (513, 513, 256, 256),  # ragged
    (128, 256, 80, 256), (100, 72, 16, 64),                           # K tail inside a k-block
    (2048, 2304, 1024, 0),                                            # many tiles per CTA, table-picked tile
])
def test_exact_integer_gemm(q, m, n, k, cta_n):
    aq, av = _int_codes((m, k), 1000 + m + k)
    bq, bv = _int_codes((n, k), 2000 + n + k)
    ref = av.astype(np.float64) @ bv.astype(np.float64).T
    c = q.gemm_fp8_codes(dev(aq), dev(bq), 1.0, 1.0, cta_n=cta_n)
    q.device_status()
    assert np.array_equal(c.cpu().numpy().astype(np.float64), ref)


@pytest.mark.parametrize("m,n,k", [
    (256, 256, 128), (256, 256, 512), (512, 768, 512),       # whole 256 x 256 tiles
    (300, 500, 384), (513, 257, 256), (17, 9, 64), (130, 130, 192), (200, 72, 80),  # ragged, K tail
    (2048, 2304, 1024), (4864, 4864, 256),                   # several tiles per CTA pair; 19 x 19 tiles
    # 80, 75 and 90 tiles on 74 pairs: the last wave is cut into 256 x 128 half tiles
    (2048, 2560, 256), (3840, 1280, 128), (2088, 2536, 192),
])
def test_exact_integer_gemm_cta_pair(q, m, n, k):
    """The cta_group::2 kernel: two CTAs of a cluster share each 256 x 256 tile."""
    aq, av = _int_codes((m, k), 3000 + m + k)
    bq, bv = _int_codes((n, k), 4000 + n + k)
    ref = av.astype(np.float64) @ bv.astype(np.float64).T
    c = q.gemm_fp8_codes(dev(aq), dev(bq), 1.0, 1.0, cta_m=256)
    q.device_status()
    assert np.array_equal(c.cpu().numpy().astype(np.float64), ref)
    # an odd CTA budget is rounded down to whole pairs
    c = q.gemm_fp8_codes(dev(aq), dev(bq), 1.0, 1.0, cta_m=256, max_ctas=5)
    q.device_status()
    assert np.array_equal(c.cpu().numpy().astype(np.float64), ref)


def test_every_cta_n_agrees_and_repeated_launches_are_bit_identical(q):
    m, n, k = 640, 768, 512
    _, _, sa, sb, aq, bqt = quantised_operands(m, n, k)
    ad, bd = dev(aq), dev(bqt)
    outs = [q.gemm_fp8_codes(ad, bd, sa, sb, cta_n=t) for t in (64, 128, 256)]
    outs.append(q.gemm_fp8_codes(ad, bd, sa, sb, cta_m=256))
    q.device_status()
    for o in outs[:3]:
        assert torch.equal(outs[3], o)  # the K order of the accumulation does not depend on the tile
    # the shared-memory race detector of the reference harness: relaunch with fixed
    # inputs, require bit-identical output (tests/test_fp8_gemm_correctness.py:156-171)
    for _ in range(20):
        again = q.gemm_fp8_codes(ad, bd, sa, sb, cta_n=256)
        assert torch.equal(again, outs[2])
        again = q.gemm_fp8_codes(ad, bd, sa, sb, cta_m=256)
        assert torch.equal(again, outs[2])
    ref = oracle.gemm_fp8(aq, bqt, sa, sb)
    for o in outs:
        assert_gemm_close(o.cpu().numpy(), ref)


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (48, 40, 128), (300, 200, 320)])
@pytest.mark.parametrize("out", ["f32", "f16", "bf16"])
def test_scale_epilogue_and_output_types(q, m, n, k, out):
    _, _, sa, sb, aq, bqt = quantised_operands(m, n, k)
    kind = {"f32": oracle.OUT_F32, "f16": oracle.OUT_F16, "bf16": oracle.OUT_BF16}[out]
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[out]
    sad = torch.tensor([sa], dtype=torch.float32, device="cuda")
    ref = oracle.gemm_fp8(aq, bqt, sa, sb, out_kind=kind)
    for cta_m in (128, 256):
        c = q.gemm_fp8_codes(dev(aq), dev(bqt), sad, sb, out_dtype=dt, cta_m=cta_m)  # one device scale, one by value
        q.device_status()
        got = c.cpu().numpy() if out == "f32" else host_bits(c)
        assert_gemm_close(to_f64(got, kind), to_f64(ref, kind), out)


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (130, 72, 192), (2048, 2560, 128)])
@pytest.mark.parametrize("bias_dtype", ["f16", "f32"])
@pytest.mark.parametrize("cta_m", [128, 256])
def test_bias_relu_epilogue(q, m, n, k, bias_dtype, cta_m):
    _, _, sa, sb, aq, bqt = quantised_operands(m, n, k)
    bias = oracle.fill_normal_f16(n, oracle.SEED_B + 1, 0.1)
    if bias_dtype == "f16":
        bd, bo = f16_dev(bias), bias
    else:
        bo = bias.view(np.float16).astype(np.float32)
        bd = dev(bo)
    for epi, oepi in ((q.EPI_BIAS, oracle.EPI_BIAS), (q.EPI_BIAS_RELU, oracle.EPI_BIAS_RELU)):
        c = q.gemm_fp8_codes(dev(aq), dev(bqt), sa, sb, bias=bd, epilogue=epi, out_dtype=torch.bfloat16,
                             cta_m=cta_m)
        q.device_status()
        ref = oracle.gemm_fp8(aq, bqt, sa, sb, bias=bo, epilogue=oepi, out_kind=oracle.OUT_BF16)
        got = to_f64(host_bits(c), oracle.OUT_BF16)
        assert_gemm_close(got, to_f64(ref, oracle.OUT_BF16), f"epi{epi}")
        if epi == q.EPI_BIAS_RELU:
            assert got.min() >= 0.0


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (130, 72, 192)])
@pytest.mark.parametrize("cta_m", [128, 256])
@pytest.mark.parametrize("with_bias", [True, False])
def test_gelu_and_silu_epilogues(q, m, n, k, cta_m, with_bias):
    """The rest of the reference's activation functor set (src/quantization_pass.rs:716-796):
    its tanh-form GELU (with the coefficients exactly as its emitter writes them) and SiLU, fused
    after the optional bias add; the device uses tanh.approx / ex2.approx as the emitted code does,
    the oracle libm, so the comparison is by the GEMM tolerance."""
    _, _, sa, sb, aq, bqt = quantised_operands(m, n, k)
    sa, sb = sa / 8, sb / 8          # keep the pre-activations in the curved part of both functions
    bias = oracle.fill_normal_f16(n, oracle.SEED_B + 1, 0.5)
    for epi, oepi in ((q.EPI_BIAS_GELU, oracle.EPI_BIAS_GELU), (q.EPI_BIAS_SILU, oracle.EPI_BIAS_SILU)):
        c = q.gemm_fp8_codes(dev(aq), dev(bqt), sa, sb, bias=f16_dev(bias) if with_bias else None, epilogue=epi,
                             out_dtype=torch.float32, cta_m=cta_m)
        q.device_status()
        ref = oracle.gemm_fp8(aq, bqt, sa, sb, bias=bias if with_bias else None, epilogue=oepi)
        pre = oracle.gemm_fp8(aq, bqt, sa, sb, bias=bias if with_bias else None,
                              epilogue=oracle.EPI_BIAS if with_bias else oracle.EPI_NONE)
        assert np.abs(ref - pre).max() > 0.05        # the activation did something
        assert_gemm_close(c.cpu().numpy(), ref, f"epilogue {epi}, bias {with_bias}")


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (100, 88, 128), (2048, 2560, 128)])
@pytest.mark.parametrize("cta_m", [128, 256])
def test_swiglu_requant(q, m, n, k, cta_m):
    a, b, sa, sb, aq, bqt = quantised_operands(m, n, k)
    codes, scale, h = q.gemm_fp8_swiglu_requant(dev(aq), dev(bqt), sa, sb, cta_m=cta_m)
    q.device_status()
    h_ref = oracle.gemm_fp8(aq, bqt, sa, sb, epilogue=oracle.EPI_SWIGLU, out_kind=oracle.OUT_BF16)
    h_got = host_bits(h)
    assert_gemm_close(to_f64(h_got, oracle.OUT_BF16), to_f64(h_ref, oracle.OUT_BF16), "h")
    # the requant step is bit-exact given the h the device produced
    q_ref, s_ref = oracle.requant_bf16_fp8(h_got)
    assert scale.item() == np.float32(s_ref)
    assert np.array_equal(codes.cpu().numpy(), q_ref)
    # and the dequantised result meets the GEMM criteria against the all-oracle chain
    qo, so = oracle.requant_bf16_fp8(h_ref)
    assert_gemm_close(oracle.e4m3_decode_array(codes.cpu().numpy()) * scale.item(),
                      oracle.e4m3_decode_array(qo) * so, "requant")


def test_committed_golden_case(q, golden_dir):
    g = np.load(os.path.join(golden_dir, "path_small.npz"))
    sa, sb = float(g["scale_a"]), float(g["scale_b"])
    c = q.gemm_fp8_codes(dev(g["aq"]), dev(g["bqt"]), sa, sb)
    assert_gemm_close(c.cpu().numpy(), g["c_f32"])
    bias = oracle.fill_normal_f16(int(g["gemm_shape"][1]), oracle.SEED_B + 1, 0.1)
    cb = q.gemm_fp8_codes(dev(g["aq"]), dev(g["bqt"]), sa, sb, bias=f16_dev(bias),
                          epilogue=q.EPI_BIAS_RELU, out_dtype=torch.bfloat16)
    assert_gemm_close(to_f64(host_bits(cb), oracle.OUT_BF16),
                      to_f64(g["c_bias_relu_bf16"], oracle.OUT_BF16))


def test_reference_entry_f32_operands(q):
    # gemm_fp8_256 of the reference: f32 A, B [K, N]; randn * 3; scale = amax / 448
    m = n = k = 256
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 3).astype(np.float32)
    sa, sb = oracle.scale_from_amax(oracle.amax_f32(a)), oracle.scale_from_amax(oracle.amax_f32(b))
    c = q.gemm_fp8_f32(dev(a), dev(b), sa, sb)
    q.device_status()
    aq = oracle.quantize_fp8_f32(a, sa)
    bqt = np.ascontiguousarray(oracle.quantize_fp8_f32(b, sb).T)
    ref = oracle.gemm_fp8(aq, bqt, sa, sb)
    assert_gemm_close(c.cpu().numpy(), ref)
    # the reference's own gate: rel-L2 < 2% (tests/test_fp8_gemm_correctness.py:208)
    full = a.astype(np.float64) @ b.astype(np.float64)
    rel_l2 = np.linalg.norm(c.cpu().numpy() - full) / np.linalg.norm(full)
    assert rel_l2 < 0.05  # e4m3 quantisation noise itself is ~3-4% on N(0,1) data
    c2 = q.fp8_gemm(dev(a), dev(b), sa, sb)
    assert torch.equal(c2, c)


def test_full_size_4096_sampled_rows_and_linearity(q):
    # the fused-epilogue config: 4096^3, f16 bias ~N(0, 0.1), ReLU, bf16 out
    m = n = k = 4096
    a = torch.randn(m, k, device="cuda", dtype=torch.float16)
    b = torch.randn(k, n, device="cuda", dtype=torch.float16)
    aq, sa = q.quantize_fp8_dynamic(a)
    bqt, sb = q.quantize_fp8_dynamic(b, transpose=True)
    bias = (torch.randn(n, device="cuda") * 0.1).to(torch.float16)
    c = q.gemm_fp8_codes(aq, bqt, sa, sb, bias=bias, epilogue=q.EPI_BIAS_RELU, out_dtype=torch.bfloat16)
    q.device_status()
    rows = [0, 1, 127, 128, 2047, 2048, 3000, 4095]
    aq_h, bqt_h = aq.cpu().numpy(), bqt.cpu().numpy()
    bias_h = host_bits(bias)
    for r in rows:
        ref = oracle.gemm_fp8(aq_h, bqt_h, sa.item(), sb.item(), bias=bias_h,
                              epilogue=oracle.EPI_BIAS_RELU, out_kind=oracle.OUT_BF16,
                              row_begin=r, row_count=1)
        got = host_bits(c[r:r + 1])
        assert_gemm_close(to_f64(got, oracle.OUT_BF16), to_f64(ref, oracle.OUT_BF16), f"row {r}")
    # size-independent property: the scale epilogue is linear in scale_a
    c1 = q.gemm_fp8_codes(aq, bqt, 1.0, 1.0)
    c2 = q.gemm_fp8_codes(aq, bqt, 2.0, 1.0)
    assert torch.equal(c2, c1 * 2)
    # and C^T = B^T A^T: swapping operand roles gives the transposed result
    ct = q.gemm_fp8_codes(bqt, aq, 1.0, 1.0)
    assert torch.allclose(ct.t(), c1, rtol=0, atol=0)


def test_swiglu_requant_at_the_benchmark_shape_sampled_rows(q):
    """The fused SwiGLU configuration at its full size: M = K = 4096, N = 2 x 11008 gate|up
    interleaved (1376 tiles over 74 CTA pairs: 18 full waves and a partial one), bf16 h with a
    running amax, then e4m3 re-quantisation. Whole rows from several M tiles against the oracle;
    the re-quantisation of the whole tensor bit-exact given the device's h."""
    m, k, n = 4096, 4096, 22016
    g = torch.Generator(device="cuda")
    g.manual_seed(44)
    a = torch.randn(m, k, device="cuda", dtype=torch.float16, generator=g)
    w = (torch.randn(k, n, device="cuda", generator=g) / 64).to(torch.float16)
    aq, sa = q.quantize_fp8_dynamic(a)
    bqt, sb = q.quantize_fp8_dynamic(w, transpose=True)
    del a, w
    codes, scale, h = q.gemm_fp8_swiglu_requant(aq, bqt, sa, sb)
    q.device_status()
    aq_h, bqt_h = aq.cpu().numpy(), bqt.cpu().numpy()
    h_got = host_bits(h)
    assert h_got.shape == (m, n // 2)
    for r in (0, 255, 256, 1000, 2047, 2048, 3333, 4095):
        ref = oracle.gemm_fp8(aq_h, bqt_h, sa.item(), sb.item(), epilogue=oracle.EPI_SWIGLU,
                              out_kind=oracle.OUT_BF16, row_begin=r, row_count=1)
        assert_gemm_close(to_f64(h_got[r:r + 1], oracle.OUT_BF16), to_f64(ref, oracle.OUT_BF16), f"h row {r}")
    q_ref, s_ref = oracle.requant_bf16_fp8(h_got)
    assert scale.item() == np.float32(s_ref)
    assert np.array_equal(codes.cpu().numpy(), q_ref)
    # the running amax the epilogue kept equals the maximum of what it stored
    assert np.float32(s_ref) == np.float32(oracle.scale_from_amax(float(np.abs(to_f64(h_got, oracle.OUT_BF16)).max())))


def test_preconditions_are_errors(q):
    from y_b200._lib import YB200Error, ERR_SHAPE, ERR_INVALID
    a = torch.zeros(16, 24, dtype=torch.uint8, device="cuda")
    with pytest.raises(YB200Error) as e:
        q.gemm_fp8_codes(a, a, 1.0, 1.0)  # K = 24 is not a multiple of 16
    assert e.value.code == ERR_SHAPE
    a = torch.zeros(16, 32, dtype=torch.uint8, device="cuda")
    with pytest.raises(YB200Error) as e:
        q.gemm_fp8_codes(a, a, 1.0, 1.0, epilogue=q.EPI_BIAS)  # bias epilogue, no bias
    assert e.value.code == ERR_INVALID
    with pytest.raises(YB200Error) as e:
        q.gemm_fp8_codes(a, a, 1.0, 1.0, cta_m=256, cta_n=128)  # the CTA pair has one tile shape
    assert e.value.code == ERR_INVALID


@pytest.mark.parametrize("m,k,inter,n_out", [(256, 256, 384, 320), (100, 128, 176, 72)])
def test_gated_mlp_chain(q, m, k, inter, n_out):
    """SwiGLU GEMM -> e4m3 re-quantisation -> down projection, one call, no host sync."""
    a, wgu, sa, sgu, aq, wgu_t = quantised_operands(m, 2 * inter, k)
    wd = oracle.fill_normal_f16(inter * n_out, oracle.SEED_B + 5).reshape(inter, n_out)
    sd = oracle.scale_from_amax(oracle.amax_f16(wd))
    wd_t = oracle.quantize_fp8_f16_transpose(wd, sd)
    out = q.mlp_swiglu_fp8(dev(aq), sa, dev(wgu_t), sgu, dev(wd_t), sd)
    q.device_status()
    got = to_f64(host_bits(out), oracle.OUT_BF16)
    # step by step from what the device produced in between: the down GEMM is held to the
    # GEMM criteria on the device's own hidden codes and scale
    hq, sh, _ = q.gemm_fp8_swiglu_requant(dev(aq), dev(wgu_t), sa, sgu)
    ref_from_dev_h = oracle.gemm_fp8(hq.cpu().numpy(), wd_t, float(sh.item()), sd, out_kind=oracle.OUT_BF16)
    assert_gemm_close(got, to_f64(ref_from_dev_h, oracle.OUT_BF16), "down")
    # and end to end against the all-oracle chain (the re-quantised hidden tensor may differ
    # by one code where h sits on a rounding boundary, so the bound is the same criteria
    # applied to the final output)
    h_ref = oracle.gemm_fp8(aq, wgu_t, sa, sgu, epilogue=oracle.EPI_SWIGLU, out_kind=oracle.OUT_BF16)
    hq_ref, sh_ref = oracle.requant_bf16_fp8(h_ref)
    ref = oracle.gemm_fp8(hq_ref, wd_t, sh_ref, sd, out_kind=oracle.OUT_BF16)
    assert_gemm_close(got, to_f64(ref, oracle.OUT_BF16), "chain")
    # a device-side scale for A gives the same result as the same scale by value
    sad = torch.tensor([sa], dtype=torch.float32, device="cuda")
    assert torch.equal(q.mlp_swiglu_fp8(dev(aq), sad, dev(wgu_t), sgu, dev(wd_t), sd), out)
