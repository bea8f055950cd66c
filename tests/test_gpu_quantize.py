"""Bit-exact parity of the HBM-bound kernels (amax, e4m3 quantise, transposed
quantise, RMSNorm prologue, input generator) with the oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import dev, f16_dev, host_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


@pytest.mark.parametrize("n", [1, 7, 8, 15, 16, 17, 255, 4096, 65536 + 5, 1 << 20])
def test_amax_and_quantise_f16_bit_exact(q, n):
    x = oracle.fill_normal_f16(n, 100 + n)
    xd = f16_dev(x)
    amax = q.amax(xd)
    assert amax.item() == oracle.amax_f16(x)
    scale = q.scale_from_amax(amax)
    s = oracle.scale_from_amax(oracle.amax_f16(x))
    assert scale.item() == np.float32(s)
    codes = q.quantize_fp8(xd, scale).cpu().numpy()
    assert np.array_equal(codes, oracle.quantize_fp8_f16(x, s))
    qd, sd = q.quantize_fp8_dynamic(xd)
    assert sd.item() == np.float32(s) and np.array_equal(qd.cpu().numpy(), codes)


def test_quantise_f32_and_bf16_inputs(q):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(100003) * 3).astype(np.float32)  # the reference harness uses randn * 3
    s = oracle.scale_from_amax(oracle.amax_f32(x))
    qd, sd = q.quantize_fp8_dynamic(dev(x))
    assert sd.item() == np.float32(s)
    assert np.array_equal(qd.cpu().numpy(), oracle.quantize_fp8_f32(x, s))
    xb = torch.from_numpy(x).to(torch.bfloat16)
    xbf = xb.float().numpy()
    sb = oracle.scale_from_amax(oracle.amax_f32(xbf))
    qb, sbd = q.quantize_fp8_dynamic(xb.cuda())
    assert sbd.item() == np.float32(sb)
    assert np.array_equal(qb.cpu().numpy(), oracle.quantize_fp8_f32(xbf, sb))


def test_quantise_edge_values(q):
    # zeros (scale floor 1e-12), saturation, subnormal codes, static scale
    z = torch.zeros(1000, dtype=torch.float16, device="cuda")
    qd, sd = q.quantize_fp8_dynamic(z)
    assert sd.item() == np.float32(1e-12) and int(qd.max()) == 0
    vals = np.array([0, 1e-4, -1e-4, 0.0009765625, 0.001953125, 0.0029296875, 1.0, 448, 449, 500,
                     60000, -60000, 0.0146484375, 0.015625], np.float32).astype(np.float16)
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    got = q.quantize_fp8(dev(vals.view(np.uint16)).view(torch.float16), one).cpu().numpy()
    assert np.array_equal(got, oracle.quantize_fp8_f16(vals.view(np.uint16), 1.0))
    assert got[7] == 0x7E and got[10] == 0x7E and got[11] == 0xFE


@pytest.mark.parametrize("rows,cols", [(128, 64), (256, 256), (4096, 1024), (17, 9), (130, 130),
                                       (513, 40), (64, 11008 // 8), (1, 16), (16, 1)])
def test_transposed_quantise_bit_exact(q, rows, cols):
    x = oracle.fill_normal_f16(rows * cols, 7 * rows + cols).reshape(rows, cols)
    s = oracle.scale_from_amax(oracle.amax_f16(x))
    qd, sd = q.quantize_fp8_dynamic(f16_dev(x), transpose=True)
    assert sd.item() == np.float32(s)
    assert np.array_equal(qd.cpu().numpy(), oracle.quantize_fp8_f16_transpose(x, s))


@pytest.mark.parametrize("rows,hidden", [(6, 512), (3, 8), (33, 2048), (64, 8192), (5, 4096 + 256), (3, 16384 + 8), (2000, 1024)])
def test_rmsnorm_quantise_bit_exact(q, rows, hidden):
    x = oracle.fill_normal_f16(rows * hidden, oracle.SEED_A + 7).reshape(rows, hidden)
    g = oracle.fill_uniform_f16(hidden, oracle.SEED_A + 2, 0.5, 1.5)
    codes, scale = q.rmsnorm_quantize_fp8(f16_dev(x), f16_dev(g), 1e-6)
    rq, rs = oracle.rmsnorm_quantize_fp8(x, g, 1e-6)
    assert scale.item() == np.float32(rs)
    assert np.array_equal(codes.cpu().numpy(), rq)


def test_rmsnorm_matches_committed_golden(q, golden_dir):
    g = np.load(os.path.join(golden_dir, "path_small.npz"))
    R, H = g["rms_shape"]
    x = oracle.fill_normal_f16(R * H, oracle.SEED_A + 7).reshape(R, H)
    gam = oracle.fill_uniform_f16(H, oracle.SEED_A + 2, 0.5, 1.5)
    codes, scale = q.rmsnorm_quantize_fp8(f16_dev(x), f16_dev(gam), 1e-6)
    assert np.array_equal(codes.cpu().numpy(), g["rms_q"]) and scale.item() == g["rms_scale"]


def test_input_generator_matches_reference_generator(q):
    n = 100000
    got = q.fill_random_f16(n, oracle.SEED_A, index0=12345).view(torch.int16).cpu().numpy().view(np.uint16)
    ref = np.array([oracle.random_f16_bits(12345 + i, oracle.SEED_A) for i in range(0, n, 997)], np.uint16)
    assert np.array_equal(got[::997], ref)


def test_full_size_properties(q):
    # 4096 x 4096 (the fused-epilogue config's operands): scale consistency, sign
    # symmetry and idempotence of re-quantising the dequantised codes.
    x = torch.randn(4096, 4096, device="cuda", dtype=torch.float16)
    codes, s = q.quantize_fp8_dynamic(x)
    assert torch.equal(s, q.scale_from_amax(q.amax(x)))
    assert int((codes & 0x7F).max()) == 0x7E
    neg, s2 = q.quantize_fp8_dynamic(-x)
    assert torch.equal(s, s2) and torch.equal(neg ^ 0x80, codes)
    deq = codes.view(torch.float8_e4m3fn).to(torch.float32) * s
    again, s3 = q.quantize_fp8_dynamic(deq)
    assert torch.equal(again, codes)
    ct, _ = q.quantize_fp8_dynamic(x, transpose=True)
    assert torch.equal(ct, codes.t().contiguous())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_transposed_quantise_strips_at_bench_size(q, dtype):
    # 8192 x 8192 is large enough for the strip kernel to give each CTA several row tiles
    x = torch.randn(8192, 8192, device="cuda", dtype=dtype)
    codes, s = q.quantize_fp8_dynamic(x)
    ct, st = q.quantize_fp8_dynamic(x, transpose=True)
    assert torch.equal(s, st) and torch.equal(ct, codes.t().contiguous())


def test_bad_arguments_are_reported_not_launched(q):
    from y_b200._lib import YB200Error, ERR_ALIGN, ERR_SHAPE
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    with pytest.raises(YB200Error) as e:
        q.amax(x[1:])
    assert e.value.code == ERR_ALIGN
    with pytest.raises(YB200Error) as e:
        q.rmsnorm_quantize_fp8(torch.zeros(2, 12, dtype=torch.float16, device="cuda"),
                               torch.zeros(12, dtype=torch.float16, device="cuda"))
    assert e.value.code == ERR_SHAPE


@pytest.mark.parametrize("rows,hidden", [(5, 256), (3, 8), (33, 2048), (64, 4096), (16, 8192), (5, 4096 + 256),
                                         (3, 16384 + 8)])
def test_fused_add_rmsnorm_bit_exact(q, rows, hidden):
    """The reference's rmsnorm_residual_<H> kernel: Out and NewResidual, both f16."""
    x = oracle.fill_normal_f16(rows * hidden, oracle.SEED_A + 11).reshape(rows, hidden)
    r = oracle.fill_normal_f16(rows * hidden, oracle.SEED_A + 12).reshape(rows, hidden)
    w = oracle.fill_uniform_f16(hidden, oracle.SEED_A + 2, 0.5, 1.5)
    out, new_res = q.fused_add_rmsnorm(f16_dev(x), f16_dev(r), f16_dev(w), 1e-5)
    ref_out, ref_res = oracle.rmsnorm_residual_f16(x, r, w, 1e-5)
    assert np.array_equal(host_bits(new_res), ref_res)
    assert np.array_equal(host_bits(out), ref_out)
    # in place on the residual stream, as a decoder layer uses it
    rd = f16_dev(r)
    out2, nr2 = q.fused_add_rmsnorm(f16_dev(x), rd, f16_dev(w), 1e-5, new_residual=rd)
    assert nr2.data_ptr() == rd.data_ptr()
    assert np.array_equal(host_bits(rd), ref_res) and np.array_equal(host_bits(out2), ref_out)


def test_fused_add_rmsnorm_through_the_launch_api(cuda):
    """compile -> load_module('rmsnorm_residual_4096') -> launch with grid = rows."""
    from y_b200 import runtime as rt
    src = ("kernel rmsnorm_residual_4096(X: GlobalMemory<F16>, Residual: GlobalMemory<F16>, "
           "Weight: GlobalMemory<F16>, Out: GlobalMemory<F16>, NewResidual: GlobalMemory<F16>) {}")
    rows, hidden = 12, 4096
    x = oracle.fill_normal_f16(rows * hidden, 21).reshape(rows, hidden)
    r = oracle.fill_normal_f16(rows * hidden, 22).reshape(rows, hidden)
    w = oracle.fill_uniform_f16(hidden, 23, 0.5, 1.5)
    xd, rdv, wd = f16_dev(x), f16_dev(r), f16_dev(w)
    out = torch.empty_like(xd)
    nres = torch.empty_like(xd)
    ctx = rt.CudaContext.new()
    kern = ctx.load_module(rt.compile_to_ptx(src), "rmsnorm_residual_4096")
    ctx.launch(kern, (rows, 1, 1), (256, 1, 1), 0,
               [xd.data_ptr(), rdv.data_ptr(), wd.data_ptr(), out.data_ptr(), nres.data_ptr()])
    ctx.synchronize()
    ref_out, ref_res = oracle.rmsnorm_residual_f16(x, r, w, 1e-5)
    assert np.array_equal(host_bits(out), ref_out) and np.array_equal(host_bits(nres), ref_res)
    with pytest.raises(rt.YB200Error):
        ctx.launch(kern, (rows, 1, 1), (128, 1, 1), 0,
                   [xd.data_ptr(), rdv.data_ptr(), wd.data_ptr(), out.data_ptr(), nres.data_ptr()])
    kern.free()
    ctx.close()


@pytest.mark.parametrize("rows,head_dim", [(1, 64), (37, 64), (200, 128), (33, 256), (4096, 128)])
def test_rope_matches_oracle(q, rows, head_dim):
    """Same inv_freq table and the same f32 theta on both sides, so only the last bit of
    sin/cos can differ: outputs agree except for rare one-ulp f16 rounding flips."""
    x = oracle.fill_normal_f16(rows * head_dim, oracle.SEED_A + 31).reshape(rows, head_dim)
    rng = np.random.default_rng(rows + head_dim)
    pos = rng.integers(0, 4096, size=rows).astype(np.int32)
    pos[0] = 0
    pos[-1] = 4095
    out = q.rope(f16_dev(x), torch.from_numpy(pos).cuda())
    got, ref = host_bits(out), oracle.rope_f16(x, pos)
    gf, rf = got.view(np.float16).astype(np.float64), ref.view(np.float16).astype(np.float64)
    assert np.all(np.abs(gf - rf) <= np.maximum(np.abs(rf) * 2.0 ** -10, 2.0 ** -14))  # one f16 ulp
    assert (got != ref).mean() < 0.01
    assert np.array_equal(got[pos == 0], x[pos == 0])  # position 0 is the identity
    # in place
    xd = f16_dev(x)
    q.rope(xd, torch.from_numpy(pos).cuda(), out=xd)
    assert np.array_equal(host_bits(xd), got)


def test_rope_through_the_launch_api(cuda):
    from y_b200 import runtime as rt
    src = "kernel rope_128(X: GlobalMemory<F16>, Positions: GlobalMemory<I32>, Out: GlobalMemory<F16>) {}"
    rows = 50
    x = oracle.fill_normal_f16(rows * 128, 77).reshape(rows, 128)
    pos = np.arange(rows, dtype=np.int32) * 80
    xd, pd = f16_dev(x), torch.from_numpy(pos).cuda()
    out = torch.empty_like(xd)
    ctx = rt.CudaContext.new()
    kern = ctx.load_module(rt.compile_to_ptx(src), "rope_128")
    ctx.launch(kern, (rows, 1, 1), (32, 1, 1), 0, [xd.data_ptr(), pd.data_ptr(), out.data_ptr()])
    ctx.synchronize()
    from y_b200 import quant
    assert torch.equal(out, quant.rope(xd, pd))
    kern.free()
    ctx.close()
