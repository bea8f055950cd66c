"""F16-operand GEMM family against the oracle (orc_gemm_f16): the tcgen05 kind::f16 kernels on
K-major operands, the drop-ins that take the reference's row-major B, the weight-streaming
decode kernel and the reference's split-K pair, and the runtime-shape entries of the launch
API. Exact-integer operands must match bit for bit; random operands meet the GEMM tolerance."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, f16_dev, host_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


def ints_f16(shape, seed, lo=-3, hi=4):
    return np.random.default_rng(seed).integers(lo, hi, size=shape).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("m,n,k,cta_m,cta_n", [
    (128, 64, 64, 128, 64), (128, 128, 128, 128, 128), (128, 256, 64, 128, 256), (256, 256, 128, 256, 0),
    (17, 9, 8, 0, 0), (33, 17, 72, 0, 0), (130, 130, 136, 0, 0), (513, 513, 264, 0, 0),
    (300, 520, 1000, 256, 0), (1024, 768, 512, 0, 0),
])
def test_kmajor_exact_integer(q, m, n, k, cta_m, cta_n):
    a, bt = ints_f16((m, k), 1), ints_f16((n, k), 2)
    want = oracle.gemm_f16(a, bt)
    got = q.gemm_f16_kmajor(f16_dev(a), f16_dev(bt), cta_m=cta_m, cta_n=cta_n)
    q.device_status()
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("out_dtype,out_kind", [(torch.float32, oracle.OUT_F32), (torch.float16, oracle.OUT_F16),
                                                (torch.bfloat16, oracle.OUT_BF16)])
@pytest.mark.parametrize("bias_f32", [True, False])
def test_kmajor_bias_relu_out_kinds(q, out_dtype, out_kind, bias_f32):
    m, n, k = 384, 640, 320
    a = oracle.fill_normal_f16(m * k, 11).reshape(m, k)
    bt = oracle.fill_normal_f16(n * k, 12, 1.0 / 16).reshape(n, k)
    if bias_f32:
        bias = (np.random.default_rng(3).standard_normal(n) * 0.5).astype(np.float32)
        bias_d = torch.from_numpy(bias).cuda()
    else:
        bias = oracle.fill_normal_f16(n, 13, 0.5)
        bias_d = f16_dev(bias)
    want = oracle.gemm_f16(a, bt, bias=bias, epilogue=oracle.EPI_BIAS_RELU, out_kind=out_kind)
    got = q.gemm_f16_kmajor(f16_dev(a), f16_dev(bt), bias=bias_d, epilogue=q.EPI_BIAS_RELU, out_dtype=out_dtype)
    q.device_status()
    g = got.float().cpu().numpy()
    from helpers import to_f64
    assert_gemm_close(g, to_f64(want, out_kind), f"bias_relu {out_dtype}")


@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (200, 136, 128), (512, 520, 96), (1024, 1536, 512), (96, 100, 40)])
def test_rowmajor_b_drop_in(q, m, n, k):
    """gemm_f16_<tag>(A, B [K, N] row-major, C f32): the K-major copy (ragged N and K tails
    included) and the GEMM behind it."""
    a, b = ints_f16((m, k), 5), ints_f16((k, n), 6)
    want = oracle.gemm_f16(a, np.ascontiguousarray(b.T))
    got = q.gemm_f16(f16_dev(a), f16_dev(b))
    assert np.array_equal(got.cpu().numpy(), want)
    a = oracle.fill_normal_f16(m * k, 21).reshape(m, k)
    b = oracle.fill_normal_f16(k * n, 22, 1.0 / 8).reshape(k, n)
    bias = (np.random.default_rng(4).standard_normal(n)).astype(np.float32)
    want = oracle.gemm_f16(a, np.ascontiguousarray(b.T), bias=bias, epilogue=oracle.EPI_BIAS_RELU)
    got = q.gemm_f16(f16_dev(a), f16_dev(b), bias=torch.from_numpy(bias).cuda(), relu=True)
    q.device_status()
    assert_gemm_close(got.cpu().numpy(), want, f"rowmajor {m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (256, 384, 256), (100, 72, 64)])
def test_swiglu_two_weight_drop_in(q, m, n, k):
    x = oracle.fill_normal_f16(m * k, 31).reshape(m, k)
    wg = oracle.fill_normal_f16(k * n, 32, 1.0 / np.sqrt(k)).reshape(k, n)
    wu = oracle.fill_normal_f16(k * n, 33, 1.0 / np.sqrt(k)).reshape(k, n)
    inter = np.empty((2 * n, k), np.uint16)
    inter[0::2], inter[1::2] = wg.T, wu.T
    want = oracle.gemm_f16(x, inter, epilogue=oracle.EPI_SWIGLU)
    got = q.gemm_f16_swiglu(f16_dev(x), f16_dev(wg), f16_dev(wu))
    q.device_status()
    assert_gemm_close(got.cpu().numpy(), want, f"swiglu {m}x{n}x{k}")


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 32])
# (72, 112): four 32-row steps, the last one half zeros, split over a cluster of four;
# (264, 2048): a cluster of eight; (40, 144): five steps, no cluster. From 17 tokens on all of them
# run on the tcgen05 kernel: (64, 64) one K block, (72, 128) a cluster of two with a column block
# that is mostly outside the matrix, (264, 2048) a cluster of eight, (72, 112) and (40, 144) a
# last K block that reaches beyond K (zero-filled by TMA), (8, 16) a single block of 16 rows
@pytest.mark.parametrize("n,k", [(8, 16), (40, 144), (72, 112), (64, 64), (72, 128), (4096, 4096), (11008, 4096), (264, 2048)])
def test_decode_weight_streaming(q, m, n, k):
    x, w = ints_f16((m, k), 41, -2, 3), ints_f16((k, n), 42, -2, 3)
    want = oracle.gemm_f16(x, np.ascontiguousarray(w.T))
    got = q.gemm_f16_decode(f16_dev(x), f16_dev(w))
    assert np.array_equal(got.cpu().numpy(), want)
    if n >= 4096 and m in (1, 8, 32):
        x = oracle.fill_normal_f16(m * k, 43).reshape(m, k)
        w = oracle.fill_normal_f16(k * n, 44, 1.0 / 64).reshape(k, n)
        want = oracle.gemm_f16(x, np.ascontiguousarray(w.T), out_kind=oracle.OUT_F16)
        first = q.gemm_f16_decode(f16_dev(x), f16_dev(w), out_dtype=torch.float16)
        assert_gemm_close(first.float().cpu().numpy(), want.view(np.float16).astype(np.float64), f"decode {m}x{n}x{k}")
        for _ in range(3):   # fixed reduction order: repeated launches are bit-identical
            assert torch.equal(q.gemm_f16_decode(f16_dev(x), f16_dev(w), out_dtype=torch.float16), first)
    q.device_status()


def test_launch_api_entries(q):
    """The runtime-shape entries under the reference's names, and the compiled-shape families
    loaded from their descriptors."""
    from y_b200 import runtime as rt
    ctx = rt.CudaContext.new()
    m, n, k = 160, 264, 128
    a = oracle.fill_normal_f16(m * k, 51).reshape(m, k)
    b = oracle.fill_normal_f16(k * n, 52, 1.0 / 8).reshape(k, n)
    bias = oracle.fill_normal_f16(n, 53, 0.5)
    ad, bd, biasd = f16_dev(a), f16_dev(b), f16_dev(bias)
    bt = np.ascontiguousarray(b.T)
    # y_tensor_core_gemm(A, B, C f16, M, N, K)
    kern = ctx.load_module(None, "y_tensor_core_gemm")
    c = torch.empty(m, n, dtype=torch.float16, device="cuda")
    ctx.launch(kern, None, None, 0, [ad.data_ptr(), bd.data_ptr(), c.data_ptr(), ("i32", m), ("i32", n), ("i32", k)])
    ctx.synchronize()
    want = oracle.gemm_f16(a, bt, out_kind=oracle.OUT_F16).view(np.float16).astype(np.float64)
    assert_gemm_close(c.float().cpu().numpy(), want, "y_tensor_core_gemm")
    # the same entry at a decode shape goes to the weight-streaming kernel
    c8 = torch.empty(8, n, dtype=torch.float16, device="cuda")
    ctx.launch(kern, None, None, 0, [ad.data_ptr(), bd.data_ptr(), c8.data_ptr(), ("i32", 8), ("i32", n), ("i32", k)])
    ctx.synchronize()
    assert_gemm_close(c8.float().cpu().numpy(), want[:8], "y_tensor_core_gemm, M = 8")
    kern.free()
    # y_fused_gemm_bias_relu_fp16(A, B, bias f16, C f16, M, N, K, is_relu)
    kern = ctx.load_module(None, "y_fused_gemm_bias_relu_fp16")
    for relu, epi in ((1, oracle.EPI_BIAS_RELU), (0, oracle.EPI_BIAS)):
        ctx.launch(kern, None, None, 0, [ad.data_ptr(), bd.data_ptr(), biasd.data_ptr(), c.data_ptr(), ("i32", m), ("i32", n),
                                         ("i32", k), ("i32", relu)])
        ctx.synchronize()
        w = oracle.gemm_f16(a, bt, bias=bias, epilogue=epi, out_kind=oracle.OUT_F16).view(np.float16).astype(np.float64)
        assert_gemm_close(c.float().cpu().numpy(), w, f"y_fused_gemm_bias_relu_fp16 relu={relu}")
    kern.free()
    # the split-K pair: partial sums per K range, then their sum rounded to f16
    ks, mm = 4, 4
    wsp = torch.full((ks, mm, n), float("nan"), device="cuda")
    k1 = ctx.load_module(None, "y_fused_gemm_splitk_workspace")
    k2 = ctx.load_module(None, "y_splitk_reduction")
    ctx.launch(k1, None, None, 0, [ad.data_ptr(), bd.data_ptr(), wsp.data_ptr(), ("i32", mm), ("i32", n), ("i32", k), ("i32", ks)])
    c4 = torch.empty(mm, n, dtype=torch.float16, device="cuda")
    ctx.launch(k2, None, None, 0, [wsp.data_ptr(), c4.data_ptr(), ("i32", mm * n), ("i32", mm), ("i32", n), ("i32", ks)])
    ctx.synchronize()
    part = wsp.cpu().numpy()
    for s in range(ks):
        sl = slice(s * (k // ks), (s + 1) * (k // ks))
        assert_gemm_close(part[s], oracle.gemm_f16(np.ascontiguousarray(a[:mm, sl]), np.ascontiguousarray(bt[:, sl])), f"split {s}")
    ref = part[0].copy()
    for s in range(1, ks):
        ref = ref + part[s]
    assert np.array_equal(host_bits(c4), ref.astype(np.float16).view(np.uint16))
    k1.free(), k2.free()
    # FP8 runtime-shape entries with fused epilogues
    aq, sa = q.quantize_fp8_dynamic(ad)
    bqt, sb = q.quantize_fp8_dynamic(bd, transpose=True)
    kern = ctx.load_module(None, "y_fp8_gemm_bias_relu")
    cb = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.launch(kern, None, None, 0, [aq.data_ptr(), bqt.data_ptr(), biasd.data_ptr(), cb.data_ptr(), float(sa), float(sb),
                                     ("i32", m), ("i32", n), ("i32", k), ("i32", 1)])
    ctx.synchronize()
    want8 = q.gemm_fp8_codes(aq, bqt, sa, sb, bias=biasd, epilogue=q.EPI_BIAS_RELU, out_dtype=torch.bfloat16)
    assert torch.equal(cb, want8)
    kern.free()
    kern = ctx.load_module(None, "y_fp8_gemm_swiglu")
    cs = torch.empty(m, n // 2, dtype=torch.bfloat16, device="cuda")
    ctx.launch(kern, None, None, 0, [aq.data_ptr(), bqt.data_ptr(), cs.data_ptr(), float(sa), float(sb), ("i32", m), ("i32", n), ("i32", k)])
    ctx.synchronize()
    assert torch.equal(cs, q.gemm_fp8_codes(aq, bqt, sa, sb, epilogue=q.EPI_SWIGLU, out_dtype=torch.bfloat16))
    kern.free()
    # launch metadata of a descriptor kernel carries the fused-epilogue count
    image = rt.compile_to_ptx("@tile(512, 512, 512)\nkernel gemm_f16_bias_relu_512(A: GlobalMemory<F16>, B: GlobalMemory<F16>, "
                              "Bias: GlobalMemory<F32>, C: GlobalMemory<F32>) {\n}\n")
    kern = ctx.load_module(image, "gemm_f16_bias_relu_512")
    info = kern.launch_info()
    assert info.fused_epilogues == 1 and info.workspace_bytes == 512 * 512 * 2 and info.block[0] == 320
    kern.free()
    q.device_status()
    ctx.close()


def test_decode_tcgen05_tensor_map_cache_wraps(q):
    # the 17..32-token kernel keeps the tensor maps of a host thread's last 64 operands: more
    # distinct weight matrices than that, twice over, must keep giving exact results
    m, n, k = 24, 72, 128
    x = ints_f16((m, k), 51, -2, 3)
    xd = f16_dev(x)
    ws = [ints_f16((k, n), 100 + i, -2, 3) for i in range(70)]
    wd = [f16_dev(w) for w in ws]
    for _ in range(2):
        for w, d in zip(ws, wd):
            want = oracle.gemm_f16(x, np.ascontiguousarray(w.T))
            assert np.array_equal(q.gemm_f16_decode(xd, d).cpu().numpy(), want)
    q.device_status()
