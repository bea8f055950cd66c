"""Three-way parity on the GPU: the reference's own kernels, the CPU oracle, this library.

The reference's compiler output for this path exists in its tree as PTX fixtures;
oracle/make_ref.py assembles them unchanged for sm_100a into oracle/_ref/. Each test
runs one of those kernels with the launch geometry its own comments state, on the same
seeded inputs as the oracle and as this library's drop-in entry of the same name, and
compares:
  * bit for bit where the arithmetic is exact (e4m3 codes recovered through a GEMM
    against the identity, exact-integer GEMMs, the f16 residual stream);
  * by the reference's own gates elsewhere (relative L2 < 2 % for GEMMs,
    tests/test_fp8_gemm_correctness.py:208; allclose(rtol 0.02, atol 0.02) for
    RMSNorm and RoPE, tests/benchmark_y_rmsnorm_rope.py:109,183; relative L2 <= 3e-3
    for attention, tests/benchmark_y_paged_decode_attention.py:62), and by this
    build's tighter GEMM tolerance (helpers.assert_gemm_close) against the oracle.
This is what pins the oracle: a wrong reading of a formula in oracle.c would disagree
with the reference kernel here.
Skipped when oracle/_ref/ has not been built.
"""
import numpy as np
import pytest
import torch

import oracle
import ref_kernels
from helpers import assert_gemm_close, dev, f16_dev, host_bits

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_kernels.available(),
                                 reason="oracle/_ref is not built (python oracle/make_ref.py needs the reference tree)")]


@pytest.fixture(scope="module")
def ref(cuda):
    rk = ref_kernels.RefKernels()
    yield rk
    torch.cuda.synchronize()
    rk.close()


@pytest.fixture(scope="module")
def ctx(cuda):
    from y_b200 import runtime as rt
    c = rt.CudaContext.new()
    assert c is not None
    yield c
    c.close()


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


def rel_l2(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def f16_ulp_diff(a_bits, b_bits):
    """Distance in f16 representable steps (sign-magnitude bit patterns mapped to a line)."""
    def line(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7fff), u & 0x7fff)
    return np.abs(line(a_bits) - line(b_bits))


# ---------------------------------------------------------------------------------------------
# FP8 GEMM: gemm_fp8_<tag>(A f32 [M,K], B f32 [K,N], scale_a, scale_b, C f32 [M,N])
# ---------------------------------------------------------------------------------------------
FP8_YSU = ("@tile({m}, {n}, {k})\nkernel {name}(A: GlobalMemory<F32>, B: GlobalMemory<F32>, scale_a: F32, "
           "scale_b: F32, C: GlobalMemory<F32>) {{\n}}\n\nfn main() {{\n}}\n")


def run_ref_fp8(ref, name, a, b, sa, sb):
    k = ref.get(name)
    m, n, _ = k.shape
    c = torch.full((m, n), float("nan"), device="cuda")
    grid, block, smem = k.gemm_geometry()
    k.launch(grid, block, smem, [a.data_ptr(), b.data_ptr(), float(sa), float(sb), c.data_ptr()])
    torch.cuda.synchronize()
    return c.cpu().numpy()


def run_mine_fp8(ctx, name, shape, a, b, sa, sb):
    from y_b200 import runtime as rt
    m, n, k = shape
    image = rt.compile_to_ptx(FP8_YSU.format(m=m, n=n, k=k, name=name))
    kern = ctx.load_module(image, name)
    c = torch.full((m, n), float("nan"), device="cuda")
    ctx.launch(kern, None, None, 0, [a.data_ptr(), b.data_ptr(), float(sa), float(sb), c.data_ptr()])
    ctx.synchronize()
    kern.free()
    return c.cpu().numpy()


def probe_values(count, scale, seed):
    """f32 inputs that exercise the quantiser: every midpoint between adjacent e4m3 values
    (and its two f32 neighbours) times `scale`, values beyond +-448 * scale, tiny values in the
    subnormal range, and seeded normals for the rest."""
    codes = np.arange(256, dtype=np.uint8)
    vals = oracle.decode_e4m3(codes)
    pos = np.sort(vals[np.isfinite(vals) & (vals >= 0)])
    mids = ((pos[:-1].astype(np.float64) + pos[1:].astype(np.float64)) / 2).astype(np.float32)
    special = np.concatenate([mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
                              np.float32([448, 449, 464, 465, 480, 1000, 1e4, 1e-3, 2e-3, 9.7e-4, 0.0])])
    special = np.concatenate([special, -special]).astype(np.float32) * np.float32(scale)
    rng = np.random.default_rng(seed)
    out = (rng.standard_normal(count) * 3.0).astype(np.float32)
    out[:special.size] = special
    return out


@pytest.mark.parametrize("name", ["gemm_fp8_256", "gemm_fp8_512", "gemm_fp8_1024"])
def test_fp8_quantiser_codes_recovered_through_the_reference_gemm(ref, ctx, name):
    """C = (sa * 1) * (q(A) @ I) returns every code of A dequantised, exactly: one nonzero
    product per sum. The same with A = I recovers B's codes. Pins e4m3 round-to-nearest-even,
    saturation at +-448, `x * (1 / scale)` and the byte order of the packed operands against
    the reference kernel itself (src/ptx_emitter.rs:2595-2658, 3405-3408)."""
    m, n, k = ref.get(name).shape
    assert m == n == k
    eye = torch.eye(k, device="cuda")
    # 0.25 and 2.0 are exact in binary: x * (1 / scale) lands exactly on the ties, so
    # round-half-to-even itself is what is compared; the other two scales exercise 1 / scale.
    for side, scale in (("A", 0.0123), ("A", 0.25), ("B", 0.31), ("B", 2.0)):
        vals = probe_values(m * k, scale, seed=7 if side == "A" else 8).reshape(m, k)
        x = torch.from_numpy(vals).cuda()
        want = oracle.decode_e4m3(oracle.quantize_fp8_f32(vals, scale)) * np.float32(np.float32(scale) * np.float32(1.0))
        if side == "A":
            got_ref = run_ref_fp8(ref, name, x, eye, scale, 1.0)
            got_mine = run_mine_fp8(ctx, name, (m, n, k), x, eye, scale, 1.0)
        else:
            got_ref = run_ref_fp8(ref, name, eye, x, 1.0, scale)
            got_mine = run_mine_fp8(ctx, name, (m, n, k), eye, x, 1.0, scale)
        assert np.array_equal(got_ref, want), f"{name}: reference kernel's {side} codes differ from the oracle's"
        assert np.array_equal(got_mine, want), f"{name}: this library's {side} codes differ from the oracle's"


@pytest.mark.parametrize("name", ["gemm_fp8_256", "gemm_fp8_512", "gemm_fp8_1024"])
def test_fp8_exact_integer_gemm_is_bit_identical_three_ways(ref, ctx, name):
    m, n, k = ref.get(name).shape
    rng = np.random.default_rng(11)
    a = rng.integers(-4, 5, size=(m, k)).astype(np.float32)
    b = rng.integers(-4, 5, size=(k, n)).astype(np.float32)
    want = oracle.gemm_fp8(oracle.quantize_fp8_f32(a, 1.0), np.ascontiguousarray(oracle.quantize_fp8_f32(b, 1.0).T), 1.0, 1.0)
    assert np.array_equal(want, (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32))
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    assert np.array_equal(run_ref_fp8(ref, name, ad, bd, 1.0, 1.0), want)
    assert np.array_equal(run_mine_fp8(ctx, name, (m, n, k), ad, bd, 1.0, 1.0), want)


@pytest.mark.parametrize("name", ["gemm_fp8_256", "gemm_fp8_512", "gemm_fp8_1024"])
def test_fp8_gemm_random_inputs_meet_the_reference_gate(ref, ctx, name):
    """The reference's own test: randn * 3, scale = amax / 448, relative L2 < 2 %
    (tests/test_fp8_gemm_correctness.py:92-100, 208); plus this build's tolerance against the
    oracle for both kernels."""
    m, n, k = ref.get(name).shape
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    a = torch.randn(m, k, device="cuda", generator=g) * 3.0
    b = torch.randn(k, n, device="cuda", generator=g) * 3.0
    sa = max(float(a.abs().max()) / 448.0, 1e-12)
    sb = max(float(b.abs().max()) / 448.0, 1e-12)
    an, bn = a.cpu().numpy(), b.cpu().numpy()
    want = oracle.gemm_fp8(oracle.quantize_fp8_f32(an, sa), np.ascontiguousarray(oracle.quantize_fp8_f32(bn, sb).T), sa, sb)
    got_ref = run_ref_fp8(ref, name, a, b, sa, sb)
    got_mine = run_mine_fp8(ctx, name, (m, n, k), a, b, sa, sb)
    assert rel_l2(got_mine, got_ref) < 2e-2
    assert_gemm_close(got_ref, want, f"{name}: reference kernel vs oracle")
    assert_gemm_close(got_mine, want, f"{name}: this library vs oracle")
    # in practice the three agree far inside the gate: same codes, f32 sums in different orders
    assert rel_l2(got_ref, want) < 1e-5 and rel_l2(got_mine, want) < 1e-5


def test_fp8_reference_kernel_is_deterministic_over_repeated_launches(ref):
    name = "gemm_fp8_256"
    m, n, k = ref.get(name).shape
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    a = torch.randn(m, k, device="cuda", generator=g) * 3.0
    b = torch.randn(k, n, device="cuda", generator=g) * 3.0
    first = run_ref_fp8(ref, name, a, b, 0.03, 0.03)
    for _ in range(5):
        assert np.array_equal(run_ref_fp8(ref, name, a, b, 0.03, 0.03), first)


# ---------------------------------------------------------------------------------------------
# F16 GEMM family: (A f16 [M,K], B f16 [K,N][, Bias f32 [N]], C f32 [M,N]); SwiGLU (X, Wgate, Wup, Out)
# ---------------------------------------------------------------------------------------------
F16_YSU = {
    "gemm_f16": "@tile({m}, {n}, {k})\nkernel {name}(A: GlobalMemory<F16>, B: GlobalMemory<F16>, C: GlobalMemory<F32>) {{\n}}\n",
    "gemm_f16_bias_relu": ("@tile({m}, {n}, {k})\nkernel {name}(A: GlobalMemory<F16>, B: GlobalMemory<F16>, "
                           "Bias: GlobalMemory<F32>, C: GlobalMemory<F32>) {{\n}}\n"),
    "gemm_f16_swiglu": ("@tile({m}, {n}, {k})\nkernel {name}(X: GlobalMemory<F16>, Wgate: GlobalMemory<F16>, "
                        "Wup: GlobalMemory<F16>, Out: GlobalMemory<F32>) {{\n}}\n"),
}


def f16_inputs(m, n, k, seed, integer=False, w_std=None):
    if integer:
        rng = np.random.default_rng(seed)
        a = rng.integers(-3, 4, size=(m, k)).astype(np.float16).view(np.uint16)
        b = rng.integers(-3, 4, size=(k, n)).astype(np.float16).view(np.uint16)
        return a, b
    a = oracle.fill_normal_f16(m * k, oracle.SEED_A + seed).reshape(m, k)
    b = oracle.fill_normal_f16(k * n, oracle.SEED_B + seed, w_std if w_std is not None else 1.0).reshape(k, n)
    return a, b


def run_ref_f16(ref, name, ptr_args, m, n):
    kr = ref.get(name)
    c = torch.full((m, n), float("nan"), device="cuda")
    grid, block, smem = kr.gemm_geometry()
    kr.launch(grid, block, smem, [*ptr_args, c.data_ptr()])
    torch.cuda.synchronize()
    return c.cpu().numpy()


def run_mine_f16(ctx, family, entry, shape, ptr_args):
    from y_b200 import runtime as rt
    m, n, k = shape
    image = rt.compile_to_ptx(F16_YSU[family].format(m=m, n=n, k=k, name=entry))
    kern = ctx.load_module(image, entry)
    c = torch.full((m, n), float("nan"), device="cuda")
    ctx.launch(kern, None, None, 0, [*ptr_args, c.data_ptr()])
    ctx.synchronize()
    kern.free()
    return c.cpu().numpy()


@pytest.mark.parametrize("name", ["gemm_f16_256", "gemm_f16_512", "tensor_core_gemm_f16_rect",
                                  "gemm_f16_decode_m1", "gemm_f16_decode_m4", "gemm_f16_decode_m8", "gemm_f16_decode_m32"])
@pytest.mark.parametrize("integer", [True, False])
def test_f16_gemm_three_ways(ref, ctx, name, integer):
    kr = ref.get(name)
    m, n, k = kr.shape
    a, b = f16_inputs(m, n, k, seed=len(name), integer=integer, w_std=None if integer else 1.0 / 64)
    want = oracle.gemm_f16(a, np.ascontiguousarray(b.T))
    ad, bd = f16_dev(a), f16_dev(b)
    got_ref = run_ref_f16(ref, name, [ad.data_ptr(), bd.data_ptr()], m, n)
    got_mine = run_mine_f16(ctx, "gemm_f16", kr.meta["entry"], (m, n, k), [ad.data_ptr(), bd.data_ptr()])
    if integer:
        assert np.array_equal(got_ref, want) and np.array_equal(got_mine, want)
    else:
        assert rel_l2(got_mine, got_ref) < 2e-2
        assert_gemm_close(got_ref, want, f"{name}: reference kernel vs oracle")
        assert_gemm_close(got_mine, want, f"{name}: this library vs oracle")


@pytest.mark.parametrize("name", ["gemm_f16_bias_relu_64", "gemm_f16_bias_relu_512"])
def test_f16_bias_relu_three_ways(ref, ctx, name):
    kr = ref.get(name)
    m, n, k = kr.shape
    a, b = f16_inputs(m, n, k, seed=5, w_std=1.0 / 16)
    bias = (np.random.default_rng(9).standard_normal(n) * 0.5).astype(np.float32)
    want = oracle.gemm_f16(a, np.ascontiguousarray(b.T), bias=bias, epilogue=oracle.EPI_BIAS_RELU)
    assert (want == 0).mean() > 0.2          # the ReLU clamps a good share of the outputs
    ad, bd, biasd = f16_dev(a), f16_dev(b), torch.from_numpy(bias).cuda()
    args = [ad.data_ptr(), bd.data_ptr(), biasd.data_ptr()]
    got_ref = run_ref_f16(ref, name, args, m, n)
    got_mine = run_mine_f16(ctx, "gemm_f16_bias_relu", kr.meta["entry"], (m, n, k), args)
    assert rel_l2(got_mine, got_ref) < 2e-2
    assert_gemm_close(got_ref, want, f"{name}: reference kernel vs oracle")
    assert_gemm_close(got_mine, want, f"{name}: this library vs oracle")
    # exact zeros agree except where the pre-activation sits within rounding of zero
    assert ((got_ref == 0) != (want == 0)).mean() < 1e-3 and ((got_mine == 0) != (want == 0)).mean() < 1e-3


def test_f16_swiglu_three_ways(ref, ctx):
    """Out = silu(X @ Wgate) * (X @ Wup) with weights ~ N(0, 1/K) as the reference's benchmark
    draws them (tests/benchmark_y_swiglu_gemm.py:120-127). Pins the SwiGLU formula of the oracle
    (src/ptx_emitter.rs:5537-5552) against the reference kernel."""
    name = "gemm_f16_swiglu_512"
    kr = ref.get(name)
    m, n, k = kr.shape
    x = oracle.fill_normal_f16(m * k, oracle.SEED_A + 21).reshape(m, k)
    wg = oracle.fill_normal_f16(k * n, oracle.SEED_B + 21, 1.0 / np.sqrt(k)).reshape(k, n)
    wu = oracle.fill_normal_f16(k * n, oracle.SEED_B + 22, 1.0 / np.sqrt(k)).reshape(k, n)
    inter = np.empty((2 * n, k), np.uint16)           # the oracle takes gate | up interleaved, K-major
    inter[0::2], inter[1::2] = wg.T, wu.T
    want = oracle.gemm_f16(x, inter, epilogue=oracle.EPI_SWIGLU)
    xd, wgd, wud = f16_dev(x), f16_dev(wg), f16_dev(wu)
    args = [xd.data_ptr(), wgd.data_ptr(), wud.data_ptr()]
    got_ref = run_ref_f16(ref, name, args, m, n)
    got_mine = run_mine_f16(ctx, "gemm_f16_swiglu", kr.meta["entry"], (m, n, k), args)
    # silu through ex2.approx / rcp.approx in the reference kernel: relative L2, its own gate
    assert rel_l2(got_ref, want) < 2e-3, rel_l2(got_ref, want)
    assert rel_l2(got_mine, want) < 2e-3, rel_l2(got_mine, want)
    assert rel_l2(got_mine, got_ref) < 2e-3
    assert_gemm_close(got_mine, want, "swiglu: this library vs oracle")
    assert_gemm_close(got_ref, want, "swiglu: reference kernel vs oracle")


def test_f16_launch_geometry_parser_reads_the_reference_comments(ref):
    """y_parse_launch_config on the emitter's real comment lines gives the geometry the
    reference's launchers derive from them."""
    import ctypes as C

    from y_b200._lib import check, lib
    for name in ("gemm_f16_512", "gemm_f16_decode_m8", "gemm_f16_bias_relu_64", "tensor_core_gemm_f16_rect"):
        kr = ref.get(name)
        m, n, _ = kr.shape
        out = (C.c_uint32 * 4)()
        check(lib.y_parse_launch_config(kr.text.encode(), m, n, out))
        grid, block, smem = kr.gemm_geometry()
        assert (out[0], out[1], out[2], out[3]) == (grid[0], grid[1], block[0], smem)


# ---------------------------------------------------------------------------------------------
# fused add + RMSNorm, RoPE, paged decode attention
# ---------------------------------------------------------------------------------------------
def test_rmsnorm_residual_three_ways(ref, q):
    rows, hidden = 96, 4096
    x = oracle.fill_normal_f16(rows * hidden, 41).reshape(rows, hidden)
    res = oracle.fill_normal_f16(rows * hidden, 42).reshape(rows, hidden)
    w = oracle.fill_uniform_f16(hidden, 43, 0.5, 1.5)
    want_out, want_res = oracle.rmsnorm_residual_f16(x, res, w, 1e-5)
    xd, rd, wd = f16_dev(x), f16_dev(res), f16_dev(w)
    out = torch.zeros(rows, hidden, dtype=torch.float16, device="cuda")
    new_res = torch.zeros_like(out)
    kr = ref.get("rmsnorm_residual_4096")
    kr.launch((rows, 1, 1), (256, 1, 1), 0, [xd.data_ptr(), rd.data_ptr(), wd.data_ptr(), out.data_ptr(), new_res.data_ptr()])
    torch.cuda.synchronize()
    ref_out, ref_res = host_bits(out), host_bits(new_res)
    mine_out_t, mine_res_t = q.fused_add_rmsnorm(xd, rd, wd, 1e-5)
    mine_out, mine_res = host_bits(mine_out_t), host_bits(mine_res_t)
    # the residual stream is one f32 add rounded to f16: exact in all three
    assert np.array_equal(ref_res, want_res) and np.array_equal(mine_res, want_res)
    assert np.array_equal(mine_out, want_out)                       # fixed reduction order: bit-exact with the oracle
    # the reference kernel uses rsqrt.approx and its own reduction order: rare one-step f16 differences
    d = f16_ulp_diff(ref_out, want_out)
    assert d.max() <= 2, d.max()
    assert (d != 0).mean() < 0.02, (d != 0).mean()
    a, b = ref_out.view(np.float16).astype(np.float64), want_out.view(np.float16).astype(np.float64)
    assert np.all(np.abs(a - b) <= 0.02 + 0.02 * np.abs(b))         # the reference's own gate


@pytest.mark.parametrize("head_dim", [64, 128, 256])
def test_rope_three_ways(ref, q, head_dim):
    rows = 512
    x = oracle.fill_normal_f16(rows * head_dim, 51 + head_dim).reshape(rows, head_dim)
    pos = np.random.default_rng(head_dim).integers(0, 4096, size=rows).astype(np.int32)
    pos[:4] = [0, 1, 4095, 2048]
    want = oracle.rope_f16(x, pos)
    xd, pd = f16_dev(x), torch.from_numpy(pos).cuda()
    out = torch.zeros(rows, head_dim, dtype=torch.float16, device="cuda")
    ref.get(f"rope_{head_dim}").launch((rows, 1, 1), (32, 1, 1), 0, [xd.data_ptr(), pd.data_ptr(), out.data_ptr()])
    torch.cuda.synchronize()
    got_ref = host_bits(out).view(np.float16).astype(np.float64)
    got_mine = host_bits(q.rope(xd, pd)).view(np.float16).astype(np.float64)
    w = want.view(np.float16).astype(np.float64)
    # the reference's own gate (sin.approx / cos.approx / ex2.approx on the device)
    assert np.all(np.abs(got_ref - w) <= 0.02 + 0.02 * np.abs(w))
    assert np.all(np.abs(got_mine - w) <= 0.02 + 0.02 * np.abs(w))
    # (sin.approx loses absolute accuracy as theta grows towards 4095 rad; the kernel here
    # reduces the argument first)
    assert rel_l2(got_ref, w) < 5e-3 and rel_l2(got_mine, w) < 1e-3 and rel_l2(got_mine, got_ref) < 5e-3
    assert np.array_equal(got_ref[0], x[0].view(np.float16).astype(np.float64))     # position 0: identity


@pytest.mark.parametrize("name,warps", [("paged_decode_attention_128_32_8_16", 32),
                                        ("paged_decode_attention_128_32_8_16_8", 8)])
def test_paged_decode_attention_three_ways(ref, q, name, warps):
    """The reference's own correctness batch shapes (tests/benchmark_y_paged_decode_attention.py:284-294)."""
    hd, hq, hkv, ps = 128, 32, 8, 16
    for seq_lens in ([0, 1, 7, 63, 64, 65, 200, 33], [1000, 4095, 2, 2048]):
        ns = len(seq_lens)
        rng = np.random.default_rng(ns + seq_lens[0])
        max_pages = max(1, max((x + ps - 1) // ps for x in seq_lens))
        num_pages = 512
        qv = oracle.fill_normal_f16(ns * hq * hd, 61).reshape(ns, hq, hd)
        kc = oracle.fill_normal_f16(num_pages * ps * hkv * hd, 62).reshape(num_pages, ps, hkv, hd)
        vc = oracle.fill_normal_f16(num_pages * ps * hkv * hd, 63).reshape(num_pages, ps, hkv, hd)
        pt = np.stack([rng.permutation(num_pages)[:max_pages] for _ in range(ns)]).astype(np.int32)
        sl = np.array(seq_lens, np.int32)
        want = oracle.paged_decode_attention(qv, kc, vc, pt, sl).view(np.float16).astype(np.float64)
        qd, kd, vd = f16_dev(qv), f16_dev(kc), f16_dev(vc)
        ptd, sld = torch.from_numpy(pt).cuda(), torch.from_numpy(sl).cuda()
        out = torch.zeros(ns, hq, hd, dtype=torch.float16, device="cuda")
        ref.get(name).launch((hq, ns, 1), (warps * 32, 1, 1), 0,
                             [qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ptd.data_ptr(), sld.data_ptr(),
                              out.data_ptr(), ("i32", max_pages)])
        torch.cuda.synchronize()
        got_ref = host_bits(out).view(np.float16).astype(np.float64)
        got_mine = host_bits(q.paged_decode_attention(qd, kd, vd, ptd, sld)).view(np.float16).astype(np.float64)
        assert rel_l2(got_ref, want) <= 3e-3, rel_l2(got_ref, want)       # the reference's gate
        assert rel_l2(got_mine, want) < 2e-3 and rel_l2(got_mine, got_ref) <= 3e-3
        for s, length in enumerate(seq_lens):
            if length == 0:
                assert not got_ref[s].any() and not got_mine[s].any()
    q.device_status()
