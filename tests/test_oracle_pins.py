"""Pins the CPU oracle: the reference's own known-answer tests, torch's CPU e4m3
conversion, NVIDIA's host conversion in cuda_fp8.h, and the committed golden vectors."""
import os

import numpy as np
import pytest

import oracle


# ---- reference known-answer tests ----------------------------------------------
def test_f16_decode_matches_known_values():
    # src/cuda_runtime.rs:688-695
    assert oracle.f16_bits_to_f32(0x3C00) == 1.0
    assert oracle.f16_bits_to_f32(0xC000) == -2.0
    assert oracle.f16_bits_to_f32(0x3800) == 0.5


def test_generated_f16_is_always_a_bounded_normal():
    # src/cuda_runtime.rs:697-705
    bits = oracle.fill_random_f16(10_000, 0x5EED_5EED)
    exp = (bits >> 10) & 0x1F
    assert exp.min() >= 12 and exp.max() <= 14
    v = np.abs(bits.view(np.float16).astype(np.float32))
    assert v.min() >= 0.125 and v.max() < 1.0
    assert bits[0] == oracle.random_f16_bits(0, 0x5EED_5EED)


def test_splitmix64_matches_the_published_sequence():
    # splitmix64 with state = seed + (index + 1) * golden gamma; seed 0 gives the
    # sequence every splitmix64 implementation documents.
    assert oracle.splitmix64(0, 0) == 0xE220A8397B1DCDAF
    assert oracle.splitmix64(1, 0) == 0x6E789E6AA1B965F4
    assert oracle.splitmix64(2, 0) == 0x06C45D188009454F


def test_block_cdiv_values():
    # tests/test_rust_triton_parity.rs:62-63, src/c_api.rs:196-201
    assert oracle.block_cdiv(10, 3) == 4
    assert oracle.block_cdiv(100, 32) == 4
    assert oracle.block_cdiv(7, 0) == 0


def test_grid_swizzle_is_a_bijection_on_every_reference_grid():
    # src/ptx_emitter.rs:7477-7513
    grids = [(8, 8), (16, 16), (32, 32), (64, 64), (4, 5), (5, 4), (7, 13), (13, 7), (3, 17),
             (16, 24), (24, 16), (1, 1), (1, 7), (7, 1), (2, 3), (64, 4), (4, 64)]
    for gx, gy in grids:
        for group in (2, 4, 8, 16):
            seen = set()
            for by in range(gy):
                for bx in range(gx):
                    n, m = oracle.grid_swizzle(bx, by, gx, gy, group)
                    assert m < gy and n < gx
                    seen.add((n, m))
            assert len(seen) == gx * gy


# ---- e4m3 codec ------------------------------------------------------------------
def test_e4m3_matches_torch_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "e4m3_torch.npz"))
    x, codes, table = g["x"], g["codes"], g["decode_table"]
    mine = np.array([oracle.e4m3_encode(float(v)) for v in x], np.uint8)
    assert np.array_equal(mine, codes)
    dec = np.array([oracle.e4m3_decode(c) for c in range(256)], np.float32)
    ok = (dec == table) | (np.isnan(dec) & np.isnan(table))
    assert ok.all()


def test_e4m3_matches_cuda_fp8_host_conversion():
    pin = oracle.load_pin()
    rng = np.random.default_rng(7)
    vals = list((rng.standard_normal(20000) * 200).astype(np.float32))
    vals += [448.0, 449.0, 464.0, 465.0, 480.0, 1e9, float("inf"), -float("inf"), 0.0, -0.0,
             2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10, 1e-10]
    for c in range(0x7E):
        lo, hi = oracle.e4m3_decode(c), oracle.e4m3_decode(c + 1)
        vals += [lo, hi, (lo + hi) / 2, -(lo + hi) / 2]
    for v in vals:
        assert oracle.e4m3_encode(float(v)) == pin.pin_nv_e4m3_encode(float(v)), v
    for c in range(256):
        a, b = oracle.e4m3_decode(c), pin.pin_nv_e4m3_decode(c)
        assert a == b or (a != a and b != b)


def test_e4m3_saturates_and_round_trips():
    assert oracle.e4m3_encode(1e9) == 0x7E and oracle.e4m3_encode(-1e9) == 0xFE
    assert oracle.e4m3_encode(float("inf")) == 0x7E
    assert oracle.e4m3_encode(float("nan")) & 0x7F == 0x7F
    for c in list(range(0x7F)) + list(range(0x80, 0xFF)):
        assert oracle.e4m3_encode(oracle.e4m3_decode(c)) == (c if c != 0x80 else 0x80)


def test_f16_and_bf16_rounding_match_numpy_and_torch():
    import torch

    rng = np.random.default_rng(3)
    x = (rng.standard_normal(50000) * np.exp(rng.uniform(-20, 11, 50000))).astype(np.float32)
    mine = np.array([oracle.f32_to_f16_bits(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        assert np.array_equal(mine, x.astype(np.float16).view(np.uint16))
    bm = np.array([oracle.f32_to_bf16_bits(float(v)) for v in x], np.uint16)
    assert np.array_equal(bm, torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy())
    allh = np.arange(65536, dtype=np.uint16)
    d = np.array([oracle.f16_bits_to_f32(int(h)) for h in allh[::7]], np.float32)
    r = allh[::7].view(np.float16).astype(np.float32)
    assert ((d == r) | (np.isnan(d) & np.isnan(r))).all()


# ---- quantiser semantics ----------------------------------------------------------
def test_quantise_is_multiply_by_reciprocal_then_round():
    import torch

    x = oracle.fill_normal_f16(4096, 11)
    amax = oracle.amax_f16(x)
    scale = oracle.scale_from_amax(amax)
    assert scale == np.float32(max(np.float32(amax) / np.float32(448.0), np.float32(1e-12)))
    q = oracle.quantize_fp8_f16(x, scale)
    inv = np.float32(1.0) / np.float32(scale)
    prod = x.view(np.float16).astype(np.float32) * inv
    ref = torch.from_numpy(prod).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(q, ref)
    assert q.max() & 0x7F <= 0x7E
    assert (q & 0x7F).max() == 0x7E  # the largest element lands on +-448
    assert oracle.scale_from_amax(0.0) == np.float32(1e-12)
    qt = oracle.quantize_fp8_f16_transpose(x.reshape(64, 64), scale)
    assert np.array_equal(qt, q.reshape(64, 64).T)


def test_int4_format():
    K, N = 256, 32
    w = oracle.fill_normal_f16(K * N, 5, 0.05).reshape(K, N)
    w[128:, 3] = 0  # an all-zero group
    qw, sc = oracle.int4_quantize(w)
    wf = w.view(np.float16).astype(np.float32)
    s = sc.view(np.float16).astype(np.float32)
    amax = np.abs(wf).reshape(2, 128, N).max(axis=1)
    assert np.array_equal(sc.view(np.float16), (amax / np.float32(7)).astype(np.float16))
    nib = np.stack([(qw >> (4 * j)) & 0xF for j in range(8)], axis=1).reshape(K, N).astype(np.int32)
    q = np.where(nib >= 8, nib - 16, nib)
    assert q.min() >= -8 and q.max() <= 7
    srep = np.repeat(s, 128, axis=0)
    with np.errstate(divide="ignore", invalid="ignore"):
        expect = np.where(srep > 0, np.clip(np.rint(wf / srep), -8, 7), 0).astype(np.int32)
    assert np.array_equal(q, expect)
    assert (q[128:, 3] == 0).all() and sc[1, 3] == 0
    stream = oracle.int4_repack(qw, sc)
    assert stream.size == oracle.int4_stream_bytes(K, N) == (N // 16) * (K // 128) * 1056
    # spot-check the streaming layout against its written definition
    pos = [0, 4, 1, 5, 2, 6, 3, 7]
    words = stream.view(np.uint32)
    for (t, g, h, lane, i) in [(0, 0, 0, 0, 0), (1, 1, 1, 31, 3), (1, 0, 0, 13, 2), (0, 1, 1, 6, 1)]:
        gq, c = lane // 4, lane % 4
        word = int(words[((t * 2 + g) * 1056) // 4 + h * 128 + lane * 4 + i])
        col = 16 * t + gq + 8 * (i % 2)
        k0 = 128 * g + 32 * (2 * h + i // 2) + 8 * c
        for j in range(8):
            assert ((word >> (4 * pos[j])) & 0xF) == q[k0 + j, col] + 8
    blk = stream[1056 * 3:1056 * 4]
    assert np.array_equal(blk[1024:].view(np.uint16), sc[1, 16:32])


def test_int4_decode_oracle_matches_dequantised_matmul():
    K, N, M = 256, 32, 5
    w = oracle.fill_normal_f16(K * N, 5, 0.05).reshape(K, N)
    x = oracle.fill_normal_f16(M * K, 6).reshape(M, K)
    qw, sc = oracle.int4_quantize(w)
    out = oracle.gemm_int4_decode(x, qw, sc).view(np.float16).astype(np.float64)
    nib = np.stack([(qw >> (4 * j)) & 0xF for j in range(8)], axis=1).reshape(K, N).astype(np.int32)
    q = np.where(nib >= 8, nib - 16, nib).astype(np.float64)
    wd = q * np.repeat(sc.view(np.float16).astype(np.float64), 128, axis=0)
    ref = x.view(np.float16).astype(np.float64) @ wd
    assert np.abs(out - ref).max() <= 2e-3 * np.abs(ref).max() + 1e-3


def test_gemm_oracle_matches_float64_matmul_and_epilogues():
    M, N, K = 16, 24, 64
    a = oracle.fill_normal_f16(M * K, 1).reshape(M, K)
    b = oracle.fill_normal_f16(K * N, 2).reshape(K, N)
    sa, sb = oracle.scale_from_amax(oracle.amax_f16(a)), oracle.scale_from_amax(oracle.amax_f16(b))
    aq, bqt = oracle.quantize_fp8_f16(a, sa), oracle.quantize_fp8_f16_transpose(b, sb)
    ref = (oracle.e4m3_decode_array(aq).astype(np.float64) @
           oracle.e4m3_decode_array(bqt).astype(np.float64).T) * (np.float32(sa) * np.float32(sb))
    c = oracle.gemm_fp8(aq, bqt, sa, sb)
    assert np.abs(c - ref).max() <= 1e-5 * np.abs(ref).max()
    bias = oracle.fill_normal_f16(N, 3, 0.1)
    cb = oracle.gemm_fp8(aq, bqt, sa, sb, bias=bias, epilogue=oracle.EPI_BIAS_RELU)
    refb = np.maximum(ref + bias.view(np.float16).astype(np.float64), 0)
    assert np.abs(cb - refb).max() <= 1e-5 * np.abs(refb).max() + 1e-6
    h = oracle.gemm_fp8(aq, bqt, sa, sb, epilogue=oracle.EPI_SWIGLU)
    g, u = ref[:, 0::2], ref[:, 1::2]
    refh = g / (1 + np.exp(-g)) * u
    assert h.shape == (M, N // 2)
    assert np.abs(h - refh).max() <= 1e-5 * np.abs(refh).max() + 1e-6
    part = oracle.gemm_fp8(aq, bqt, sa, sb, row_begin=5, row_count=4)
    assert np.array_equal(part, c[5:9])
    # the reference's GELU (its coefficients as emitted, src/quantization_pass.rs:748-796) and SiLU
    x = ref / 64 + bias.view(np.float16).astype(np.float64)
    cg = oracle.gemm_fp8(aq, bqt, sa / 8, sb / 8, bias=bias, epilogue=oracle.EPI_BIAS_GELU)
    refg = 0.5 * x * (1 + np.tanh(x * (0.79788456 + 0.044715 * x * x)))
    assert np.abs(cg - refg).max() <= 1e-5 * np.abs(refg).max() + 1e-6
    cs = oracle.gemm_fp8(aq, bqt, sa / 8, sb / 8, bias=bias, epilogue=oracle.EPI_BIAS_SILU)
    assert np.abs(cs - x / (1 + np.exp(-x))).max() <= 1e-5 * np.abs(x).max() + 1e-6
    x0 = ref / 64
    c0 = oracle.gemm_fp8(aq, bqt, sa / 8, sb / 8, epilogue=oracle.EPI_BIAS_SILU)      # no bias given
    assert np.abs(c0 - x0 / (1 + np.exp(-x0))).max() <= 1e-5 * np.abs(x0).max() + 1e-6


def test_rmsnorm_oracle():
    R, H = 4, 1024
    x = oracle.fill_normal_f16(R * H, 21).reshape(R, H)
    g = oracle.fill_uniform_f16(H, 22, 0.5, 1.5)
    y, rstd, amax = oracle.rmsnorm_f16(x, g, 1e-6)
    xf, gf = x.view(np.float16).astype(np.float64), g.view(np.float16).astype(np.float64)
    ref = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-6) * gf
    assert np.abs(y - ref).max() <= 1e-5
    assert amax == np.abs(y).max()
    q, s = oracle.rmsnorm_quantize_fp8(x, g, 1e-6)
    assert s == oracle.scale_from_amax(amax)
    assert np.array_equal(q, oracle.quantize_fp8_f32(y, s))
    gf16 = g.view(np.float16).astype(np.float32)
    assert gf16.min() >= 0.5 and gf16.max() <= 1.5


def test_committed_path_vectors_still_hold(golden_dir):
    g = np.load(os.path.join(golden_dir, "path_small.npz"))
    M, N, K = g["gemm_shape"]
    a = oracle.fill_normal_f16(M * K, oracle.SEED_A).reshape(M, K)
    b = oracle.fill_normal_f16(K * N, oracle.SEED_B).reshape(K, N)
    sa = oracle.scale_from_amax(oracle.amax_f16(a))
    sb = oracle.scale_from_amax(oracle.amax_f16(b))
    assert np.float32(sa) == g["scale_a"] and np.float32(sb) == g["scale_b"]
    aq, bqt = oracle.quantize_fp8_f16(a, sa), oracle.quantize_fp8_f16_transpose(b, sb)
    assert np.array_equal(aq, g["aq"]) and np.array_equal(bqt, g["bqt"])
    assert np.array_equal(oracle.gemm_fp8(aq, bqt, sa, sb), g["c_f32"])
    h = oracle.gemm_fp8(aq, bqt, sa, sb, epilogue=oracle.EPI_SWIGLU, out_kind=oracle.OUT_BF16)
    assert np.array_equal(h, g["h_swiglu_bf16"])
    q, s = oracle.requant_bf16_fp8(h)
    assert np.array_equal(q, g["swiglu_q"]) and np.float32(s) == g["swiglu_scale"]
    M4, N4, K4 = g["int4_shape"]
    w = oracle.fill_normal_f16(K4 * N4, oracle.SEED_B + 3, 1.0 / 16.0).reshape(K4, N4)
    qw, sc = oracle.int4_quantize(w)
    assert np.array_equal(qw, g["int4_qweight"]) and np.array_equal(sc, g["int4_scales"])
    assert np.array_equal(oracle.int4_repack(qw, sc), g["int4_stream"])


def test_fused_add_rmsnorm_restatement_against_float64():
    """orc_rmsnorm_residual_f16 against the formula in float64: both outputs are within one
    f16 rounding of it, and NewResidual is exactly the f16 rounding of the f32 sum."""
    rows, hidden = 7, 768
    x = oracle.fill_normal_f16(rows * hidden, 5).reshape(rows, hidden)
    r = oracle.fill_normal_f16(rows * hidden, 6).reshape(rows, hidden)
    w = oracle.fill_uniform_f16(hidden, 7, 0.5, 1.5)
    out, new_res = oracle.rmsnorm_residual_f16(x, r, w, 1e-5)
    xf, rf, wf = (a.view(np.float16).astype(np.float64) for a in (x, r, w))
    h = xf + rf
    ref = h / np.sqrt((h * h).mean(axis=1, keepdims=True) + 1e-5) * wf
    got = out.view(np.float16).astype(np.float64)
    assert np.all(np.abs(got - ref) <= np.maximum(np.abs(ref) * 2.0 ** -10, 2.0 ** -24))
    h32 = x.view(np.float16).astype(np.float32) + r.view(np.float16).astype(np.float32)
    assert np.array_equal(new_res, h32.astype(np.float16).view(np.uint16))


def test_rope_restatement_against_float64():
    rows, hd = 9, 128
    x = oracle.fill_normal_f16(rows * hd, 3).reshape(rows, hd)
    pos = np.array([0, 1, 2, 17, 100, 1000, 2047, 4000, 4095], np.int32)
    out = oracle.rope_f16(x, pos).view(np.float16).astype(np.float64)
    xf = x.view(np.float16).astype(np.float64).reshape(rows, hd // 2, 2)
    theta = pos[:, None].astype(np.float64) * 10000.0 ** (-2.0 * np.arange(hd // 2) / hd)
    ref = np.stack([xf[..., 0] * np.cos(theta) - xf[..., 1] * np.sin(theta),
                    xf[..., 0] * np.sin(theta) + xf[..., 1] * np.cos(theta)], -1).reshape(rows, hd)
    # f32 theta at positions in the thousands is good to ~2.5e-4 rad; then one f16 rounding
    assert np.abs(out - ref).max() < 4e-3
    assert np.array_equal(oracle.rope_f16(x[:1], pos[:1]), x[:1])  # position 0 is the identity
    # rotations preserve the norm of each pair
    n_in = np.hypot(xf[..., 0], xf[..., 1])
    o = out.reshape(rows, hd // 2, 2)
    assert np.abs(np.hypot(o[..., 0], o[..., 1]) - n_in).max() < 4e-3
