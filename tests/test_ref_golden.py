"""The CPU oracle against outputs of the reference's own kernels, recorded on a B200
(tests/golden/ref_kernels.npz, written by tests/golden/make_ref_golden.py from oracle/_ref/).
Inputs are rebuilt from the same seeds. Exact where the arithmetic is exact (e4m3 codes seen
through a GEMM against the identity, the f16 residual stream), the reference's own gates and
this build's GEMM tolerance elsewhere. This is the pin of the oracle that runs without a GPU."""
import importlib.util
import os

import numpy as np
import pytest

import oracle
from helpers import assert_gemm_close

HERE = os.path.dirname(os.path.abspath(__file__))
NPZ = os.path.join(HERE, "golden", "ref_kernels.npz")

pytestmark = pytest.mark.skipif(not os.path.exists(NPZ), reason="tests/golden/ref_kernels.npz has not been recorded")


@pytest.fixture(scope="module")
def cases():
    spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(HERE, "golden", "make_ref_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.golden_inputs(), np.load(NPZ)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def f16(bits):
    return bits.view(np.float16).astype(np.float64)


@pytest.mark.parametrize("case,side", [("fp8_probe_a", "a"), ("fp8_probe_a_exact", "a"), ("fp8_probe_b", "b")])
def test_e4m3_codes_equal_the_reference_kernels(cases, case, side):
    inputs, ref = cases
    i = inputs[case]
    scale = i["sa"] if side == "a" else i["sb"]
    want = oracle.decode_e4m3(oracle.quantize_fp8_f32(i[side], scale)) * np.float32(np.float32(scale) * np.float32(1.0))
    assert np.array_equal(ref[case], want)


def test_fp8_gemm_random(cases):
    inputs, ref = cases
    i = inputs["fp8_random"]
    want = oracle.gemm_fp8(oracle.quantize_fp8_f32(i["a"], i["sa"]), np.ascontiguousarray(oracle.quantize_fp8_f32(i["b"], i["sb"]).T),
                           i["sa"], i["sb"])
    assert_gemm_close(ref["fp8_random"], want, "reference gemm_fp8_256 vs oracle")
    assert rel_l2(ref["fp8_random"], want) < 1e-5


def test_f16_gemm_family(cases):
    inputs, ref = cases
    i = inputs["f16_gemm_256"]
    assert_gemm_close(ref["f16_gemm_256"], oracle.gemm_f16(i["a"], np.ascontiguousarray(i["b"].T)), "gemm_f16_256")
    i = inputs["f16_bias_relu_64"]
    want = oracle.gemm_f16(i["a"], np.ascontiguousarray(i["b"].T), bias=i["bias"], epilogue=oracle.EPI_BIAS_RELU)
    assert_gemm_close(ref["f16_bias_relu_64"], want, "gemm_f16_bias_relu_64")
    assert (want == 0).any() and ((ref["f16_bias_relu_64"] == 0) != (want == 0)).mean() < 5e-3
    i = inputs["f16_swiglu_512"]
    inter = np.empty((1024, 512), np.uint16)
    inter[0::2], inter[1::2] = i["wg"].T, i["wu"].T
    want = oracle.gemm_f16(i["x"], inter, epilogue=oracle.EPI_SWIGLU, row_begin=0, row_count=32)
    assert_gemm_close(ref["f16_swiglu_512_rows0_32"], want, "gemm_f16_swiglu_512")
    assert rel_l2(ref["f16_swiglu_512_rows0_32"], want) < 2e-3


def test_rmsnorm_rope_attention(cases):
    inputs, ref = cases
    i = inputs["rmsnorm_residual_4096"]
    want_out, want_res = oracle.rmsnorm_residual_f16(i["x"], i["res"], i["w"], 1e-5)
    assert np.array_equal(ref["rmsnorm_new_residual"], want_res)
    a, b = f16(ref["rmsnorm_out"]), f16(want_out)
    assert np.all(np.abs(a - b) <= 0.02 + 0.02 * np.abs(b))          # tests/benchmark_y_rmsnorm_rope.py:109
    assert (ref["rmsnorm_out"] != want_out).mean() < 0.02             # rsqrt.approx: rare one-step differences
    i = inputs["rope_128"]
    want = f16(oracle.rope_f16(i["x"], i["pos"]))
    got = f16(ref["rope_128"])
    assert np.all(np.abs(got - want) <= 0.02 + 0.02 * np.abs(want))   # :183
    assert np.array_equal(got[0], f16(i["x"])[0])                     # position 0 is the identity
    i = inputs["paged_decode_attention"]
    want = f16(oracle.paged_decode_attention(i["q"], i["k"], i["v"], i["pt"], i["sl"]))
    got = f16(ref["paged_decode_attention"])
    assert rel_l2(got, want) <= 3e-3                                  # tests/benchmark_y_paged_decode_attention.py:62
    assert not got[0].any()                                           # the zero-length sequence
