"""The C-ABI library loads without a GPU, exports every symbol the headers declare,
and the host-side entry points (c_api.rs surface, error paths) behave as the
reference's do. No compute call is made here."""
import ctypes as C
import json
import os
import re

import pytest

from y_b200 import _lib, runtime
from y_b200._lib import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for hdr in ("y_b200.h", "y_b200_runtime.h"):
        text = open(os.path.join(ROOT, "include", hdr)).read()
        names |= set(re.findall(r"Y_B200_API[^;(]*?\b(y_[a-z0-9_]+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported_and_bound():
    declared = _declared_symbols()
    assert len(declared) > 50
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "python binding table and headers disagree"


def test_block_cdiv_matches_reference_values():
    # tests/test_rust_triton_parity.rs:62-63 and src/c_api.rs:196-201
    assert runtime.block_cdiv(10, 3) == 4
    assert runtime.block_cdiv(100, 32) == 4
    assert runtime.block_cdiv(5, 0) == 0
    assert runtime.block_cdiv(0, 7) == 0


def test_autotune_json_has_the_reference_keys():
    # tests/test_rust_triton_parity.rs:65-73
    space = runtime.autotune_search_space(1024, 1024, 1024, True)
    assert space and all({"cta_m", "cta_n", "cta_k", "warps_m", "warps_n", "num_stages", "num_warps",
                          "is_fp8"} <= set(c) for c in space)
    assert all(c["is_fp8"] is True for c in space)
    assert all(c["num_stages"] >= 2 and c["num_warps"] >= 4 for c in space)
    cfg = runtime.autotune_select_config(2048, 2048, 2048, True)
    assert set(cfg) == {"cta_m", "cta_n", "cta_k", "warps_m", "warps_n", "num_stages", "num_warps"}
    assert cfg["cta_m"] >= 64 and cfg["num_stages"] >= 2 and cfg["num_warps"] >= 4
    # decode shapes resolve to the weight-streaming kernel's geometry
    dec = runtime.autotune_select_config(8, 11008, 4096, False)
    assert dec["cta_m"] == 8 and dec["cta_n"] == 16


FP8_SRC = """
// FP8 GEMM fixture shape
@tile(256, 256, 256)
kernel gemm_fp8_256(A: GlobalMemory<F32>, B: GlobalMemory<F32>, scale_a: F32, scale_b: F32, C: GlobalMemory<F32>) {
}

fn main() {
}
"""


def test_compile_returns_a_launch_descriptor_for_tile_kernels():
    text = runtime.compile_to_ptx(FP8_SRC, "sm_100a")
    assert "entry=gemm_fp8_256 family=gemm_fp8" in text
    assert "M=256 N=256 K=256" in text
    assert "Dynamic shared memory required:" in text and "Launch grid required:" in text
    out = (C.c_uint32 * 4)()
    fake = "// [Y TENSOR CORE GEMM] M=1024 N=1024 K=1024 | CTA 64x128x32 | 2x2 warps | x\n" \
           "// Dynamic shared memory required: 61952 bytes.\n"
    # src/empirical_autotune.rs:1003-1019
    assert lib.y_parse_launch_config(fake.encode(), 1024, 1024, out) == 0
    assert list(out) == [8, 16, 128, 61952]
    # the synchronous fallback prints no byte count: 0 is the answer (:1021-1030)
    fake2 = "    // [Y TENSOR CORE GEMM] M=64 N=64 K=32 | CTA 32x32x32 | 2x1 warps | wmma\n"
    assert lib.y_parse_launch_config(fake2.encode(), 64, 64, out) == 0
    assert out[3] == 0 and out[2] == 64
    assert lib.y_parse_launch_config(b".version 8.4\n", 64, 64, out) != 0
    # the library's own descriptor parses with the same routine
    assert lib.y_parse_launch_config(text.encode(), 256, 256, out) == 0
    assert out[3] > 0


def test_compile_errors_follow_the_reference_contract():
    # null source -> error text, not a crash (src/c_api.rs:32-37)
    err = C.c_void_p()
    assert lib.y_compile_to_ptx(None, b"sm_100a", C.byref(err)) is None
    assert _lib.take_string(err.value) == "Source pointer is null"
    assert lib.y_interpret_kernel(None, C.byref(err)) == -1
    assert _lib.take_string(err.value) == "Source pointer is null"
    assert lib.y_interpret_kernel(FP8_SRC.encode(), C.byref(err)) == 0
    lib.y_free_string(None)  # null is allowed (src/c_api.rs:208-212)
    # 5-parameter shape with a wrong element type (src/type_checker.rs:944-975)
    bad = FP8_SRC.replace("A: GlobalMemory<F32>", "A: GlobalMemory<F16>")
    with pytest.raises(ValueError, match="5 parameters"):
        runtime.compile_to_ptx(bad)
    # K % 64 precondition of the FP8 family (src/ptx_emitter.rs:3297-3304)
    with pytest.raises(ValueError, match="multiple of 64"):
        runtime.compile_to_ptx(FP8_SRC.replace("@tile(256, 256, 256)", "@tile(256, 256, 96)"))
    # K is not optional on a kernel-level @tile (src/type_checker.rs:911-916)
    with pytest.raises(ValueError):
        runtime.compile_to_ptx(FP8_SRC.replace("@tile(256, 256, 256)", "@tile(256, 256)"))
    with pytest.raises(ValueError, match="requires 3 parameters"):
        runtime.compile_to_ptx("@tile(64,64,64)\nkernel k(A: GlobalMemory<F16>, C: GlobalMemory<F32>) {\n}\n")


def test_other_reference_shapes_are_classified():
    for name, params, fam in [
        ("gemm_f16_decode_m1", "A: GlobalMemory<F16>, B: GlobalMemory<F16>, C: GlobalMemory<F32>", "gemm_f16"),
        ("gemm_f16_bias_relu_512", "A: GlobalMemory<F16>, B: GlobalMemory<F16>, Bias: GlobalMemory<F32>, "
                                   "C: GlobalMemory<F32>", "gemm_f16_bias_relu"),
        ("gemm_f16_swiglu_512", "X: GlobalMemory<F16>, Wgate: GlobalMemory<F16>, Wup: GlobalMemory<F16>, "
                                "Out: GlobalMemory<F32>", "gemm_f16_swiglu"),
    ]:
        text = runtime.compile_to_ptx(f"@tile(512, 512, 512)\nkernel {name}({params}) {{\n}}\n")
        assert f"entry={name} family={fam}" in text
        # the descriptor names the kernel that really runs, its workspace and the fused-epilogue count
        assert "tcgen05.mma.cta_group::1.kind::f16" in text and "Workspace required:" in text
        assert ("Fused epilogues: 0" if fam == "gemm_f16" else "Fused epilogues: 1") in text
    # decode shapes of the plain F16 GEMM stream the row-major weights: no workspace, no tcgen05 claim
    dec = runtime.compile_to_ptx("@tile(8, 4096, 4096)\nkernel gemm_f16_decode_m8(A: GlobalMemory<F16>, "
                                 "B: GlobalMemory<F16>, C: GlobalMemory<F32>) {\n}\n")
    assert "weight streaming" in dec and "Workspace required: 0 bytes" in dec and "tcgen05" not in dec
    out = (C.c_uint32 * 4)()
    assert lib.y_parse_launch_config(dec.encode(), 8, 4096, out) == 0
    assert (out[0], out[1], out[2], out[3]) == (64, 1, 256, 106496)   # 64-column blocks (the parser knows no clusters)
    assert "Launch grid required: (256, 1, 1) CTAs, block (256,1,1), cluster (4,1,1)" in dec
    # 17..32 tokens run on tcgen05 with the weights as the MN-major operand: still no workspace
    dec32 = runtime.compile_to_ptx("@tile(32, 4096, 4096)\nkernel gemm_f16_decode_m32(A: GlobalMemory<F16>, "
                                   "B: GlobalMemory<F16>, C: GlobalMemory<F32>) {\n}\n")
    assert "weight streaming, tcgen05.mma.cta_group::1.kind::f16" in dec32 and "Workspace required: 0 bytes" in dec32
    assert "block (128,1,1), cluster (4,1,1)" in dec32
    rms = ("kernel rmsnorm_residual_4096(X: GlobalMemory<F16>, Residual: GlobalMemory<F16>, "
           "Weight: GlobalMemory<F16>, Out: GlobalMemory<F16>, NewResidual: GlobalMemory<F16>) {\n}\n")
    assert "family=rmsnorm_residual" in runtime.compile_to_ptx(rms)
    with pytest.raises(ValueError, match="128"):
        runtime.compile_to_ptx("@tile(100, 128, 64)\nkernel s(X: GlobalMemory<F16>, G: GlobalMemory<F16>, "
                               "U: GlobalMemory<F16>, O: GlobalMemory<F32>) {\n}\n")


def test_argument_errors_are_codes_not_crashes():
    assert lib.y_b200_amax(None, _lib.F16, 10, None, None) == _lib.ERR_INVALID
    assert "null" in _lib.last_error()
    assert lib.y_b200_gemm_fp8(None, None) == _lib.ERR_INVALID
    assert lib.y_b200_gemm_int4_decode(None, None, None, 1, 16, 128, None) == _lib.ERR_INVALID
    assert lib.y_b200_int4_stream_bytes(4096, 11008) == 22_544_384 + 704_512
    assert lib.y_b200_gemm_fp8_f32_workspace_bytes(256, 256, 256) == 2 * 65536 + 256
    assert lib.y_b200_swiglu_workspace_bytes(4096, 22016) == 256 + 4096 * 11008 * 2
    assert lib.y_b200_rmsnorm_workspace_bytes(8192) == 8192 * 4 + 256
    assert lib.y_b200_gemm_f16_rowmajor_workspace_bytes(4096, 4096) == 4096 * 4096 * 2
    assert lib.y_b200_gemm_f16_swiglu_workspace_bytes(11008, 4096) == 2 * 11008 * 4096 * 2
    assert lib.y_b200_gemm_f16(None, None) == _lib.ERR_INVALID
    assert not lib.y_colpar_create(None, None, None, 1e-6, 8, 16, 8, 2) and "null" in _lib.last_error()
    assert lib.y_colpar_submit_host(None, None, None, None) == _lib.ERR_INVALID
    assert lib.y_colpar_drain(None, None) == _lib.ERR_INVALID
    lib.y_colpar_destroy(None)
    us = C.c_float(0.0)
    assert lib.y_b200_probe_chain_read(None, 0, 16, 1, 1, None, C.byref(us), None) == _lib.ERR_INVALID
    one = (C.c_void_p * 1)(64)
    assert lib.y_b200_probe_chain_read(one, 1, 24, 1, 1, 64, C.byref(us), None) == _lib.ERR_SHAPE
    assert lib.y_b200_probe_chain_read(one, 1, 32, 1, 65, 64, C.byref(us), None) == _lib.ERR_SHAPE
    odd = (C.c_void_p * 1)(72)
    assert lib.y_b200_probe_chain_read(odd, 1, 32, 1, 1, 64, C.byref(us), None) == _lib.ERR_ALIGN
    assert lib.y_b200_gemm_f16_decode(None, 0, None, None, 0, 1, 8, 16, None) == _lib.ERR_INVALID
    one = C.c_int(0)
    p = C.addressof(one)
    assert lib.y_b200_gemm_f16_decode(p, 4096, p, p, _lib.F32, 33, 4096, 4096, None) == _lib.ERR_SHAPE
    assert lib.y_b200_gemm_f16_decode(p, 4096, p, p, _lib.F32, 1, 4096, 4100, None) == _lib.ERR_SHAPE
    assert b"sm_100a" in lib.y_b200_version()


def test_context_creation_never_aborts_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    assert runtime.CudaContext.new() is None  # src/cuda_runtime.rs:330-364


def _reference_tests_dir():
    """The reference checkout's tests/ directory: $Y_REFERENCE_ROOT, else a directory named
    `reference` beside the repository; None when neither exists (the GPU box has none)."""
    roots = [os.environ.get("Y_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference")]
    for r in roots:
        if r and os.path.isdir(os.path.join(r, "tests")):
            return os.path.join(os.path.abspath(r), "tests")
    return None


@pytest.mark.skipif(_reference_tests_dir() is None, reason="the reference checkout is not on this machine")
def test_the_references_own_kernel_fixtures_compile_to_the_right_family():
    """Every .ysu kernel fixture of the reference goes through y_compile_to_ptx verbatim and
    lands in the family its name says (a CPU-side check: the GPU box has no reference tree)."""
    import glob
    expect = (("gemm_fp8_", "gemm_fp8"), ("gemm_f16_bias_relu_", "gemm_f16_bias_relu"),
              ("gemm_f16_swiglu_", "gemm_f16_swiglu"), ("gemm_f16_", "gemm_f16"),
              ("rmsnorm_residual_", "rmsnorm_residual"), ("rope_", "rope"),
              ("paged_decode_attention_", "paged_decode_attention"))
    seen = 0
    for path in sorted(glob.glob(os.path.join(_reference_tests_dir(), "*.ysu"))):
        stem = os.path.basename(path)[:-4]
        fam = next((f for prefix, f in expect if stem.startswith(prefix)), None)
        if fam is None:
            continue
        image = runtime.compile_to_ptx(open(path).read())
        assert f" family={fam} " in image and "entry=" + stem.rsplit("_", 1)[0] in image, stem
        seen += 1
    assert seen >= 30
