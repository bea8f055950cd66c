"""The host launch API on a GPU: the compile -> load -> launch flow of the reference
(c_api.rs + cuda_runtime.rs) drives the sm_100a kernels and matches the oracle."""
import ctypes as C
import json

import numpy as np
import pytest

import oracle
from helpers import assert_gemm_close

pytestmark = pytest.mark.gpu

SRC = """
@tile(256, 256, 256)
kernel gemm_fp8_256(A: GlobalMemory<F32>, B: GlobalMemory<F32>, scale_a: F32, scale_b: F32, C: GlobalMemory<F32>) {
}
fn main() {
}
"""


@pytest.fixture(scope="module")
def rt(cuda):
    from y_b200 import runtime
    return runtime


def test_context_buffers_and_range_checks(rt):
    from y_b200._lib import YB200Error
    ctx = rt.CudaContext.new()
    assert ctx is not None and "B200" in ctx.device_name()
    assert ctx.device_attribute(rt.CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE) > 64 << 20
    assert ctx.device_attribute(16) >= 100  # multiprocessor count
    free, total = ctx.mem_info()
    assert 0 < free <= total
    buf = ctx.alloc(1024)
    assert buf.len_bytes() == 1024 and buf.device_ptr() != 0
    ctx.memset_u8(buf, 0xAB)
    assert ctx.memcpy_dtoh_at(4, buf, 1020) == b"\xab" * 4
    ctx.memcpy_htod_at(buf, 8, b"hello")
    assert ctx.memcpy_dtoh_at(5, buf, 8) == b"hello"
    with pytest.raises(YB200Error, match="out of range"):      # src/cuda_runtime.rs:408-416
        ctx.memcpy_htod_at(buf, 1020, b"12345")
    with pytest.raises(YB200Error, match="out of range"):      # src/cuda_runtime.rs:438-446
        ctx.memcpy_dtoh_at(8, buf, 1020)
    small = ctx.alloc(16)
    ctx.memcpy_dtod(small, buf)                                 # copies min(len) bytes
    assert ctx.memcpy_dtoh_at(16, small, 0)[8:13] == b"hello"
    ctx.synchronize()
    small.free(), buf.free(), ctx.close()


def test_compile_load_launch_matches_oracle(rt):
    from y_b200._lib import YB200Error
    ctx = rt.CudaContext.new()
    image = rt.compile_to_ptx(SRC, "sm_100a")
    kern = ctx.load_module(image, "gemm_fp8_256")
    with pytest.raises(YB200Error, match="no kernel named"):
        ctx.load_module(image, "gemm_fp8_512")
    info = kern.launch_info()
    assert info.block[0] == 320 and info.dyn_smem_bytes > 48 * 1024 and info.workspace_bytes > 0
    kern.set_max_dynamic_smem(info.dyn_smem_bytes)
    m = n = k = 256
    rng = np.random.default_rng(1)
    a = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 3).astype(np.float32)
    sa, sb = oracle.scale_from_amax(oracle.amax_f32(a)), oracle.scale_from_amax(oracle.amax_f32(b))
    da, db, dc = ctx.alloc(a.nbytes), ctx.alloc(b.nbytes), ctx.alloc(m * n * 4)
    ctx.memcpy_htod_at(da, 0, a.tobytes())
    ctx.memcpy_htod_at(db, 0, b.tobytes())
    grid, block = tuple(info.grid), tuple(info.block)
    ctx.launch(kern, grid, block, info.dyn_smem_bytes, [da, db, float(sa), float(sb), dc])
    ctx.synchronize()
    got = np.frombuffer(ctx.memcpy_dtoh_at(m * n * 4, dc, 0), np.float32).reshape(m, n)
    ref = oracle.gemm_fp8(oracle.quantize_fp8_f32(a, sa),
                          np.ascontiguousarray(oracle.quantize_fp8_f32(b, sb).T), sa, sb)
    assert_gemm_close(got, ref)
    # a geometry the kernel was not built for is refused, not launched
    with pytest.raises(YB200Error, match="differs"):
        ctx.launch(kern, (grid[0] + 1, 1, 1), block, info.dyn_smem_bytes, [da, db, float(sa), float(sb), dc])
    with pytest.raises(YB200Error, match="argument"):
        ctx.launch(kern, None, None, 0, [da, db, dc])
    # time_launches: mean microseconds over a batch, argument sets rotate
    us = ctx.time_launches(kern, None, None, 0, [[da, db, float(sa), float(sb), dc]] * 2, 10)
    assert 1.0 < us < 5000.0
    with pytest.raises(YB200Error, match="iters = 0"):           # src/cuda_runtime.rs:590-592
        ctx.time_launches(kern, None, None, 0, [[da, db, float(sa), float(sb), dc]], 0)
    with pytest.raises(YB200Error, match="no argument sets"):    # src/cuda_runtime.rs:593-595
        ctx.time_launches(kern, None, None, 0, [], 3)
    for h in (da, db, dc):
        h.free()
    kern.free(), ctx.close()


def test_measured_autotune_ranks_persists_and_is_reused(rt, tmp_path):
    from y_b200._lib import lib, take_string
    prof = tmp_path / ".ysu_hw_profile"
    lib.y_autotune_set_profile_path(str(prof).encode())
    try:
        ranked = json.loads(take_string(lib.y_autotune_measure_fp8_json(1024, 1024, 1024)))
        assert 1 <= len(ranked) <= 4 and all(r["best_us"] > 0 and r["tflops"] > 1 for r in ranked)
        assert all(r["best_us"] <= r["median_us"] <= r["max_us"] for r in ranked)
        text = prof.read_text()
        assert text.startswith("AUTOTUNE_FP8_1024x1024x1024_NVIDIAB200=")
        lib.y_autotune_clear_cache()
        lib.y_autotune_set_mode(0)
        out, near = (C.c_uint32 * 7)(), (C.c_uint32 * 3)()
        assert lib.y_autotune_lookup(1024, 1024, 1024, 3, b"NVIDIA B200", out, near) == 1
        assert out[1] == ranked[0]["cta_n"]
    finally:
        lib.y_autotune_set_profile_path(b"")
        lib.y_autotune_clear_cache()


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(cuda):
    """Failure detection without a fault: a barrier nothing completes, a wait budget of about
    0.1 ms, an error status the host reads; afterwards the GPU computes as before."""
    import torch

    from y_b200 import quant as q
    from y_b200._lib import ERR_DEVICE, YB200Error, check, lib
    q.device_status()                                   # clean to begin with
    check(lib.y_b200_selftest_bounded_wait(200_000, None))
    with pytest.raises(YB200Error) as e:
        q.device_status()
    assert e.value.code == ERR_DEVICE and "0x7e57" in e.value.message
    q.device_status()                                   # reading cleared it
    a = torch.randint(0, 0x78, (256, 256), dtype=torch.uint8, device="cuda")
    c1 = q.gemm_fp8_codes(a, a, 1.0, 1.0)
    c2 = q.gemm_fp8_codes(a, a, 1.0, 1.0)
    q.device_status()
    assert torch.equal(c1, c2) and torch.isfinite(c1).all()
