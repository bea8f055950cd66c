"""The allocation-free GEMM entry point, for callers that may not allocate device
memory at call time (an engine whose pool owns all of HBM, a latency-critical loop,
a plugin host that passes only inputs and outputs). Its scratch is a fixed array in
the library image, shared by every call, so this file runs last and checks two calls
in a row against the workspace-taking entry point they are a variant of."""
import numpy as np
import pytest
import torch

from helpers import assert_gemm_close

pytestmark = pytest.mark.gpu


def _inputs(m, n, k, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    a = torch.randn(m, k, device="cuda", generator=g) * 3
    b = torch.randn(k, n, device="cuda", generator=g) * 3
    sa, sb = float(a.abs().max()) / 448.0, float(b.abs().max()) / 448.0
    return a, b, sa, sb


def _static_call(a, b, sa, sb, got):
    from y_b200._lib import check, lib
    m, k = a.shape
    n = b.shape[1]
    check(lib.y_b200_gemm_fp8_f32_static(a.data_ptr(), b.data_ptr(), sa, sb, got.data_ptr(), m, n, k,
                                         torch.cuda.current_stream().cuda_stream))


def _pair(m, n, k, seed):
    from y_b200 import quant as q
    a, b, sa, sb = _inputs(m, n, k, seed)
    want = q.gemm_fp8_f32(a, b, sa, sb)                      # existing entry: caller-provided workspace
    got = torch.full((m, n), float("nan"), device="cuda")
    _static_call(a, b, sa, sb, got)
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_two_calls_in_a_row_match_the_workspace_entry(cuda):
    # the second call is smaller and differently shaped: whatever the first call left
    # in the shared scratch must not show in its result
    for m, n, k, seed in [(512, 384, 256, 1), (200, 136, 128, 2)]:
        got, want = _pair(m, n, k, seed)
        assert_gemm_close(got, want, f"{m}x{n}x{k}")
    from y_b200 import quant as q
    q.device_status()   # also reads the status word that lives inside the built-in scratch


def test_calls_leave_free_device_memory_unchanged(cuda):
    # What the entry is for: once the module is loaded (the warm-up call below, which is
    # also when the built-in array is reserved), further calls take no device memory.
    a, b, sa, sb = _inputs(256, 256, 256, 3)
    got = torch.empty(256, 256, device="cuda")
    _static_call(a, b, sa, sb, got)                           # warm-up: module load, address lookup
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        _static_call(a, b, sa, sb, got)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)


def test_sizes_beyond_the_built_in_scratch_are_refused(cuda):
    from y_b200._lib import ERR_WORKSPACE, last_error, lib
    m = n = k = 4096                                          # 2 x 16 MiB of operands > 8 MiB
    a = torch.zeros(16, device="cuda")
    rc = lib.y_b200_gemm_fp8_f32_static(a.data_ptr(), a.data_ptr(), 1.0, 1.0, a.data_ptr(), m, n, k, None)
    assert rc == ERR_WORKSPACE and "exceed the built-in scratch" in last_error()
