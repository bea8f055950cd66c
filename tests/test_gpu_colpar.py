"""The column-parallel operator on one GPU: its device path against the oracle chain,
and its pipelined host path (copy-in, kernels and copy-out on three streams, two
buffer slots) against the device path over more steps than slots."""
import numpy as np
import pytest
import torch

import oracle
from helpers import assert_gemm_close, dev, f16_dev, host_bits, to_f64

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def layer_and_inputs(cuda):
    from y_b200 import colpar, quant as q
    m, k, n = 320, 512, 384
    w = oracle.fill_normal_f16(k * n, oracle.SEED_B).reshape(k, n)
    sb = oracle.scale_from_amax(oracle.amax_f16(w))
    bqt_h = oracle.quantize_fp8_f16_transpose(w, sb)
    g = oracle.fill_uniform_f16(k, oracle.SEED_A + 2, 0.5, 1.5)
    layer = colpar.ColumnParallelFp8Linear(dev(bqt_h), sb, f16_dev(g), 1e-6, m)
    xs = [oracle.fill_normal_f16(m * k, oracle.SEED_A + 100 + i).reshape(m, k) for i in range(5)]
    return layer, xs, g, bqt_h, sb, q


def test_forward_matches_the_oracle_chain(layer_and_inputs):
    layer, xs, g, bqt_h, sb, q = layer_and_inputs
    c = layer.forward(f16_dev(xs[0]))
    q.device_status()
    aq, sa = oracle.rmsnorm_quantize_fp8(xs[0], g, 1e-6)
    ref = oracle.gemm_fp8(aq, bqt_h, sa, sb, out_kind=oracle.OUT_BF16)
    assert_gemm_close(to_f64(host_bits(c), oracle.OUT_BF16), to_f64(ref, oracle.OUT_BF16))


def test_step_at_the_benchmark_shape(cuda):
    """The column-parallel step at its full size (M = K = N = 8192): the RMSNorm -> e4m3 prologue
    bit-exact on the whole tensor (codes and scale), whole GEMM rows from several M tiles against
    the oracle, and repeated steps bit-identical."""
    from y_b200 import colpar, quant as q
    m = k = n = 8192
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    x = torch.randn(m, k, device="cuda", dtype=torch.float16, generator=g)
    gamma = (torch.rand(k, device="cuda", generator=g) + 0.5).to(torch.float16)
    w = torch.randn(k, n, device="cuda", dtype=torch.float16, generator=g)
    bqt, sb = q.quantize_fp8_dynamic(w, transpose=True)
    del w
    layer = colpar.ColumnParallelFp8Linear(bqt, sb, gamma, 1e-6, m)
    c = layer.forward(x).clone()
    q.device_status()
    x_h, g_h = host_bits(x), host_bits(gamma)
    aq_ref, sa_ref = oracle.rmsnorm_quantize_fp8(x_h, g_h, 1e-6)
    aq_dev, sa_dev = q.rmsnorm_quantize_fp8(x, gamma, 1e-6)
    assert sa_dev.item() == np.float32(sa_ref)
    assert np.array_equal(aq_dev.cpu().numpy(), aq_ref)
    bqt_h = bqt.cpu().numpy()
    for r in (0, 129, 2047, 2048, 4100, 6000, 8063, 8191):
        ref = oracle.gemm_fp8(aq_ref, bqt_h, sa_ref, sb.item(), out_kind=oracle.OUT_BF16, row_begin=r, row_count=1)
        assert_gemm_close(to_f64(host_bits(c[r:r + 1]), oracle.OUT_BF16), to_f64(ref, oracle.OUT_BF16), f"row {r}")
    for _ in range(2):
        assert torch.equal(layer.forward(x), c)


def test_c_abi_handle_forward_and_shape_errors(layer_and_inputs):
    """y_colpar_forward (the device path behind the C handle) gives the operator's result, and a
    bad shape or depth is an error code at creation."""
    from y_b200._lib import check, last_error, lib
    layer, xs, g, bqt_h, sb, q = layer_and_inputs
    want = layer.forward(f16_dev(xs[1])).clone()
    sb_dev = torch.tensor([sb], dtype=torch.float32, device="cuda")
    h = lib.y_colpar_create(layer.bqt.data_ptr(), sb_dev.data_ptr(), layer.gamma.data_ptr(), 1e-6, layer.m, layer.k,
                            layer.n_shard, 2)
    assert h, last_error()
    x = f16_dev(xs[1])
    c = torch.empty(layer.m, layer.n_shard, dtype=torch.bfloat16, device="cuda")
    for slot in (0, 1):
        c.zero_()
        check(lib.y_colpar_forward(h, x.data_ptr(), c.data_ptr(), slot, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert torch.equal(c, want)
    assert lib.y_colpar_forward(h, x.data_ptr(), c.data_ptr(), 2, None) != 0 and "slot" in last_error()
    lib.y_colpar_destroy(h)
    assert not lib.y_colpar_create(layer.bqt.data_ptr(), sb_dev.data_ptr(), layer.gamma.data_ptr(), 1e-6, layer.m, 24,
                                   layer.n_shard, 2)
    assert not lib.y_colpar_create(layer.bqt.data_ptr(), sb_dev.data_ptr(), layer.gamma.data_ptr(), 1e-6, layer.m, layer.k,
                                   layer.n_shard, 9)
    q.device_status()


def test_host_pipeline_equals_device_path_step_by_step(layer_and_inputs):
    layer, xs, g, bqt_h, sb, q = layer_and_inputs
    m, k, n = layer.m, layer.k, layer.n_shard
    want = [layer.forward(f16_dev(x)).clone() for x in xs]
    torch.cuda.synchronize()
    x_host = [torch.from_numpy(x.view(np.float16).copy()).pin_memory() for x in xs]
    c_host = [torch.empty(m, n, dtype=torch.bfloat16).pin_memory() for _ in xs]
    for _ in range(3):  # several rounds: slots are reused while earlier steps are in flight
        for c in c_host:
            c.zero_()
        for xh, ch in zip(x_host, c_host):
            layer.submit_host(xh, ch)
        layer.drain()
        torch.cuda.synchronize()
        q.device_status()
        for ch, w in zip(c_host, want):
            assert torch.equal(ch, w.cpu())


def test_epilogue_replicas_receive_the_same_bits(layer_and_inputs):
    """The fused all-gather's mechanism on one GPU: the replicas are local buffers here, peer
    memory on a multi-GPU node; vector-store and ragged (scalar-store) shapes."""
    layer, xs, g, bqt_h, sb, q = layer_and_inputs
    for (m, n, k) in ((320, 384, 512), (100, 72, 128), (320, 96, 256), (257, 160, 128), (512, 8192, 128)):
        aq = torch.randint(0, 0x78, (m, k), dtype=torch.uint8, device="cuda")
        bq = torch.randint(0, 0x78, (n, k), dtype=torch.uint8, device="cuda")
        for cta_m, dt in ((128, torch.bfloat16), (256, torch.bfloat16), (256, torch.float16), (128, torch.float32)):
            want = q.gemm_fp8_codes(aq, bq, 0.5, 0.25, out_dtype=dt, cta_m=cta_m)
            reps = [torch.zeros_like(want) for _ in range(7)]
            got = q.gemm_fp8_codes(aq, bq, 0.5, 0.25, out_dtype=dt, cta_m=cta_m, replicas=reps)
            q.device_status()
            assert torch.equal(got, want)
            for r in reps:
                assert torch.equal(r, want)


def test_gathered_output_on_one_rank(layer_and_inputs):
    """World size 1: the gathered buffer has one slot, filled by the GEMM, read back through the library."""
    from y_b200 import colpar
    layer, xs, g, bqt_h, sb, q = layer_and_inputs
    gathered = colpar.GatheredOutput(layer.m, layer.n_shard)
    try:
        want = layer.forward(f16_dev(xs[1]))
        layer.forward(f16_dev(xs[1]), gathered=gathered)
        gathered.barrier()
        assert torch.equal(gathered.to_host()[0], want.cpu())
    finally:
        gathered.close()
