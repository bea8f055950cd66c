"""The fused all-gather over several steps with different activations every step, on two
GPUs (skipped on a single-GPU box): every step's gathered buffer on every rank equals NCCL's
all-gather of the same step, while the peers run ahead by up to one step. This is the
write-after-read case two alternating buffers exist for: rank A still reads step i's buffer
when rank B's step i+1 epilogue is already storing into A's memory.
Plain peer stores only; NVLS off for the collectives used beside them."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    from y_b200 import colpar, quant as q
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok = True
    try:
        m, k, n_s = 1024, 512, 768
        g = torch.Generator(device="cuda")
        g.manual_seed(100 + rank)
        w = torch.randn(k, n_s, device="cuda", dtype=torch.float16, generator=g)
        sb = q.scale_from_amax(colpar.agree_amax(q.amax(w)))
        bqt = q.quantize_fp8(w, sb, transpose=True)
        gamma = torch.ones(k, device="cuda", dtype=torch.float16)
        layer = colpar.ColumnParallelFp8Linear(bqt, sb, gamma, 1e-6, m)
        fused = colpar.GatheredOutput(m, n_s, buffers=2)
        g.manual_seed(7)  # the same activations on every rank
        c = torch.empty(m, n_s, dtype=torch.bfloat16, device="cuda")
        want = torch.empty(world, m, n_s, dtype=torch.bfloat16, device="cuda")
        view = None
        for step in range(12):
            x = torch.randn(m, k, device="cuda", dtype=torch.float16, generator=g)
            layer.forward(x, gathered=fused)
            fused.barrier()
            # read this step's buffer on the step's stream; rank 1 dawdles so that rank 0 runs ahead
            got = torch.empty(world, m, n_s, dtype=torch.bfloat16, device="cuda")
            if rank == 1:
                torch.cuda._sleep(2_000_000)
            import ctypes as C
            C.CDLL("libcudart.so.12").cudaMemcpyAsync(C.c_void_p(got.data_ptr()), C.c_void_p(fused.base + fused._buffer_offset()),
                                                      C.c_size_t(fused.buffer_bytes), C.c_int(3),
                                                      C.c_void_p(torch.cuda.current_stream().cuda_stream))
            layer.forward(x, out=c)
            colpar.gather_columns(c, out=want)
            torch.cuda.synchronize()
            ok = ok and torch.equal(got, want)
            fused.advance()
        q.device_status()
        fused.close()
    finally:
        dist.destroy_process_group()
    ret[rank] = ok


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gather_matches_nccl_every_step_with_changing_inputs():
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[0] and ret[1]
