"""Host logic of the N-sharded path on two gloo ranks (CPU). The kernels are stood in
for by the oracle; what is tested is the sharding arithmetic, the agreed weight scale
(sharded result == unsharded result, bit for bit) and the gathered layout."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from y_b200 import colpar


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, n, k, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a = oracle.fill_normal_f16(m * k, oracle.SEED_A).reshape(m, k)
        b = oracle.fill_normal_f16(k * n, oracle.SEED_B).reshape(k, n)
        lo, hi = colpar.shard_range(n, world, rank)
        b_shard = np.ascontiguousarray(b[:, lo:hi])
        amax = torch.tensor([oracle.amax_f16(b_shard)], dtype=torch.float32)
        colpar.agree_amax(amax)
        sb = oracle.scale_from_amax(amax.item())
        sa = oracle.scale_from_amax(oracle.amax_f16(a))
        aq = oracle.quantize_fp8_f16(a, sa)
        bqt = oracle.quantize_fp8_f16_transpose(b_shard, sb)
        c_local = oracle.gemm_fp8(aq, bqt, sa, sb, out_kind=oracle.OUT_BF16)
        c_t = torch.from_numpy(c_local.view(np.int16).copy()).view(torch.bfloat16)
        gathered = colpar.gather_columns(c_t)
        full = colpar.assemble(gathered)
        if rank == 0:
            ret["sb"] = sb
            ret["full"] = full.view(torch.int16).numpy().view(np.uint16).copy()
    finally:
        dist.destroy_process_group()


def test_sharded_equals_unsharded_on_two_ranks():
    m, n, k = 24, 64, 128
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), m, n, k, ret), nprocs=2, join=True)
    a = oracle.fill_normal_f16(m * k, oracle.SEED_A).reshape(m, k)
    b = oracle.fill_normal_f16(k * n, oracle.SEED_B).reshape(k, n)
    sa, sb = oracle.scale_from_amax(oracle.amax_f16(a)), oracle.scale_from_amax(oracle.amax_f16(b))
    assert ret["sb"] == sb  # the agreed scale is the scale of the whole weight
    ref = oracle.gemm_fp8(oracle.quantize_fp8_f16(a, sa), oracle.quantize_fp8_f16_transpose(b, sb), sa, sb,
                          out_kind=oracle.OUT_BF16)
    assert np.array_equal(ret["full"], ref)


def test_shard_ranges_and_layout():
    assert colpar.shard_range(65536, 8, 3) == (3 * 8192, 4 * 8192)
    assert colpar.shard_range(11008, 8, 7) == (7 * 1376, 11008)  # the decode N shards at 1376 = 16 * 86
    with pytest.raises(ValueError):
        colpar.shard_range(11008, 3, 0)
    with pytest.raises(ValueError):
        colpar.shard_range(64, 8, 0)  # 8-column shards would break 16-byte row alignment
    with pytest.raises(ValueError):
        colpar.shard_range(64, 2, 2)
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    full = colpar.assemble(g)
    assert full.shape == (3, 8) and full[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]
    # single rank: gather is a copy, agree_amax is the identity
    c = torch.ones(3, 4)
    assert colpar.gather_columns(c).shape == (1, 3, 4)
    assert colpar.agree_amax(torch.tensor([2.0])).item() == 2.0
