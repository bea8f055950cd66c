"""Paged decode attention against the double-precision oracle: shuffled page tables,
ragged and zero sequence lengths, partial last pages, GQA ratios 1..8, head sizes
64/128/256, page sizes 1/16/32/64, long contexts (the reference's own validation list,
src/ptx_emitter.rs:6438-6446), plus repeat-launch determinism."""
import numpy as np
import pytest
import torch

import oracle
from helpers import dev, f16_dev, host_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q(cuda):
    from y_b200 import quant
    return quant


def _case(hd, hq, hkv, ps, seq_lens, seed):
    rng = np.random.default_rng(seed)
    ns = len(seq_lens)
    max_pages = max(1, max((int(x) + ps - 1) // ps for x in seq_lens))
    num_pages = max_pages * ns + 3
    qv = oracle.fill_normal_f16(ns * hq * hd, seed + 1).reshape(ns, hq, hd)
    kc = oracle.fill_normal_f16(num_pages * ps * hkv * hd, seed + 2).reshape(num_pages, ps, hkv, hd)
    vc = oracle.fill_normal_f16(num_pages * ps * hkv * hd, seed + 3).reshape(num_pages, ps, hkv, hd)
    pt = np.stack([rng.permutation(num_pages)[:max_pages] for _ in range(ns)]).astype(np.int32)
    return qv, kc, vc, pt, np.array(seq_lens, np.int32)


def _check(got_bits, ref_bits):
    g = got_bits.view(np.float16).astype(np.float64)
    r = ref_bits.view(np.float16).astype(np.float64)
    rel_l2 = np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)
    assert rel_l2 < 2e-3, rel_l2          # probabilities travel as f16 into the second MMA
    assert np.abs(g - r).max() < 1e-2 * max(1.0, np.abs(r).max())


@pytest.mark.parametrize("hd,hq,hkv,ps,seq_lens", [
    (128, 32, 8, 16, [1, 17, 100, 0, 333]),          # the reference fixture's shape, ragged and empty
    (128, 32, 8, 16, [4096]),                         # long context, one sequence: split across CTAs
    (64, 8, 8, 1, [5, 64, 65]),                       # MHA, page size 1
    (64, 16, 2, 32, [31, 32, 33, 700]),               # GQA 8:1, partial last pages
    (256, 8, 4, 64, [200, 1]),                        # head 256
    (128, 16, 1, 16, [50] * 40),                      # 16 query heads on one KV head; splits thinner than one tile
    (128, 8, 2, 16, [40, 9] * 100),                   # more CTAs than the SMs hold at once: no split, no merge kernel
    (128, 4, 4, 16, [0, 0]),                          # nothing to attend to
])
def test_paged_decode_attention_matches_oracle(q, hd, hq, hkv, ps, seq_lens):
    qv, kc, vc, pt, sl = _case(hd, hq, hkv, ps, seq_lens, 100 + hd + hq)
    out = q.paged_decode_attention(f16_dev(qv), f16_dev(kc), f16_dev(vc), torch.from_numpy(pt).cuda(),
                                   torch.from_numpy(sl).cuda())
    q.device_status()
    got = host_bits(out)
    _check(got, oracle.paged_decode_attention(qv, kc, vc, pt, sl))
    for s, n in enumerate(seq_lens):
        if n == 0:
            assert not got[s].any()


def test_repeat_launches_are_bit_identical_and_pages_really_are_looked_up(q):
    hd, hq, hkv, ps = 128, 32, 8, 16
    qv, kc, vc, pt, sl = _case(hd, hq, hkv, ps, [777, 300, 1024], 9)
    args = (f16_dev(qv), f16_dev(kc), f16_dev(vc))
    ptd, sld = torch.from_numpy(pt).cuda(), torch.from_numpy(sl).cuda()
    first = q.paged_decode_attention(*args, ptd, sld)
    for _ in range(20):
        assert torch.equal(q.paged_decode_attention(*args, ptd, sld), first)
    # the same logical cache under a different physical page order gives the same result
    perm = np.random.default_rng(1).permutation(kc.shape[0])
    inv = np.argsort(perm)
    kc2, vc2 = kc[perm], vc[perm]          # physical page i now holds what page perm[i] held
    pt2 = inv[pt].astype(np.int32)
    again = q.paged_decode_attention(f16_dev(qv), f16_dev(kc2), f16_dev(vc2), torch.from_numpy(pt2).cuda(), sld)
    assert torch.equal(again, first)


def test_through_the_launch_api_with_the_reference_fixture_name(q):
    """compile -> load_module('paged_decode_attention_128_32_8_16') -> launch with the
    reference's grid (num_q_heads, num_seqs, 1) and seven arguments."""
    from y_b200 import runtime as rt
    src = ("kernel paged_decode_attention_128_32_8_16(Q: GlobalMemory<F16>, KCache: GlobalMemory<F16>, "
           "VCache: GlobalMemory<F16>, PageTable: GlobalMemory<I32>, SeqLens: GlobalMemory<I32>, "
           "Out: GlobalMemory<F16>, MaxPages: I32) {}")
    image = rt.compile_to_ptx(src)
    assert "family=paged_decode_attention" in image
    qv, kc, vc, pt, sl = _case(128, 32, 8, 16, [40, 1000, 7], 5)
    qd, kd, vd = f16_dev(qv), f16_dev(kc), f16_dev(vc)
    ptd, sld = torch.from_numpy(pt).cuda(), torch.from_numpy(sl).cuda()
    out = torch.empty_like(qd)
    ctx = rt.CudaContext.new()
    kern = ctx.load_module(image, "paged_decode_attention_128_32_8_16")
    ctx.launch(kern, (32, 3, 1), None, 0, [qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ptd.data_ptr(), sld.data_ptr(),
                                           out.data_ptr(), ("i32", pt.shape[1])])
    ctx.synchronize()
    assert torch.equal(out, q.paged_decode_attention(qd, kd, vd, ptd, sld))
    with pytest.raises(rt.YB200Error):  # the grid's x must be the number of query heads
        ctx.launch(kern, (8, 3, 1), None, 0, [qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ptd.data_ptr(),
                                              sld.data_ptr(), out.data_ptr(), ("i32", pt.shape[1])])
    kern.free()
    ctx.close()


@pytest.mark.parametrize("hd,hq,hkv,ps,ns", [
    (128, 32, 8, 16, 3),      # 12 splits per sequence
    (128, 32, 8, 16, 37),     # one split: more CTAs than the SMs hold
    (64, 8, 1, 16, 9),        # one KV head, few sequences: the maximum of 32 splits, most of them empty
    (256, 16, 2, 32, 150),    # head 256 (one CTA per SM), no split
    (128, 16, 16, 8, 5),      # MHA, 3 splits
])
def test_ragged_batches_over_the_range_of_split_counts(q, hd, hq, hkv, ps, ns):
    """The split count depends on the number of sequences and KV heads only, so ragged
    lengths leave some splits short or empty; whatever the count, the result is the oracle's."""
    rng = np.random.default_rng(1000 + ns)
    seq_lens = [int(v) for v in rng.integers(0, 700, size=ns)]
    seq_lens[0] = max(seq_lens[0], 1)
    if ns <= 5:
        seq_lens = [v * 5 for v in seq_lens]
    qv, kc, vc, pt, sl = _case(hd, hq, hkv, ps, seq_lens, 500 + ns)
    out = q.paged_decode_attention(f16_dev(qv), f16_dev(kc), f16_dev(vc), torch.from_numpy(pt).cuda(),
                                   torch.from_numpy(sl).cuda())
    q.device_status()
    _check(host_bits(out), oracle.paged_decode_attention(qv, kc, vc, pt, sl))
