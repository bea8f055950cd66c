"""Small, self-contained launches of one kernel family each, sized for a profiler
capture (a few launches, a few hundred MB on the device, inputs larger than L2).

  python -m y_b200.profile_cases step   [--m 8192 --n 8192 --k 8192] [--iters 3]
  python -m y_b200.profile_cases gemm   [--m ... --n ... --k ... --epilogue none|bias_relu|swiglu]
  python -m y_b200.profile_cases decode [--tokens 8] [--iters 48]
  python -m y_b200.profile_cases quantize [--m 8192 --k 8192]
  python -m y_b200.profile_cases layer_ops [--m 8192 --k 8192]     fused add+RMSNorm, RoPE
  python -m y_b200.profile_cases attention [--seqs 16 --seq-len 4096]
"""
from __future__ import annotations

import argparse

import torch

from . import quant as q


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["step", "gemm", "decode", "quantize", "layer_ops", "attention"])
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--cta-n", type=int, default=0)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias_relu", "swiglu"])
    a = ap.parse_args()
    torch.manual_seed(0)
    dev = "cuda"
    if a.case in ("step", "gemm", "quantize", "layer_ops"):
        x = torch.randn(a.m, a.k, device=dev, dtype=torch.float16)
    if a.case == "layer_ops":
        r = torch.randn_like(x)
        g = (torch.rand(a.k, device=dev) + 0.5).to(torch.float16)
        heads = x.view(-1, 128)  # rows of one head each
        pos = torch.randint(0, 4096, (heads.shape[0],), dtype=torch.int32, device=dev)
        for _ in range(a.iters):
            q.fused_add_rmsnorm(x, r, g, 1e-5)
            q.rope(heads, pos)
    elif a.case == "attention":
        hq, hkv, hd, ps = 32, 8, 128, 16
        pages = a.seqs * (a.seq_len // ps)
        kc = torch.randn(pages, ps, hkv, hd, device=dev, dtype=torch.float16)
        vc = torch.randn(pages, ps, hkv, hd, device=dev, dtype=torch.float16)
        qv = torch.randn(a.seqs, hq, hd, device=dev, dtype=torch.float16)
        pt = torch.randperm(pages, device=dev).to(torch.int32).view(a.seqs, a.seq_len // ps)
        sl = torch.full((a.seqs,), a.seq_len, dtype=torch.int32, device=dev)
        for _ in range(a.iters):
            q.paged_decode_attention(qv, kc, vc, pt, sl)
    elif a.case == "quantize":
        for _ in range(a.iters):
            q.quantize_fp8_dynamic(x)
            q.quantize_fp8_dynamic(x, transpose=True)
    elif a.case in ("step", "gemm"):
        w = torch.randn(a.k, a.n, device=dev, dtype=torch.float16)
        bqt, sb = q.quantize_fp8_dynamic(w, transpose=True)
        del w
        gamma = (torch.rand(a.k, device=dev) + 0.5).to(torch.float16)
        aq, sa = q.quantize_fp8_dynamic(x)
        bias = (torch.randn(a.n, device=dev) * 0.1).to(torch.float16)
        for _ in range(a.iters):
            if a.case == "step":
                aq, sa = q.rmsnorm_quantize_fp8(x, gamma, 1e-6)
            if a.epilogue == "swiglu":
                q.gemm_fp8_swiglu_requant(aq, bqt, sa, sb, cta_n=a.cta_n)
            elif a.epilogue == "bias_relu":
                q.gemm_fp8_codes(aq, bqt, sa, sb, bias=bias, epilogue=q.EPI_BIAS_RELU,
                                 out_dtype=torch.bfloat16, cta_n=a.cta_n)
            else:
                q.gemm_fp8_codes(aq, bqt, sa, sb, out_dtype=torch.bfloat16, cta_n=a.cta_n)
    else:
        k, n = 4096, 11008
        w = (torch.randn(k, n, device=dev) / 64).to(torch.float16)
        qw, sc = q.int4_quantize(w)
        pool = [q.int4_repack(qw, sc) for _ in range(24)]  # 24 x 23 MB > 4 x L2
        xs = torch.randn(a.tokens, k, device=dev, dtype=torch.float16)
        out = torch.empty(a.tokens, n, device=dev, dtype=torch.float16)
        for i in range(a.iters):
            q.gemm_int4_decode(xs, pool[i % len(pool)], n, out=out)
    torch.cuda.synchronize()
    q.device_status()
    print("ok")


if __name__ == "__main__":
    main()
