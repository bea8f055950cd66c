#!/usr/bin/env python
"""Benchmark of the quantised-inference GEMM path on 1..8 B200s.

One "step" is one pass of the hot path over one batch of synthetic input, on
the column-parallel configuration: X [8192, 8192] f16 -> fused RMSNorm
(eps 1e-6, gamma ~ U(0.5, 1.5)) -> per-tensor e4m3 quantisation -> FP8 GEMM
against this GPU's weight shard Bt [8192 (N shard), 8192 (K)] e4m3 -> bf16 C.
Each GPU keeps its own weight shard (weak scaling along N); the weights are
quantised once, before the timed region, with one scale agreed across ranks.
The all-gather of C is measured separately and reported under "gather".

Prints ONE JSON line (rank 0). `--impl reference` times the CPU restatement of
the same step on the host cores instead (rank 0 only).

`--only <case>` runs a few launches of one kernel family and prints "ok" instead: small,
self-contained runs sized for a profiler capture (inputs larger than L2, a few hundred MB
on the device):
  --only step      [--m 8192 --n 8192 --k 8192] [--iters 3]    prologue + GEMM
  --only gemm      [--m .. --n .. --k ..] [--epilogue none|bias_relu|swiglu] [--cta-n N]
  --only decode    [--tokens 8] [--iters 48]                   INT4 decode GEMM, K=4096, N=11008
  --only f16_decode [--tokens 8] [--iters 48]                  F16 weight streaming, K=N=4096
  --only quantize  [--m 8192 --k 8192]                         dynamic e4m3 quantisation, both layouts
  --only int4_quantize [--iters 6]                             INT4 group quantise + repack, 4096 x 11008
  --only layer_ops [--m 8192 --k 8192]                         fused add+RMSNorm, RoPE
  --only attention [--seqs 16 --seq-len 4096]                  paged decode attention
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = K = 8192
N_SHARD = 8192
EPS = 1e-6
METRIC = "fp8_gemm_tflops"
WORKLOAD = "colpar_fp8_gemm_M8192_K8192_Nshard8192_rmsnorm_fp8_prologue"
DECODE_K, DECODE_N = 4096, 11008
NOMINAL_FP8_TFLOPS = 4500.0


_emit = print  # replaced in main() by a writer to the process's original stdout


def workload_config(world: int) -> dict:
    """The `config` object of the JSON line: the workload, identical for both arms."""
    return {"workload": WORKLOAD, "m": M, "k": K, "n_per_gpu": N_SHARD, "n_total": N_SHARD * max(world, 1),
            "parallelism": f"column-parallel N over {max(world, 1)} GPU(s)",
            "step": "rmsnorm_stats + rmsnorm_quantize_fp8 + gemm_fp8 (weights pre-quantised)",
            "l2": "inputs larger than L2 (X 134 MB + Bt 67 MB + C 134 MB per step)",
            "all_gather": "not in value; see gather"}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


_REASON_NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


def clock_sampler_main(gpu_id: str):
    """Child process: reads SM clock, power and throttle reasons of one GPU through NVML
    (read-only queries) as fast as NVML answers and prints one line per sample,
    stamped with the system-wide monotonic clock, until its stdin closes."""
    import select

    import pynvml as nv

    nv.nvmlInit()
    uuid, _, index = gpu_id.partition("|")  # "GPU-<uuid>|<index>": the index is the fallback
    try:
        h = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
    except Exception:
        h = nv.nvmlDeviceGetHandleByIndex(int(index or 0))
    mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
    bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
    import collections

    out = collections.deque(maxlen=600000)  # five minutes at the 2 kHz below
    print("ready", flush=True)
    while not select.select([sys.stdin], [], [], 0.0005)[0]:
        t = time.monotonic()
        mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
        out.append("%.6f,%d,%d,%.1f,%s" % (t, mhz, mx, pw, ",".join("1" if r & bits[n] else "0" for n in _REASON_NAMES)))
    sys.stdout.write("\n".join(out) + "\n")
    sys.stdout.flush()


class ClockSampler:
    """Samples one GPU's SM clock and throttle reasons from a child process (a thread of
    this process is starved by the launch loop) and reports the samples that fall
    inside named windows of the monotonic clock."""

    def __init__(self, gpu_id: str):
        self.windows, self.samples, self.proc = {}, [], None
        try:
            self.proc = subprocess.Popen([sys.executable, os.path.abspath(__file__), "--clock-sampler", gpu_id],
                                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
            if self.proc.stdout.readline().strip() != "ready":
                self.proc = None
        except Exception:
            self.proc = None

    def window(self, name):
        sampler = self

        class _W:
            def __enter__(self):
                self.t0 = time.monotonic()

            def __exit__(self, *exc):
                sampler.windows[name] = (self.t0, time.monotonic())

        return _W()

    def close(self):
        if self.proc is None:
            return
        try:
            out, _ = self.proc.communicate(input="stop\n", timeout=30)
            for ln in out.splitlines():
                f = ln.split(",")
                if len(f) == 8:
                    self.samples.append((float(f[0]), float(f[1]), float(f[2]), float(f[3]), [v == "1" for v in f[4:]]))
        except Exception:
            self.proc.kill()
        self.proc = None

    def summary(self, name):
        t0, t1 = self.windows.get(name, (0.0, -1.0))
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        mhz = sorted(s[1] for s in inside)
        reasons = sorted({n for s in inside for n, on in zip(_REASON_NAMES, s[4]) if on})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": max((s[2] for s in inside), default=None), "reasons": reasons,
                "samples": len(mhz), "sm_mhz_min": mhz[0] if mhz else None,
                "power_w_max": max((s[3] for s in inside), default=None),
                "window_ms": (t1 - t0) * 1e3 if inside else None}


def cpu_step_sample(rows: int, seed: int = 1234):
    """The oracle's restatement of one step on `rows` output rows: RMSNorm statistics
    and quantisation over the sampled rows (the per-tensor amax is taken over the
    sample), weight shard quantised beforehand, GEMM + bf16 rounding on the rows."""
    import numpy as np

    import oracle

    x = oracle.fill_normal_f16(rows * K, seed).reshape(rows, K)
    g = oracle.fill_uniform_f16(K, seed + 2, 0.5, 1.5)
    w = oracle.fill_normal_f16(N_SHARD * K, seed + 1).reshape(N_SHARD, K)
    sb = oracle.scale_from_amax(oracle.amax_f16(w))
    # weights are prepared outside the timed step, like the GPU arm: quantised, then
    # decoded once to the f32 values the CPU multiplies with
    bf = oracle.decode_e4m3(oracle.quantize_fp8_f16(w, sb))

    def step():
        aq, sa = oracle.rmsnorm_quantize_fp8(x, g, EPS)
        return oracle.gemm_fp8_decoded(aq, bf, sa, sb, out_kind=oracle.OUT_BF16)

    return step, oracle.num_threads()


def run_reference(args):
    """CPU arm: the oracle port of the step on the host cores, a bounded row sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if "RANK" in os.environ:
        # torchrun pins OMP_NUM_THREADS=1 for its workers; this arm runs on rank 0 alone
        # and is meant to use every host core (the oracle library reads it when loaded).
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    rows = 64
    step, cores = cpu_step_sample(rows)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 2.0 * rows * K * N_SHARD / dt / 1e12
    sample = f"{rows} of {M} output rows per step (RMSNorm+quantise of those rows, GEMM against the full {N_SHARD}x{K} shard)"
    _emit(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over e4m3 (CPU)", "data": "synthetic",
        "config": workload_config(args.gpus),
        "runs_on": "host cores of rank 0 only; the oracle port of the step (the reference has no CPU path for it)",
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def other_config_metrics(peaks):
    """The remaining single-GPU configurations of the path, each timed with CUDA events over
    back-to-back launches after warm-up (operands larger than L2 or rotated, as noted)."""
    import torch

    from y_b200 import quant as q
    from y_b200._lib import check, lib

    def timeit(fn, iters=20, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    out = {}
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    # fused bias + ReLU epilogue, 4096^3, bf16 out; three operand sets rotate (3 x 67 MB > L2)
    m = n = k = 4096
    sets = []
    for i in range(3):
        a = torch.randn(m, k, device="cuda", dtype=torch.float16)
        b = torch.randn(k, n, device="cuda", dtype=torch.float16)
        aq, sa = q.quantize_fp8_dynamic(a)
        bqt, sb = q.quantize_fp8_dynamic(b, transpose=True)
        sets.append((aq, bqt, sa, sb, torch.empty(m, n, dtype=torch.bfloat16, device="cuda")))
        del a, b
    bias = (torch.randn(n, device="cuda") * 0.1).to(torch.float16)
    it = [0]

    def bias_relu():
        aq, bqt, sa, sb, c = sets[it[0] % 3]
        it[0] += 1
        q.gemm_fp8_codes(aq, bqt, sa, sb, bias=bias, epilogue=q.EPI_BIAS_RELU, out_dtype=torch.bfloat16, out=c)

    us = timeit(bias_relu, iters=30)
    tf = 2.0 * m * n * k / us / 1e6
    out["fp8_gemm_4096_bias_relu_bf16"] = {"us": round(us, 2), "tflops": round(tf, 1), "frac_of_2x_bf16_peak": round(tf / fp8_peak, 4)}
    # The plain GEMM of the same operands against cuBLASLt's (torch._scaled_mm), in interleaved
    # bursts like the step's comparator: a yardstick, nothing of the product path goes through it.
    try:
        cmp_out = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(3)]

        def ours_plain():
            aq, bqt, sa, sb, c = sets[it[0] % 3]
            it[0] += 1
            q.gemm_fp8_codes(aq, bqt, sa, sb, out_dtype=torch.bfloat16, out=c)

        def lib_plain():
            aq, bqt, sa, sb, _ = sets[it[0] % 3]
            c2 = cmp_out[it[0] % 3]
            it[0] += 1
            torch._scaled_mm(aq.view(torch.float8_e4m3fn), bqt.view(torch.float8_e4m3fn).t(), scale_a=sa.reshape(()),
                             scale_b=sb.reshape(()), out_dtype=torch.bfloat16, out=c2)

        lib_plain()
        ours_us, lib_us = [], []
        for i in range(6):
            for fn, acc in ((ours_plain, ours_us), (lib_plain, lib_us)) if i % 2 == 0 else ((lib_plain, lib_us), (ours_plain, ours_us)):
                acc.append(timeit(fn, iters=12, warm=1))
        ours_us.sort(), lib_us.sort()
        mo, ml = 0.5 * (ours_us[2] + ours_us[3]), 0.5 * (lib_us[2] + lib_us[3])
        out["fp8_gemm_4096_bias_relu_bf16"]["plain_gemm_vs_cublaslt"] = {
            "ours_us": round(mo, 2), "library_us": round(ml, 2), "ours_over_library": round(ml / mo, 4),
            "what": "e4m3 x e4m3 -> bf16 without the epilogue, torch._scaled_mm on the same operands, 6 interleaved bursts of 12"}
        del cmp_out
    except Exception as e:
        out["fp8_gemm_4096_bias_relu_bf16"]["plain_gemm_vs_cublaslt"] = {"unavailable": str(e)[:200]}
    del sets
    # SwiGLU GEMM + re-quantisation, M = K = 4096, N = 2 x 11008 (gate|up interleaved)
    m, k, n = 4096, 4096, 22016
    a = torch.randn(m, k, device="cuda", dtype=torch.float16)
    aq, sa = q.quantize_fp8_dynamic(a)
    w = torch.randn(k, n, device="cuda", dtype=torch.float16)
    bqt, sb = q.quantize_fp8_dynamic(w, transpose=True)
    del a, w
    ws = torch.empty(int(q.lib.y_b200_swiglu_workspace_bytes(m, n)), dtype=torch.uint8, device="cuda")
    us = timeit(lambda: q.gemm_fp8_swiglu_requant(aq, bqt, sa, sb, workspace=ws), iters=20)
    tf = 2.0 * m * n * k / us / 1e6
    out["fp8_swiglu_requant_4096x22016x4096"] = {"us": round(us, 2), "tflops": round(tf, 1),
                                                 "frac_of_2x_bf16_peak": round(tf / fp8_peak, 4),
                                                 "includes": "GEMM with SwiGLU epilogue and amax, then the e4m3 re-quantise kernel"}
    # the whole gated MLP: SwiGLU GEMM + re-quantise + down projection 11008 -> 4096
    wd = torch.randn(n // 2, k, device="cuda", dtype=torch.float16)
    wd_t, sd = q.quantize_fp8_dynamic(wd, transpose=True)
    del wd
    mws = torch.empty(int(q.lib.y_b200_mlp_workspace_bytes(m, n // 2)), dtype=torch.uint8, device="cuda")
    o = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
    us = timeit(lambda: q.mlp_swiglu_fp8(aq, sa, bqt, sb.item(), wd_t, sd.item(), out=o, workspace=mws), iters=20)
    fl = 2.0 * m * n * k + 2.0 * m * (n // 2) * k
    out["fp8_gated_mlp_4096_h4096_i11008"] = {"us": round(us, 2), "tflops": round(fl / us / 1e6, 1),
                                              "frac_of_2x_bf16_peak": round(fl / us / 1e6 / fp8_peak, 4),
                                              "includes": "SwiGLU GEMM, e4m3 re-quantise, down projection; 3 kernels + memset"}
    del aq, bqt, ws, wd_t, mws, o
    # dynamic per-tensor quantisation of 8192 x 8192 f16 (amax + quantise: 5 bytes per element)
    x = torch.randn(8192, 8192, device="cuda", dtype=torch.float16)
    for name, tr in (("quantize_fp8_dynamic_8192x8192", False), ("quantize_fp8_dynamic_transposed_8192x8192", True)):
        us = timeit(lambda: q.quantize_fp8_dynamic(x, transpose=tr), iters=20)
        gbs = 5.0 * x.numel() / us / 1e3
        out[name] = {"us": round(us, 2), "gb_s": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
                     "bytes": "5 per element: read twice (amax, quantise), write once"}
    # fused add + RMSNorm with the residual stream, f16 in and out: 8 bytes per element
    r = torch.randn(8192, 8192, device="cuda", dtype=torch.float16)
    g = (torch.rand(8192, device="cuda") + 0.5).to(torch.float16)
    o, nr = torch.empty_like(x), torch.empty_like(x)
    us = timeit(lambda: q.fused_add_rmsnorm(x, r, g, 1e-5, out=o, new_residual=nr), iters=20)
    gbs = 8.0 * x.numel() / us / 1e3
    out["fused_add_rmsnorm_f16_8192x8192"] = {"us": round(us, 2), "gb_s": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
                                              "bytes": "8 per element: read x and residual, write out and new residual"}
    # rotary embedding, 8192 tokens x 32 heads x 128: 4 bytes per element + one position per row
    del r, o, nr
    xr = torch.randn(8192 * 32, 128, device="cuda", dtype=torch.float16)
    pos = torch.randint(0, 4096, (8192 * 32,), dtype=torch.int32, device="cuda")
    orope = torch.empty_like(xr)
    us = timeit(lambda: q.rope(xr, pos, out=orope), iters=20)
    gbs = (4.0 * xr.numel() + 4.0 * pos.numel()) / us / 1e3
    out["rope_f16_8192x32x128"] = {"us": round(us, 2), "gb_s": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4)}
    # paged decode attention, the reference fixture's heads (32 query, 8 KV, head 128, page 16),
    # 64 sequences of 4096 tokens behind a shuffled page table: K and V are each read once
    del xr, pos, orope
    ns, L, hq, hkv, hd, ps = 64, 4096, 32, 8, 128, 16
    pages = ns * (L // ps)
    kc = torch.randn(pages, ps, hkv, hd, device="cuda", dtype=torch.float16)
    vc = torch.randn(pages, ps, hkv, hd, device="cuda", dtype=torch.float16)
    qv = torch.randn(ns, hq, hd, device="cuda", dtype=torch.float16)
    pt = torch.randperm(pages, device="cuda").to(torch.int32).view(ns, L // ps)
    sl = torch.full((ns,), L, dtype=torch.int32, device="cuda")
    oa = torch.empty_like(qv)
    aws = torch.empty(max(int(q.lib.y_b200_paged_decode_attention_workspace_bytes(ns, hq, hkv, hd)), 256),
                      dtype=torch.uint8, device="cuda")
    us = timeit(lambda: q.paged_decode_attention(qv, kc, vc, pt, sl, out=oa, workspace=aws), iters=20)
    nbytes = 2.0 * ns * L * hkv * hd * 2
    out["paged_decode_attention_64x4096_h32_kv8_d128_p16"] = {
        "us": round(us, 2), "gb_s": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
        "bytes": "K and V of every sequence once (1.07 GB)"}
    # INT4 group quantisation and the repack into the streaming layout, K = 4096, N = 11008
    del qv, kc, vc, pt, sl, oa, aws
    kk, nn = DECODE_K, DECODE_N
    wsets = [(torch.randn(kk, nn, device="cuda") / 64).to(torch.float16) for _ in range(3)]  # 3 x 90 MB, rotated
    qw = torch.empty(kk // 8, nn, dtype=torch.int32, device="cuda")
    sc = torch.empty(kk // 128, nn, dtype=torch.float16, device="cuda")
    it = [0]

    def int4_q():
        w = wsets[it[0] % 3]
        it[0] += 1
        check(lib.y_b200_int4_quantize(w.data_ptr(), kk, nn, qw.data_ptr(), sc.data_ptr(), torch.cuda.current_stream().cuda_stream))

    us = timeit(int4_q, iters=30)
    nbytes = kk * nn * 2 + kk * nn // 2 + (kk // 128) * nn * 2
    out["int4_quantize_4096x11008_g128"] = {"us": round(us, 2), "gb_s": round(nbytes / us / 1e3, 1),
                                            "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
                                            "bytes": "read f16 weights once (90.2 MB), write nibbles (22.5 MB) and group scales (0.7 MB)"}
    stream = torch.empty(int(lib.y_b200_int4_stream_bytes(kk, nn)), dtype=torch.uint8, device="cuda")
    us = timeit(lambda: check(lib.y_b200_int4_repack(qw.data_ptr(), sc.data_ptr(), kk, nn, stream.data_ptr(),
                                                      torch.cuda.current_stream().cuda_stream)), iters=30)
    nbytes = 2 * stream.numel()
    out["int4_repack_4096x11008"] = {"us": round(us, 2), "gb_s": round(nbytes / us / 1e3, 1),
                                     "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
                                     "bytes": "read and write 23.2 MB each (L2-resident at this size: once per weight matrix, not a hot path)"}
    del wsets, qw, sc, stream
    # F16 family: the reference's decode fixture shape (weights [4096, 4096] f16 streamed once,
    # 16 rotating buffers = 4 x L2) through the launch API's own timing loop, under the
    # reference's .cu entry name, and the tensor-core GEMM on K-major f16 operands
    from y_b200 import runtime as rt

    ctx = rt.CudaContext.new()
    kern = ctx.load_module(None, "y_tensor_core_gemm")
    for nn2 in (4096, DECODE_N):
        wpool = [(torch.randn(4096, nn2, device="cuda") / 64).to(torch.float16) for _ in range(16 if nn2 == 4096 else 8)]
        for mtok in (1, 8, 32):
            xs = torch.randn(mtok, 4096, device="cuda", dtype=torch.float16)
            o16 = torch.empty(mtok, nn2, device="cuda", dtype=torch.float16)
            sets = [[xs.data_ptr(), wp.data_ptr(), o16.data_ptr(), ("i32", mtok), ("i32", nn2), ("i32", 4096)] for wp in wpool]
            ctx.time_launches(kern, None, None, 0, sets, len(sets))
            us = min(ctx.time_launches(kern, None, None, 0, sets, 100) for _ in range(5))
            nbytes = 4096 * nn2 * 2 + mtok * 4096 * 2 + mtok * nn2 * 2
            out[f"f16_decode_m{mtok}_4096x{nn2}"] = {"us": round(us, 2), "gb_s": round(nbytes / us / 1e3, 1),
                                                      "frac_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4), "bytes": nbytes}
        del wpool
    kern.free()
    ctx.close()
    m = n = k = 4096
    sets = [(torch.randn(m, k, device="cuda", dtype=torch.float16), (torch.randn(n, k, device="cuda") / 64).to(torch.float16),
             torch.empty(m, n, device="cuda", dtype=torch.float32)) for _ in range(2)]
    it[0] = 0

    def f16_gemm():
        a, bt, c = sets[it[0] % 2]
        it[0] += 1
        q.gemm_f16_kmajor(a, bt, out=c)

    us = timeit(f16_gemm, iters=20)
    tf = 2.0 * m * n * k / us / 1e6
    out["f16_gemm_4096_kmajor_f32_out"] = {"us": round(us, 2), "tflops": round(tf, 1),
                                           "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
                                           "note": "tcgen05 kind::f16; two rotating operand sets (2 x 134 MB)"}
    # the same product with f16 output against cuBLAS (torch.matmul), interleaved bursts
    try:
        c16 = [torch.empty(m, n, device="cuda", dtype=torch.float16) for _ in range(4)]

        def ours_f16():
            a, bt, _ = sets[it[0] % 2]
            it[0] += 1
            q.gemm_f16_kmajor(a, bt, out_dtype=torch.float16, out=c16[it[0] % 2])

        def lib_f16():
            a, bt, _ = sets[it[0] % 2]
            it[0] += 1
            torch.matmul(a, bt.t(), out=c16[2 + it[0] % 2])

        lib_f16()
        ours_us, lib_us = [], []
        for i in range(6):
            for fn, acc in ((ours_f16, ours_us), (lib_f16, lib_us)) if i % 2 == 0 else ((lib_f16, lib_us), (ours_f16, ours_us)):
                acc.append(timeit(fn, iters=12, warm=1))
        ours_us.sort(), lib_us.sort()
        mo, ml = 0.5 * (ours_us[2] + ours_us[3]), 0.5 * (lib_us[2] + lib_us[3])
        out["f16_gemm_4096_kmajor_f32_out"]["f16_out_vs_cublas"] = {
            "ours_us": round(mo, 2), "library_us": round(ml, 2), "ours_over_library": round(ml / mo, 4),
            "what": "f16 x f16 -> f16, torch.matmul on the same operands, 6 interleaved bursts of 12"}
    except Exception as e:
        out["f16_gemm_4096_kmajor_f32_out"]["f16_out_vs_cublas"] = {"unavailable": str(e)[:200]}
    q.device_status()
    return out


def decode_metrics(peaks, iters=200, n=None, tokens=(1, 4, 8, 32)):
    """INT4 decode GEMM, K=4096, N=11008 (or `n`), M in `tokens`: HBM-bound weight streaming.
    Launches are issued by the library's own timing loop (the mirror of the reference's
    time_launches) over a rotating pool of weight buffers of >= 4x L2 so every launch
    reads its weights from HBM, not L2."""
    DECODE_N = n or globals()["DECODE_N"]
    import torch

    from y_b200 import quant as q
    from y_b200 import runtime as rt
    from y_b200._lib import lib

    ctx = rt.CudaContext.new()
    l2 = ctx.device_attribute(rt.CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE) or (126 << 20)
    stream_bytes = lib.y_b200_int4_stream_bytes(DECODE_K, DECODE_N)
    free = torch.cuda.mem_get_info()[0]
    nbuf = int(lib.y_autotune_plan_weight_replicas(stream_bytes, 32 * DECODE_K * 2, 32 * DECODE_N * 2, l2, free))
    w = (torch.randn(DECODE_K, DECODE_N, device="cuda") / 64).to(torch.float16)
    qw, sc = q.int4_quantize(w)
    pool = [q.int4_repack(qw, sc) for _ in range(nbuf)]
    kern = ctx.load_module(None, "y_int4_decode_gemm")
    out = []
    for m in tokens:
        x = torch.randn(m, DECODE_K, device="cuda", dtype=torch.float16)
        o = torch.empty(m, DECODE_N, device="cuda", dtype=torch.float16)
        sets = [[x.data_ptr(), p.data_ptr(), o.data_ptr(), ("i32", m), ("i32", DECODE_N), ("i32", DECODE_K)]
                for p in pool]
        ctx.time_launches(kern, None, None, 0, sets, nbuf)  # warm-up: one pass over the pool
        best = min(ctx.time_launches(kern, None, None, 0, sets, iters) for _ in range(5))
        nbytes = stream_bytes + m * DECODE_K * 2 + m * DECODE_N * 2
        gbs = nbytes / best / 1e3
        out.append({"m": m, "us": round(best, 3), "gb_s": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
                    "bytes": nbytes})
    # what a launch that only reads the same bytes costs in the same kind of chain
    # (programmatic dependent launches over the same rotating buffers)
    floor_us = q.probe_chain_read(pool, stream_bytes, launches=iters, reps=7)
    for e in out:
        e["frac_of_bare_read"] = round(floor_us / e["us"], 4)
    q.device_status()
    kern.free()
    ctx.close()
    return {"workload": f"int4_decode_K{DECODE_K}_N{DECODE_N}_g128", "weight_buffers": nbuf,
            "l2_bytes": l2, "peak_gb_s": peaks["hbm_gbs"], "peak_source": peaks["source"], "by_m": out,
            "bare_read_same_chain": {"us": round(floor_us, 3), "gb_s": round(stream_bytes / floor_us / 1e3, 1),
                                     "frac_hbm": round(stream_bytes / floor_us / 1e3 / peaks["hbm_gbs"], 4),
                                     "what": "a kernel that only reads one weight buffer per launch, 148 CTAs x 512 "
                                             "threads, 128 KB per CTA requested before griddepcontrol.wait, launched "
                                             "as the same chain of programmatic dependent launches"}}


def bind_near_gpu(uuid: str, index: int):
    """Runs this process on the CPUs NVML lists as local to its GPU and asks the kernel to
    prefer that GPU's NUMA node for this process's pages, so that the pinned host buffers it
    allocates afterwards land in the memory next to the GPU's PCIe root: with eight ranks
    copying 134 MB per step each, buffers that all sit on one socket cross the socket link.
    Returns what was possible here: {"cpus": CPUs bound or None, "gpu_node": the GPU's NUMA
    node or None, "mems_allowed": the nodes this process may allocate on, "prefer_node": whether
    the memory policy call succeeded}. Every step is best-effort; none changes a GPU setting."""
    import ctypes

    info = {"cpus": None, "gpu_node": None, "mems_allowed": None, "prefer_node": False}
    try:
        for line in open("/proc/self/status"):
            if line.startswith("Mems_allowed_list:"):
                info["mems_allowed"] = line.split(":", 1)[1].strip()
    except OSError:
        pass
    try:
        import pynvml as nv

        nv.nvmlInit()
        try:
            h = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            h = nv.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, bits in enumerate(mask) for b in range(64) if (int(bits) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info["cpus"] = len(cpus)
        bus = nv.nvmlDeviceGetPciInfo(h).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        for cand in (bus, bus[-12:]):  # NVML prints an 8-digit domain, sysfs a 4-digit one
            path = f"/sys/bus/pci/devices/{cand}/numa_node"
            if os.path.exists(path):
                node = int(open(path).read().strip())
                info["gpu_node"] = node if node >= 0 else None
                break
    except Exception:
        pass
    if info["gpu_node"] is not None:
        try:
            libc = ctypes.CDLL(None, use_errno=True)
            MPOL_PREFERRED, SYS_set_mempolicy = 1, 238  # x86-64
            nodemask = (ctypes.c_ulong * 16)()
            nodemask[info["gpu_node"] // 64] = 1 << (info["gpu_node"] % 64)
            rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, nodemask, ctypes.c_ulong(16 * 64))
            info["prefer_node"] = rc == 0
        except Exception:
            pass
    return info


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    _uuid = str(torch.cuda.get_device_properties(local).uuid)
    placement = bind_near_gpu(("" if _uuid.startswith("GPU-") else "GPU-") + _uuid, local)

    from y_b200 import colpar
    from y_b200 import quant as q

    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    uuid = str(torch.cuda.get_device_properties(local).uuid)
    clk = ClockSampler(("" if uuid.startswith("GPU-") else "GPU-") + uuid + "|" + str(local))

    # ---- synthetic inputs (seeded; same X on every rank, a different weight shard per rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    x = torch.randn(M, K, device=dev, dtype=torch.float16, generator=gen)
    gamma = (torch.rand(K, device=dev, generator=gen) + 0.5).to(torch.float16)
    gen.manual_seed(5678 + rank)
    w = torch.randn(K, N_SHARD, device=dev, dtype=torch.float16, generator=gen)  # B [K, N] row-major
    w_amax = colpar.agree_amax(q.amax(w))  # one scale for the whole (sharded) B
    sb = q.scale_from_amax(w_amax)
    bqt = q.quantize_fp8(w, sb, transpose=True)  # [N_shard, K] e4m3, K-major
    del w
    layer = colpar.ColumnParallelFp8Linear(bqt, sb, gamma, EPS, M)
    c = torch.empty(M, N_SHARD, dtype=torch.bfloat16, device=dev)
    x_host = torch.empty(M, K, dtype=torch.float16).pin_memory()
    x_host.copy_(x.cpu())
    c_host = [torch.empty(M, N_SHARD, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    gathered = torch.empty(world, M, N_SHARD, dtype=torch.bfloat16, device=dev) if world > 1 else None

    gemm_events = []

    def step(x_dev, record=False):
        if not record:
            layer.forward(x_dev, out=c)
            return
        # the same two calls as layer.forward, with events around the GEMM
        aq, sa = q.rmsnorm_quantize_fp8(x_dev, gamma, EPS, workspace=layer._ws[0], out=layer._aq[0])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        q.gemm_fp8_codes(aq, bqt, sa, sb, out_dtype=torch.bfloat16, out=c)
        e1.record()
        gemm_events.append((e0, e1))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def gather_objects(obj):
        """[obj of rank 0, obj of rank 1, ...] on every rank."""
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def timed(fn, steps):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(max(args.warmup, 3)):
        step(x)
    q.device_status()

    # ---- device-resident timed region
    # Every fourth step has CUDA events around its GEMM (the roofline sample); the steps
    # between run as the operator launches them, kernels back to back.
    step_no = [0]

    def timed_step():
        step(x, record=step_no[0] % 4 == 0)
        step_no[0] += 1

    with clk.window("value"):
        ms = timed(timed_step, args.steps)
    ms_per_step = ms / args.steps
    flops_step = 2.0 * M * K * N_SHARD * world
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events) / len(gemm_events)
    gemm_tflops = 2.0 * M * K * N_SHARD / (gemm_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    info = q.gemm_fp8_launch_info(M, N_SHARD, K)
    gemm_kernel = ("gemm_fp8_pair_kernel<NONE, BF16> (tcgen05.mma.cta_group::2, 256x256 tile per CTA pair)"
                   if info.cta_m == 256 else f"gemm_fp8_kernel<{info.cta_n}, NONE, BF16> (128x{info.cta_n} tile per CTA)")

    # ---- a measured FP8 yardstick in the same run: cuBLASLt's e4m3 x e4m3 -> bf16 GEMM through
    # torch._scaled_mm on the same operands, timed like the GEMM above and interleaved with it so
    # both see the same clocks. A comparator only: nothing of the product path goes through it.
    comparator = None
    try:
        if args.no_comparator:
            raise RuntimeError("skipped (--no-comparator)")
        aq_c, sa_c = q.rmsnorm_quantize_fp8(x, gamma, EPS)
        a8, b8 = aq_c.view(torch.float8_e4m3fn), bqt.view(torch.float8_e4m3fn).t()
        sb_c = sb if isinstance(sb, torch.Tensor) else torch.tensor([sb], device=dev)
        sa_s, sb_s = sa_c.reshape(()), sb_c.reshape(())
        c_cmp = torch.empty(M, N_SHARD, dtype=torch.bfloat16, device=dev)

        def ours_gemm():
            q.gemm_fp8_codes(aq_c, bqt, sa_c, sb, out_dtype=torch.bfloat16, out=c)

        def lib_gemm():
            torch._scaled_mm(a8, b8, scale_a=sa_s, scale_b=sb_s, out_dtype=torch.bfloat16, out=c_cmp)

        def burst(fn, iters=10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            fn()
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters * 1e3

        lib_gemm()
        torch.cuda.synchronize()
        ours_us, lib_us = [], []
        for i in range(6):  # the order alternates so that neither side always runs on the warmer chip
            for fn, acc in ((ours_gemm, ours_us), (lib_gemm, lib_us)) if i % 2 == 0 else ((lib_gemm, lib_us), (ours_gemm, ours_us)):
                acc.append(burst(fn, 8))
        ours_us.sort(), lib_us.sort()
        flop = 2.0 * M * K * N_SHARD
        med = lambda v: 0.5 * (v[2] + v[3])
        comparator = {"what": "torch._scaled_mm (cuBLASLt) e4m3 x e4m3 -> bf16, same operands, 6 interleaved bursts of 8 each, order alternating",
                      "library_us_median": med(lib_us), "library_tflops": flop / med(lib_us) / 1e6,
                      "ours_us_median": med(ours_us), "ours_tflops": flop / med(ours_us) / 1e6,
                      "ours_over_library": med(lib_us) / med(ours_us),
                      "max_abs_diff_vs_library": float((c.float() - c_cmp.float()).abs().max())}
        del a8, b8, c_cmp
    except Exception as e:  # the yardstick is optional; the product path does not depend on it
        comparator = {"unavailable": str(e)[:200]}

    # ---- sustained: the same step back to back for about two seconds, with the clocks the
    # GPU held over that window (a burst of a few ms ends before the power cap reacts)
    sustained = None
    if args.sustained_seconds > 0:
        n_sus = max(50, int(args.sustained_seconds * 1.1 / (ms_per_step * 1e-3)))
        sus_events = []

        def sus_step(i):
            if i % 64 == 0:
                aq_s, sa_s2 = q.rmsnorm_quantize_fp8(x, gamma, EPS, workspace=layer._ws[0], out=layer._aq[0])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                q.gemm_fp8_codes(aq_s, bqt, sa_s2, sb, out_dtype=torch.bfloat16, out=c)
                e1.record()
                sus_events.append((e0, e1))
            else:
                layer.forward(x, out=c)

        with clk.window("sustained"):
            barrier()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for i in range(n_sus):
                sus_step(i)
            t1.record()
            barrier()
        sus_ms = t0.elapsed_time(t1)
        # the GEMM samples of the second half of the window: the first half is the ramp into the cap
        half = sus_events[len(sus_events) // 2:]
        sus_gemm_ms = sum(a.elapsed_time(b) for a, b in half) / len(half)
        sustained = {"seconds": sus_ms / 1e3, "steps": n_sus, "ms_per_step": sus_ms / n_sus,
                     "tflops": flops_step / (sus_ms / n_sus * 1e-3) / 1e12,
                     "gemm_us_second_half": sus_gemm_ms * 1e3,
                     "gemm_tflops_second_half": 2.0 * M * K * N_SHARD / (sus_gemm_ms * 1e-3) / 1e12}

    # ---- end to end through the operator API with host buffers: every step copies its X
    # from pinned host memory and its C back; the operator overlaps the copy-in of step
    # i+1, the kernels of step i and the copy-out of step i-1 on three streams.
    e2e_count = [0]

    def e2e_step():
        layer.submit_host(x_host, c_host[e2e_count[0] & 1])
        e2e_count[0] += 1

    def e2e_run(steps):
        for _ in range(steps):
            e2e_step()
        layer.drain()

    e2e_run(3)
    with clk.window("e2e"):
        e2e_ms = timed(lambda: e2e_run(args.steps), 1) / args.steps
    clk.close()
    clocks = clk.summary("value")
    clocks["e2e_region"] = clk.summary("e2e")
    if sustained is not None:
        sc = clk.summary("sustained")
        sustained.update({"sm_mhz": sc["sm_mhz"], "sm_mhz_min": sc["sm_mhz_min"], "reasons": sc["reasons"],
                          "power_w_max": sc["power_w_max"], "clock_samples": sc["samples"],
                          "ms_per_step_x_sm_mhz": (sustained["ms_per_step"] * sc["sm_mhz"]) if sc["sm_mhz"] else None,
                          "bf16_sustained_yardstick_tflops": peaks["bf16_tflops_sustained"],
                          "gemm_frac_of_2x_bf16_sustained": sustained["gemm_tflops_second_half"] / (2.0 * peaks["bf16_tflops_sustained"])})
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12

    # ---- what the host link itself carries: bare pinned copies of one step's output and input,
    # every rank at once (the floor the pipelined step is held against)
    def link_gbs(dst, src):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        t1.record()
        barrier()
        ms_ = torch.tensor([t0.elapsed_time(t1)], device=dev)
        if world > 1:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return world * 10 * src.numel() * src.element_size() / (ms_.item() * 1e-3) / 1e9

    def link_both_ms():
        """One step's output going out and one step's input coming in at the same time, on two
        streams, ten times: the milliseconds per pair, which is what the pipelined step can at
        best take per step when both directions of the link are busy."""
        s_out, s_in = torch.cuda.Stream(), torch.cuda.Stream()
        h2d_src = x_host if world == 1 else x_host[: x_host.shape[0] // world]
        h2d_dst = x if world == 1 else x[: x.shape[0] // world]
        barrier()
        t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        t0.record()
        s_out.wait_event(t0), s_in.wait_event(t0)
        with torch.cuda.stream(s_out):
            for _ in range(10):
                c_host[0].copy_(c, non_blocking=True)
            t1.record()
        with torch.cuda.stream(s_in):
            for _ in range(10):
                h2d_dst.copy_(h2d_src, non_blocking=True)
            t2.record()
        barrier()
        ms_ = torch.tensor([max(t0.elapsed_time(t1), t0.elapsed_time(t2)) / 10], device=dev)
        if world > 1:
            dist.all_reduce(ms_, op=dist.ReduceOp.MAX)
        return ms_.item()

    both_ms = link_both_ms()
    host_link = {"d2h_gb_s_all_ranks": link_gbs(c_host[0], c), "h2d_gb_s_all_ranks": link_gbs(x, x_host),
                 "both_directions_ms_per_step": both_ms, "e2e_ms_over_both_directions_ms": e2e_ms / both_ms,
                 "what": f"10 pinned {M * N_SHARD * 2 >> 20} MiB copies per rank, all {world} rank(s) at once, one direction at a time",
                 "e2e_bytes_gb_s_all_ranks": world * sum(layer.host_bytes_per_step()) / (e2e_ms * 1e-3) / 1e9,
                 "placement_per_rank": gather_objects(placement)}

    # ---- the exchange step, reported separately: the same step followed by NCCL's all-gather,
    # and the step whose GEMM epilogue stores its shard straight into every peer's gathered
    # buffer over NVLink (no separate collective; a one-element all-reduce orders the ranks)
    gather = None
    if world > 1:
        def gather_step():
            step(x)
            colpar.gather_columns(c, out=gathered)

        for _ in range(2):
            gather_step()
        g_ms = timed(gather_step, args.steps) / args.steps
        recv = (world - 1) * M * N_SHARD * 2
        # floor of a step that delivers the whole C to every GPU: each GPU has to take in `recv`
        # bytes over NVLink (measured peer copy on this pool: 770 GB/s per direction per GPU)
        floor_ms = max(ms_per_step, recv / 770e9 * 1e3)
        gather = {"nccl": {"ms_per_step": g_ms, "tflops": flops_step / (g_ms * 1e-3) / 1e12, "floor_over_time": floor_ms / g_ms},
                  "gathered_layout": "[rank, M, N_shard] bf16", "recv_bytes_per_gpu": recv,
                  "floor_ms": floor_ms, "floor_is": "max(step without gather, received bytes / 770 GB/s measured peer copy)"}
        fused, why = None, ""
        try:
            fused = colpar.GatheredOutput(M, N_SHARD)
        except Exception as e:  # peer mapping refused (e.g. no IPC between the ranks' containers)
            why = str(e)[:200]
        ok = torch.tensor([1.0 if fused is not None else 0.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() > 0:
            def fused_step():
                layer.forward(x, gathered=fused)
                fused.barrier()

            for _ in range(2):
                fused_step()
            f_ms = timed(fused_step, args.steps) / args.steps
            same = torch.equal(fused.to_host(), gathered.cpu())  # against NCCL's result, every rank
            agree = torch.tensor([1.0 if same else 0.0], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN)
            gather["fused_epilogue_stores"] = {"ms_per_step": f_ms, "tflops": flops_step / (f_ms * 1e-3) / 1e12,
                                               "floor_over_time": floor_ms / f_ms,
                                               "equals_nccl_result_on_every_rank": bool(agree.item() > 0)}
            fused.close()
        else:
            gather["fused_epilogue_stores"] = {"unavailable": why or "another rank could not map its peers"}
            if fused is not None:
                fused.close()
    q.device_status()

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 accumulate, bf16 out", "data": "synthetic",
            "config": workload_config(world),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "api": layer.host_api() + f", depth {layer.depth}",
                    "h2d_bytes_per_step": layer.host_bytes_per_step()[0], "d2h_bytes_per_step": layer.host_bytes_per_step()[1],
                    "bytes_are": "per rank; with N > 1 each rank copies 1/N of X from the host and the ranks "
                                 "all-gather it over NVLink",
                    "host_link": host_link},
            "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "tensor", "kernel": gemm_kernel, "achieved": gemm_tflops,
                         "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                         "peak_note": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s): the peaks file "
                                      f"holds no FP8 figure; nominal dense FP8 is {NOMINAL_FP8_TFLOPS}; a measured FP8 "
                                      "yardstick of the same run is under comparator",
                         "frac_of_nominal": gemm_tflops / NOMINAL_FP8_TFLOPS, "us_per_launch": gemm_ms * 1e3,
                         "flops_per_launch": 2.0 * M * K * N_SHARD,
                         "traffic": traffic_for(gemm_kernel, M, N_SHARD, K), "traffic_source": GEMM_TRAFFIC["source"],
                         "launches_timed": len(gemm_events), "comparator": comparator, "sustained": sustained},
        }
        if gather:
            line["gather"] = gather
    if world > 1:
        dist.barrier()
    if rank == 0 and world == 1:
        if not args.no_decode:
            # BASELINE's second metric (INT4 decode GB/s against the HBM roofline) and the other
            # single-GPU configurations travel inside `roofline`, the object the record keeps
            dec = decode_metrics(peaks)
            # the same kernel on a twice as wide weight matrix (gate and up projections as
            # one launch): the per-launch fixed latencies weigh half as much
            dec["wider"] = decode_metrics(peaks, n=2 * DECODE_N, tokens=(1, 8))
            line["roofline"]["decode"] = dec
            line["roofline"]["other_configs"] = other_config_metrics(peaks)
        if not args.no_cpu:
            rows = args.cpu_rows
            stepfn, cores = cpu_step_sample(rows)
            stepfn()
            t0 = time.perf_counter()
            reps = 0
            while time.perf_counter() - t0 < 10.0:
                stepfn()
                reps += 1
            dt = (time.perf_counter() - t0) / reps
            line["cpu_baseline"] = {
                "value": 2.0 * rows * K * N_SHARD / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"{rows} of {M} output rows per step, {reps} steps in {dt * reps:.1f} s"}
    if rank == 0:
        _emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes of one launch of the dominant kernel, keyed by what produced the figure: it is
# reported only for the kernel and shape it was captured on (a profiler run cannot be part of a
# timed benchmark, so this is the one number of the line that is not measured live).
GEMM_TRAFFIC = {"kernel_prefix": "gemm_fp8_pair_kernel<NONE, BF16>", "shape": (8192, 8192, 8192),
                "bytes": 222.0e6 + 115.3e6,
                "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at this shape "
                          "(222.0 MB + 115.3 MB; algorithmic 134.2 MB + 134.2 MB)"}


def traffic_for(kernel: str, m: int, n: int, k: int):
    if kernel.startswith(GEMM_TRAFFIC["kernel_prefix"]) and (m, n, k) == GEMM_TRAFFIC["shape"]:
        return GEMM_TRAFFIC["bytes"]
    return None


def run_only(a):
    """A few launches of one kernel family (see the module docstring), then "ok"."""
    import torch

    from y_b200 import quant as q

    torch.manual_seed(0)
    dev = "cuda"
    if a.only in ("step", "gemm", "quantize", "layer_ops"):
        x = torch.randn(a.m, a.k, device=dev, dtype=torch.float16)
    if a.only == "layer_ops":
        r = torch.randn_like(x)
        g = (torch.rand(a.k, device=dev) + 0.5).to(torch.float16)
        heads = x.view(-1, 128)  # rows of one head each
        pos = torch.randint(0, 4096, (heads.shape[0],), dtype=torch.int32, device=dev)
        for _ in range(a.iters):
            q.fused_add_rmsnorm(x, r, g, 1e-5)
            q.rope(heads, pos)
    elif a.only == "attention":
        hq, hkv, hd, ps = 32, 8, 128, 16
        pages = a.seqs * (a.seq_len // ps)
        kc = torch.randn(pages, ps, hkv, hd, device=dev, dtype=torch.float16)
        vc = torch.randn(pages, ps, hkv, hd, device=dev, dtype=torch.float16)
        qv = torch.randn(a.seqs, hq, hd, device=dev, dtype=torch.float16)
        pt = torch.randperm(pages, device=dev).to(torch.int32).view(a.seqs, a.seq_len // ps)
        sl = torch.full((a.seqs,), a.seq_len, dtype=torch.int32, device=dev)
        for _ in range(a.iters):
            q.paged_decode_attention(qv, kc, vc, pt, sl)
    elif a.only == "quantize":
        for _ in range(a.iters):
            q.quantize_fp8_dynamic(x)
            q.quantize_fp8_dynamic(x, transpose=True)
    elif a.only == "int4_quantize":
        ws = [(torch.randn(4096, DECODE_N, device=dev) / 64).to(torch.float16) for _ in range(3)]  # 3 x 90 MB
        for i in range(a.iters):
            qw, sc = q.int4_quantize(ws[i % 3])
            q.int4_repack(qw, sc)
    elif a.only in ("step", "gemm"):
        w = torch.randn(a.k, a.n, device=dev, dtype=torch.float16)
        bqt, sb = q.quantize_fp8_dynamic(w, transpose=True)
        del w
        gamma = (torch.rand(a.k, device=dev) + 0.5).to(torch.float16)
        aq, sa = q.quantize_fp8_dynamic(x)
        bias = (torch.randn(a.n, device=dev) * 0.1).to(torch.float16)
        for _ in range(a.iters):
            if a.only == "step":
                aq, sa = q.rmsnorm_quantize_fp8(x, gamma, EPS)
            if a.epilogue == "swiglu":
                q.gemm_fp8_swiglu_requant(aq, bqt, sa, sb, cta_n=a.cta_n)
            elif a.epilogue == "bias_relu":
                q.gemm_fp8_codes(aq, bqt, sa, sb, bias=bias, epilogue=q.EPI_BIAS_RELU,
                                 out_dtype=torch.bfloat16, cta_n=a.cta_n)
            else:
                q.gemm_fp8_codes(aq, bqt, sa, sb, out_dtype=torch.bfloat16, cta_n=a.cta_n)
    elif a.only == "f16_decode":
        pool = [(torch.randn(4096, 4096, device=dev) / 64).to(torch.float16) for _ in range(16)]  # 16 x 33.5 MB > 4 x L2
        xs = torch.randn(a.tokens, 4096, device=dev, dtype=torch.float16)
        for i in range(a.iters):
            q.gemm_f16_decode(xs, pool[i % len(pool)])
    else:
        k, n = DECODE_K, DECODE_N
        w = (torch.randn(k, n, device=dev) / 64).to(torch.float16)
        qw, sc = q.int4_quantize(w)
        pool = [q.int4_repack(qw, sc) for _ in range(24)]  # 24 x 23 MB > 4 x L2
        xs = torch.randn(a.tokens, k, device=dev, dtype=torch.float16)
        out = torch.empty(a.tokens, n, device=dev, dtype=torch.float16)
        for i in range(a.iters):
            q.gemm_int4_decode(xs, pool[i % len(pool)], n, out=out)
    torch.cuda.synchronize()
    q.device_status()
    _emit("ok")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--sustained-seconds", type=float, default=2.0, help="length of the sustained leg (0 = skip)")
    ap.add_argument("--only", default=None, choices=["step", "gemm", "decode", "f16_decode", "quantize", "int4_quantize", "layer_ops", "attention"],
                    help="run a few launches of one kernel family (for a profiler capture) and print ok")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--cta-n", type=int, default=0)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias_relu", "swiglu"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the INT4 decode section")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-comparator", action="store_true", help="skip the cuBLASLt FP8 yardstick (a library kernel)")
    ap.add_argument("--cpu-rows", type=int, default=64)
    ap.add_argument("--clock-sampler", default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.clock_sampler is not None:
        return clock_sampler_main(args.clock_sampler)
    # Only the JSON line may reach stdout: libraries (NCCL prints its version there) write
    # to file descriptor 1 directly, so point it at stderr and keep the real one aside.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    global _emit
    _emit = lambda text: os.write(real_stdout, (text + "\n").encode())
    if args.only is not None:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
