"""Writes tests/golden/ref_kernels.npz: outputs of the reference's own kernels (oracle/_ref/,
assembled from its PTX fixtures by oracle/make_ref.py) on seeded inputs, produced on a B200.

Run on a machine with a GPU and oracle/_ref/ built:
    python tests/golden/make_ref_golden.py [out.npz]
Only outputs are stored; tests/test_ref_golden.py rebuilds the inputs from the same seeds
through `golden_inputs` below and holds the CPU oracle against these outputs, so the CPU-only
suite pins the oracle to what the reference's kernels computed.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import oracle  # noqa: E402


def probe_values(count, scale, seed):
    """Every midpoint between adjacent e4m3 values and its f32 neighbours, values past +-448,
    tiny values, then seeded normals; all times `scale`."""
    vals = oracle.decode_e4m3(np.arange(256, dtype=np.uint8))
    pos = np.sort(vals[np.isfinite(vals) & (vals >= 0)])
    mids = ((pos[:-1].astype(np.float64) + pos[1:].astype(np.float64)) / 2).astype(np.float32)
    special = np.concatenate([mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)),
                              np.float32([448, 449, 464, 465, 480, 1000, 1e4, 1e-3, 2e-3, 9.7e-4, 0.0])])
    special = np.concatenate([special, -special]).astype(np.float32) * np.float32(scale)
    out = (np.random.default_rng(seed).standard_normal(count) * 3.0).astype(np.float32)
    out[:special.size] = special
    return out


def golden_inputs():
    """name -> dict of input arrays (and scalars), a pure function of fixed seeds."""
    g = {}
    m = n = k = 256
    g["fp8_probe_a"] = {"a": probe_values(m * k, 0.0123, 7).reshape(m, k), "b": np.eye(k, dtype=np.float32), "sa": 0.0123, "sb": 1.0}
    g["fp8_probe_a_exact"] = {"a": probe_values(m * k, 0.25, 7).reshape(m, k), "b": np.eye(k, dtype=np.float32), "sa": 0.25, "sb": 1.0}
    g["fp8_probe_b"] = {"a": np.eye(k, dtype=np.float32), "b": probe_values(k * n, 0.31, 8).reshape(k, n), "sa": 1.0, "sb": 0.31}
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    b = (rng.standard_normal((k, n)) * 3).astype(np.float32)
    g["fp8_random"] = {"a": a, "b": b, "sa": oracle.scale_from_amax(oracle.amax_f32(a)), "sb": oracle.scale_from_amax(oracle.amax_f32(b))}
    g["f16_gemm_256"] = {"a": oracle.fill_normal_f16(m * k, oracle.SEED_A + 12).reshape(m, k),
                         "b": oracle.fill_normal_f16(k * n, oracle.SEED_B + 12, 1.0 / 16).reshape(k, n)}
    g["f16_bias_relu_64"] = {"a": oracle.fill_normal_f16(64 * 64, oracle.SEED_A + 5).reshape(64, 64),
                             "b": oracle.fill_normal_f16(64 * 64, oracle.SEED_B + 5, 1.0 / 8).reshape(64, 64),
                             "bias": (np.random.default_rng(9).standard_normal(64) * 0.5).astype(np.float32)}
    kk = 512
    g["f16_swiglu_512"] = {"x": oracle.fill_normal_f16(kk * kk, oracle.SEED_A + 21).reshape(kk, kk),
                           "wg": oracle.fill_normal_f16(kk * kk, oracle.SEED_B + 21, 1.0 / np.sqrt(kk)).reshape(kk, kk),
                           "wu": oracle.fill_normal_f16(kk * kk, oracle.SEED_B + 22, 1.0 / np.sqrt(kk)).reshape(kk, kk)}
    rows, hidden = 8, 4096
    g["rmsnorm_residual_4096"] = {"x": oracle.fill_normal_f16(rows * hidden, 41).reshape(rows, hidden),
                                  "res": oracle.fill_normal_f16(rows * hidden, 42).reshape(rows, hidden),
                                  "w": oracle.fill_uniform_f16(hidden, 43, 0.5, 1.5)}
    pos = np.random.default_rng(128).integers(0, 4096, size=64).astype(np.int32)
    pos[:4] = [0, 1, 4095, 2048]
    g["rope_128"] = {"x": oracle.fill_normal_f16(64 * 128, 51 + 128).reshape(64, 128), "pos": pos}
    hd, hq, hkv, ps, num_pages = 128, 32, 8, 16, 64
    seq_lens = [0, 1, 7, 63, 64, 65, 200, 33]
    ns = len(seq_lens)
    max_pages = max(1, max((x + ps - 1) // ps for x in seq_lens))
    prng = np.random.default_rng(5)
    g["paged_decode_attention"] = {
        "q": oracle.fill_normal_f16(ns * hq * hd, 61).reshape(ns, hq, hd),
        "k": oracle.fill_normal_f16(num_pages * ps * hkv * hd, 62).reshape(num_pages, ps, hkv, hd),
        "v": oracle.fill_normal_f16(num_pages * ps * hkv * hd, 63).reshape(num_pages, ps, hkv, hd),
        "pt": np.stack([prng.permutation(num_pages)[:max_pages] for _ in range(ns)]).astype(np.int32),
        "sl": np.array(seq_lens, np.int32), "max_pages": max_pages}
    return g


def main():
    import torch

    import ref_kernels
    from helpers import f16_dev, host_bits

    rk = ref_kernels.RefKernels()
    g = golden_inputs()
    out = {}

    def gemm(name, ptrs, m, n):
        kr = rk.get(name)
        c = torch.full((m, n), float("nan"), device="cuda")
        grid, block, smem = kr.gemm_geometry()
        kr.launch(grid, block, smem, [*ptrs, c.data_ptr()])
        torch.cuda.synchronize()
        return c.cpu().numpy()

    for case in ("fp8_probe_a", "fp8_probe_a_exact", "fp8_probe_b", "fp8_random"):
        i = g[case]
        a, b = torch.from_numpy(i["a"]).cuda(), torch.from_numpy(i["b"]).cuda()
        out[case] = gemm("gemm_fp8_256", [a.data_ptr(), b.data_ptr(), float(i["sa"]), float(i["sb"])], 256, 256)
    i = g["f16_gemm_256"]
    a, b = f16_dev(i["a"]), f16_dev(i["b"])
    out["f16_gemm_256"] = gemm("gemm_f16_256", [a.data_ptr(), b.data_ptr()], 256, 256)
    i = g["f16_bias_relu_64"]
    a, b, bias = f16_dev(i["a"]), f16_dev(i["b"]), torch.from_numpy(i["bias"]).cuda()
    out["f16_bias_relu_64"] = gemm("gemm_f16_bias_relu_64", [a.data_ptr(), b.data_ptr(), bias.data_ptr()], 64, 64)
    i = g["f16_swiglu_512"]
    x, wg, wu = f16_dev(i["x"]), f16_dev(i["wg"]), f16_dev(i["wu"])
    out["f16_swiglu_512_rows0_32"] = gemm("gemm_f16_swiglu_512", [x.data_ptr(), wg.data_ptr(), wu.data_ptr()], 512, 512)[:32].copy()
    i = g["rmsnorm_residual_4096"]
    x, res, w = f16_dev(i["x"]), f16_dev(i["res"]), f16_dev(i["w"])
    o, nr = torch.zeros(8, 4096, dtype=torch.float16, device="cuda"), torch.zeros(8, 4096, dtype=torch.float16, device="cuda")
    rk.get("rmsnorm_residual_4096").launch((8, 1, 1), (256, 1, 1), 0, [x.data_ptr(), res.data_ptr(), w.data_ptr(), o.data_ptr(), nr.data_ptr()])
    torch.cuda.synchronize()
    out["rmsnorm_out"], out["rmsnorm_new_residual"] = host_bits(o), host_bits(nr)
    i = g["rope_128"]
    x, pos = f16_dev(i["x"]), torch.from_numpy(i["pos"]).cuda()
    o = torch.zeros(64, 128, dtype=torch.float16, device="cuda")
    rk.get("rope_128").launch((64, 1, 1), (32, 1, 1), 0, [x.data_ptr(), pos.data_ptr(), o.data_ptr()])
    torch.cuda.synchronize()
    out["rope_128"] = host_bits(o)
    i = g["paged_decode_attention"]
    q, k, v = f16_dev(i["q"]), f16_dev(i["k"]), f16_dev(i["v"])
    pt, sl = torch.from_numpy(i["pt"]).cuda(), torch.from_numpy(i["sl"]).cuda()
    o = torch.zeros(8, 32, 128, dtype=torch.float16, device="cuda")
    rk.get("paged_decode_attention_128_32_8_16").launch((32, 8, 1), (1024, 1, 1), 0,
                                                        [q.data_ptr(), k.data_ptr(), v.data_ptr(), pt.data_ptr(), sl.data_ptr(),
                                                         o.data_ptr(), ("i32", int(i["max_pages"]))])
    torch.cuda.synchronize()
    out["paged_decode_attention"] = host_bits(o)
    rk.close()
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_kernels.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
