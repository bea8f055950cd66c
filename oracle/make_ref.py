"""Builds oracle/_ref/: the reference's own kernels for this path, assembled for sm_100a.

Test infrastructure, not part of the shipped library. The reference project holds the
kernels its compiler emits for the quantised GEMM path as PTX text next to its tests
(`tests/gemm_fp8_256.ptx` and friends, `.target sm_89`, plain forward-compatible PTX).
They are the only runnable form of the reference's implementation that exists without
its Rust toolchain: the CPU back ends lower an empty kernel body.

This script runs `ptxas -arch=sm_100a` on those files where they lie in the reference
tree and writes only into oracle/_ref/: one `.cubin` per kernel and `manifest.json`
with, per kernel, the entry name, the baked shape and the launch comments the emitter
wrote into the PTX (the reference's launchers scrape the same lines:
tests/benchmark_y_swiglu_gemm.py:84-104, src/empirical_autotune.rs:317-359). Nothing
of the reference's text is copied into the repository; oracle/_ref/ is git-ignored.

The GPU parity tests load the cubins with the CUDA driver, launch them with the
geometry their own comments state and compare reference kernel, CPU oracle and this
library's kernels on the same inputs.

    python oracle/make_ref.py [reference_root]

The reference root defaults to $Y_REFERENCE_ROOT, else the directory `reference` beside
the repository. Without it (or without ptxas) the script does nothing and the tests
that need oracle/_ref/ skip.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

# file stem (under <reference>/tests) -> family
KERNELS = {
    "gemm_fp8_256": "gemm_fp8",            # BASELINE config 1
    "gemm_fp8_512": "gemm_fp8",
    "gemm_fp8_1024": "gemm_fp8",           # the large-tile variant (128x128, 256 threads)
    "gemm_f16_256": "gemm_f16",
    "gemm_f16_512": "gemm_f16",
    "tensor_core_gemm_f16_rect": "gemm_f16",
    "gemm_f16_decode_m1": "gemm_f16",
    "gemm_f16_decode_m4": "gemm_f16",
    "gemm_f16_decode_m8": "gemm_f16",
    "gemm_f16_decode_m32": "gemm_f16",
    "gemm_f16_bias_relu_64": "gemm_f16_bias_relu",
    "gemm_f16_bias_relu_512": "gemm_f16_bias_relu",
    "gemm_f16_swiglu_512": "gemm_f16_swiglu",
    "rmsnorm_residual_4096": "rmsnorm_residual",
    "rope_64": "rope",
    "rope_128": "rope",
    "rope_256": "rope",
    "paged_decode_attention_128_32_8_16": "paged_decode_attention",
    "paged_decode_attention_128_32_8_16_8": "paged_decode_attention",
}

ENTRY_RE = re.compile(r"^\.visible \.entry (\w+)\(", re.M)
SHAPE_RE = re.compile(r"M=(\d+) N=(\d+) K=(\d+)")


def reference_root(argv) -> str | None:
    cands = [argv[1]] if len(argv) > 1 else []
    if os.environ.get("Y_REFERENCE_ROOT"):
        cands.append(os.environ["Y_REFERENCE_ROOT"])
    cands.append(os.path.join(HERE, "..", "..", "reference"))
    for c in cands:
        if os.path.isdir(os.path.join(c, "tests")):
            return os.path.abspath(c)
    return None


def launch_comments(ptx: str) -> list[str]:
    """The machine-readable comment lines of a kernel: `[Y ...]` banners, the launch grid
    and the dynamic shared memory requirement."""
    keep = []
    for ln in ptx.splitlines():
        t = ln.strip()
        if t.startswith("//") and ("[Y " in t or "Launch grid required" in t or "Dynamic shared memory required" in t):
            if "ASYNC TILE LOAD" in t or "REGISTER ALLOCATOR" in t:
                continue
            keep.append(t)
    return keep


def build(root: str | None) -> int:
    if root is None:
        print("make_ref: no reference tree found; oracle/_ref/ not built")
        return 0
    ptxas = shutil.which("ptxas") or "/usr/local/cuda/bin/ptxas"
    if not os.path.exists(ptxas):
        print("make_ref: ptxas not found; oracle/_ref/ not built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    manifest = {}
    for stem, family in KERNELS.items():
        src = os.path.join(root, "tests", stem + ".ptx")
        if not os.path.exists(src):
            print(f"make_ref: {stem}.ptx is not in the reference tree, skipped")
            continue
        cubin = os.path.join(OUT, stem + ".cubin")
        r = subprocess.run([ptxas, "-arch=sm_100a", "-o", cubin, src], capture_output=True, text=True)
        if r.returncode != 0:
            print(f"make_ref: ptxas rejected {stem}.ptx:\n{r.stderr}")
            continue
        with open(src) as f:
            ptx = f.read()
        entry = ENTRY_RE.search(ptx)
        comments = launch_comments(ptx)
        shape = SHAPE_RE.search("\n".join(comments))
        static_smem = sum(int(n) for n in re.findall(r"^\s*\.shared \.align \d+ \.b8 \w+\[(\d+)\];", ptx, re.M))
        manifest[stem] = {
            "family": family,
            "entry": entry.group(1) if entry else stem,
            "cubin": os.path.basename(cubin),
            "source": f"tests/{stem}.ptx",
            "shape": [int(v) for v in shape.groups()] if shape else None,
            "static_smem_bytes": static_smem,
            "comments": comments,
        }
    with open(os.path.join(OUT, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    print(f"make_ref: {len(manifest)} reference kernels assembled for sm_100a into {OUT}")
    return 0


if __name__ == "__main__":
    sys.exit(build(reference_root(sys.argv)))
