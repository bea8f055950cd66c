"""Loader for the reference's own kernels (oracle/_ref/, built by oracle/make_ref.py).

Test infrastructure. The cubins are the reference compiler's emitted PTX, assembled for
sm_100a unchanged. They are loaded with the CUDA driver into the process's primary
context (the one torch uses) and launched with exactly the geometry their own comments
state, the way the reference's launchers do (tests/test_fp8_gemm_correctness.py:40-44
for the FP8 family, whose grid.x walks M; tests/benchmark_y_swiglu_gemm.py:84-104 for
the F16 families, whose grid.x walks N; tests/benchmark_y_rmsnorm_rope.py:87,155 and
tests/benchmark_y_paged_decode_attention.py:188-189 for the rest).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
MANIFEST = os.path.join(REF_DIR, "manifest.json")

CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8


def available() -> bool:
    return os.path.exists(MANIFEST)


def manifest() -> dict:
    with open(MANIFEST) as f:
        return json.load(f)


class RefKernel:
    def __init__(self, owner, name, meta, fn):
        self.owner, self.name, self.meta, self.fn = owner, name, meta, fn
        self.text = "\n".join(meta["comments"])
        self.shape = tuple(meta["shape"]) if meta["shape"] else None

    def dyn_smem(self) -> int:
        m = re.search(r"Dynamic shared memory required: (\d+) bytes", self.text)
        return int(m.group(1)) if m else 0

    def gemm_geometry(self):
        """(grid, block, dynamic shared bytes) of a GEMM-family kernel, from its comments."""
        fam = self.meta["family"]
        if fam == "gemm_fp8":
            m = re.search(r"Launch grid required: \((\d+), (\d+), (\d+)\) CTAs, block \((\d+),1,1\)", self.text)
            g = tuple(int(v) for v in m.groups())
            return g[:3], (g[3], 1, 1), 0
        m = re.search(r"M=(\d+) N=(\d+) K=(\d+) \| CTA (\d+)x(\d+)x(\d+)[^|]*\| (\d+)x(\d+) warps", self.text)
        M, N, _, cta_m, cta_n, _, wm, wn = (int(v) for v in m.groups())
        return ((N + cta_n - 1) // cta_n, (M + cta_m - 1) // cta_m, 1), (wm * wn * 32, 1, 1), self.dyn_smem()

    def launch(self, grid, block, smem, args, stream=0):
        """args: ints are 64-bit device pointers, floats are f32, ('i32', v) is a 32-bit int."""
        self.owner.launch(self.fn, grid, block, smem, args, stream)


class RefKernels:
    def __init__(self):
        import torch

        torch.cuda.init()
        torch.zeros(1, device="cuda")  # the primary context exists and is current on this thread
        self.cu = C.CDLL("libcuda.so.1")
        self._check(self.cu.cuInit(0), "cuInit")
        ctx = C.c_void_p()
        self._check(self.cu.cuCtxGetCurrent(C.byref(ctx)), "cuCtxGetCurrent")
        if not ctx.value:
            dev = C.c_int()
            self._check(self.cu.cuDeviceGet(C.byref(dev), torch.cuda.current_device()), "cuDeviceGet")
            self._check(self.cu.cuDevicePrimaryCtxRetain(C.byref(ctx), dev), "cuDevicePrimaryCtxRetain")
            self._check(self.cu.cuCtxSetCurrent(ctx), "cuCtxSetCurrent")
        self.meta = manifest()
        self._mods = {}

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    def get(self, name) -> RefKernel:
        meta = self.meta[name]
        if name not in self._mods:
            with open(os.path.join(REF_DIR, meta["cubin"]), "rb") as f:
                image = f.read()
            mod, fn = C.c_void_p(), C.c_void_p()
            self._check(self.cu.cuModuleLoadData(C.byref(mod), image), f"cuModuleLoadData({name})")
            self._check(self.cu.cuModuleGetFunction(C.byref(fn), mod, meta["entry"].encode()), "cuModuleGetFunction")
            self._mods[name] = (mod, fn)
        return RefKernel(self, name, meta, self._mods[name][1])

    def launch(self, fn, grid, block, smem, args, stream=0):
        if smem > 48 * 1024:
            self._check(self.cu.cuFuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, C.c_int(smem)),
                        "cuFuncSetAttribute(max dynamic shared)")
        store = []
        for a in args:
            if isinstance(a, tuple) and a[0] == "i32":
                store.append(C.c_int32(int(a[1])))
            elif isinstance(a, float):
                store.append(C.c_float(a))
            else:
                store.append(C.c_uint64(int(a)))
        params = (C.c_void_p * len(store))(*[C.cast(C.pointer(s), C.c_void_p) for s in store])
        self._check(self.cu.cuLaunchKernel(fn, C.c_uint(grid[0]), C.c_uint(grid[1]), C.c_uint(grid[2]),
                                           C.c_uint(block[0]), C.c_uint(block[1]), C.c_uint(block[2]),
                                           C.c_uint(smem), C.c_void_p(stream), params, None), "cuLaunchKernel")

    def close(self):
        for mod, _ in self._mods.values():
            self.cu.cuModuleUnload(mod)
        self._mods = {}
