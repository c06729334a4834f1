"""Golden vectors of the reference's own device kernels, for the plain implementation.

The reference's model code is Rust and cannot be built where these tests run, but its CUDA
port of one decoder layer's small operations, ``crates/vipera-backend-gpu/src/layer.cu``, is a
self-contained file of ``extern "C"`` kernels, each "a straight port of the CPU function of the
same name" (its header).  This script compiles that file unchanged with nvcc, runs its kernels
on a GPU with seeded inputs at the sizes of the two tiny test configurations, and stores inputs
and outputs in ``reference_ops.npz`` beside this script.  ``tests/test_golden.py`` then holds
every function of ``tests/plain_qwen2.py`` that has a counterpart there to those outputs, on
the CPU.

    python tests/golden/make_reference_ops.py --reference-cu <reference>/crates/vipera-backend-gpu/src/layer.cu

Kernels run: rmsnorm, rope, attention_decode, attention_split + attention_combine, swiglu,
add_inplace.  Launch shapes follow the kernels' own comments (one block per head, one thread
per value of a head, shared memory as their first lines lay it out).  The reference file is
not part of this repository and nothing of it is stored here but the numbers it computes.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import subprocess
import tempfile

import numpy as np
import torch
from cuda.bindings import driver


def _check(result):
    code = result[0]
    if int(code) != 0:
        raise RuntimeError(f"CUDA driver call failed: {code}")
    return result[1] if len(result) == 2 else result[1:]


class Module:
    def __init__(self, source: str):
        out = os.path.join(tempfile.mkdtemp(prefix="vipera_golden_"), "layer.cubin")
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-cubin", "-o", out, source], check=True)
        torch.zeros(1, device="cuda")  # makes torch's context current
        with open(out, "rb") as handle:
            self.module = _check(driver.cuModuleLoadData(handle.read()))

    def launch(self, name: str, grid, block, shared_bytes: int, *args):
        function = _check(driver.cuModuleGetFunction(self.module, name.encode()))
        values, kinds = [], []
        for arg in args:
            if isinstance(arg, torch.Tensor):
                values.append(arg.data_ptr())
                kinds.append(ctypes.c_void_p)
            elif isinstance(arg, int):
                values.append(arg)
                kinds.append(ctypes.c_int)
            else:
                values.append(float(arg))
                kinds.append(ctypes.c_float)
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        _check(driver.cuLaunchKernel(function, *grid, *block, shared_bytes, 0, (tuple(values), tuple(kinds)), 0))
        torch.cuda.synchronize()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference-cu", required=True)
    parser.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_ops.npz"))
    args = parser.parse_args()
    module = Module(args.reference_cu)
    rng = torch.Generator().manual_seed(20240607)
    saved = {}

    def rand(*shape, scale=1.0):
        return (torch.randn(*shape, generator=rng) * scale).float()

    # rmsnorm: one block, shared = one float per thread
    for tag, n, eps in (("a", 256, 1e-6), ("b", 384, 1e-5)):
        x, w = rand(n), 1.0 + rand(n, scale=0.01)
        out = torch.empty(n, device="cuda")
        module.launch("rmsnorm", (1,), (128,), 128 * 4, x.cuda(), w.cuda(), out, n, eps)
        saved.update({f"rmsnorm_{tag}_x": x, f"rmsnorm_{tag}_w": w, f"rmsnorm_{tag}_eps": np.float32(eps),
                      f"rmsnorm_{tag}_out": out.cpu()})

    # rope: one block per head, in place
    for tag, heads, d, base, position in (("a", 4, 64, 10000.0, 37), ("b", 3, 128, 1000000.0, 301), ("c", 2, 64, 10000.0, 0)):
        x = rand(heads, d)
        v = x.clone().cuda()
        module.launch("rope", (heads,), (32,), 0, v, position, heads, d, base)
        saved.update({f"rope_{tag}_x": x, f"rope_{tag}_base": np.float32(base), f"rope_{tag}_position": np.int32(position),
                      f"rope_{tag}_out": v.cpu()})

    # attention for one new position over dense 32-bit keys and values [positions, kv_heads, d]
    for tag, heads, kv_heads, d, positions in (("a", 4, 2, 64, 77), ("b", 3, 1, 128, 130)):
        q, k, v = rand(heads, d), rand(positions, kv_heads, d), rand(positions, kv_heads, d)
        scale = 1.0 / float(np.sqrt(np.float32(d)))
        qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
        out = torch.empty(heads, d, device="cuda")
        module.launch("attention_decode", (heads,), (d,), (positions + d) * 4, qd, kd, vd, out, positions, heads, kv_heads, d, scale)
        saved.update({f"attn_{tag}_q": q, f"attn_{tag}_k": k, f"attn_{tag}_v": v, f"attn_{tag}_out": out.cpu()})
        # the split form: chunks of 32 positions, then the combine
        chunk = 32
        chunks = (positions + chunk - 1) // chunk
        group = heads // kv_heads
        partial = torch.zeros(heads * (2 * chunks + chunks * d), device="cuda")
        shared = (d + group * chunk + group * (d // 32) + 2 * group) * 4
        module.launch("attention_split", (kv_heads, chunks), (group * d,), shared, qd, kd, vd, partial, positions, chunk, chunks,
                      heads, kv_heads, d, scale)
        out2 = torch.empty(heads, d, device="cuda")
        module.launch("attention_combine", (heads,), (d,), 0, partial, out2, chunks, heads, d)
        saved[f"attn_{tag}_split_out"] = out2.cpu()

    # swiglu and the residual addition
    gate, up = rand(704, scale=2.0), rand(704)
    out = torch.empty(704, device="cuda")
    module.launch("swiglu", (4,), (128,), 0, gate.cuda(), up.cuda(), out, 704)
    saved.update({"swiglu_gate": gate, "swiglu_up": up, "swiglu_out": out.cpu()})
    a, b = rand(256), rand(256)
    ad = a.clone().cuda()
    module.launch("add_inplace", (2,), (128,), 0, ad, b.cuda(), 256)
    saved.update({"add_a": a, "add_b": b, "add_out": ad.cpu()})

    np.savez(args.out, **{key: (value.numpy() if isinstance(value, torch.Tensor) else value) for key, value in saved.items()})
    print(f"wrote {args.out}: {len(saved)} arrays")


if __name__ == "__main__":
    main()
