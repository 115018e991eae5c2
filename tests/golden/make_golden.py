#!/usr/bin/env python3
"""Makes ``tests/golden/reference_kernels.safetensors``: outputs of the
reference's OWN CUDA kernels (infernum-rs/infernum, ``infernum-cuda/kernels/*.cu``)
on small random inputs, for ``tests/test_golden.py`` to hold the plain
implementation against.

The reference is a Rust workspace and cannot be built where this repository
is developed (no cargo, no rustc), so its model code cannot be run as a
whole.  Its kernels, however, are self-contained ``extern "C" __global__``
functions in plain ``.cu`` files: this script compiles those files unchanged
with nvcc, loads them through the CUDA driver API and launches the float32
variants with the launch geometry of the reference's Rust wrappers (cited at
each call).  Everything that is not a matrix product - embedding, RMSNorm,
add + RMSNorm, rotary embedding, causal grouped-query attention, SiLU * up -
is therefore the reference's code.  Matrix products (the reference
calls cuBLAS, infernum-cuda/src/inner/cuda/ops/matmul.rs:92-116) are float32
``torch.mm`` here.  The last case strings the kernels together in the order of
infernum-llama/src/graph_builder.rs:442-536 into a whole forward pass of a
tiny random model.

    python tests/golden/make_golden.py --kernels /path/to/infernum/infernum-cuda/kernels

Needs a CUDA device, nvcc and the ``cuda-python`` package; run once, the small
output file is committed.  The inputs are stored beside the outputs, so the
test needs neither a GPU nor the reference.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

DEV = "cuda:0"


class Kernels:
    """The reference's kernel files, compiled one by one and launched by name."""

    def __init__(self, folder: str):
        from cuda.bindings import driver as cu

        self.cu = cu
        self.folder = folder
        self.tmp = tempfile.mkdtemp(prefix="golden_")
        self.modules = {}
        torch.zeros(1, device=DEV)  # torch's context is the current one
        cap = torch.cuda.get_device_capability(0)
        self.arch = f"sm_{cap[0]}{cap[1]}" + ("a" if cap[0] >= 9 else "")

    def _check(self, res):
        err = res[0]
        if int(err) != 0:
            raise RuntimeError(f"CUDA driver call failed: {err}")
        return res[1] if len(res) == 2 else res[1:]

    def function(self, file: str, name: str):
        if file not in self.modules:
            src = os.path.join(self.folder, file)
            out = os.path.join(self.tmp, file.replace(".cu", ".cubin"))
            subprocess.run(["nvcc", "-cubin", f"-arch={self.arch}", "-O2", src, "-o", out], check=True)
            with open(out, "rb") as fh:
                self.modules[file] = self._check(self.cu.cuModuleLoadData(fh.read()))
        return self._check(self.cu.cuModuleGetFunction(self.modules[file], name.encode()))

    def launch(self, file: str, name: str, grid, block, shared: int, args):
        """``args``: torch tensors (passed as device pointers), ints and floats."""
        fn = self.function(file, name)
        values, types = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                values.append(a.data_ptr())
                types.append(ctypes.c_void_p)
            elif isinstance(a, float):
                values.append(a)
                types.append(ctypes.c_float)
            else:
                values.append(int(a))
                types.append(ctypes.c_int)
        grid = tuple(grid) + (1,) * (3 - len(grid))
        block = tuple(block) + (1,) * (3 - len(block))
        stream = torch.cuda.current_stream().cuda_stream
        self._check(self.cu.cuLaunchKernel(fn, *grid, *block, shared, stream, (tuple(values), tuple(types)), 0))
        torch.cuda.synchronize()


# ---- the reference's operations, launched as its Rust wrappers launch them ----------------------
def embedding(K, table, ids):
    # infernum-cuda/src/inner/cuda/ops/embed.rs:61-67
    T, H = ids.numel(), table.shape[1]
    out = torch.empty(T, H, device=DEV)
    K.launch("embed.cu", "embedding_gather_f32", (T, (H + 255) // 256), (256,), 0,
             [out, table, ids.to(torch.int32), T, H])
    return out


def rmsnorm(K, x, w, eps):
    # infernum-cuda/src/inner/cuda/ops/rmsnorm.rs:80-88
    rows, H = x.shape
    block = min(256, H)
    out = torch.empty_like(x)
    K.launch("rmsnorm.cu", "rmsnorm_f32", (rows,), (block,), 4 * ((block + 31) // 32), [out, x, w, H, float(eps)])
    return out


def add_rmsnorm(K, residual, x, w, eps):
    # infernum-cuda/src/inner/cuda/ops/add_rmsnorm.rs:80-87
    rows, H = x.shape
    block = min(256, H)
    total, normed = torch.empty_like(x), torch.empty_like(x)
    K.launch("add_rmsnorm.cu", "add_rmsnorm_f32", (rows,), (block,), 4 * ((block + 31) // 32),
             [total, normed, residual, x, w, H, float(eps)])
    return total, normed


def rope_tables(max_len, head_dim, base):
    """cos/sin caches as infernum/src/rope.rs:14-35 computes them on the host, in
    float32: freq = 1 / base^(2i / head_dim), angle = pos * freq."""
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(base), np.float32(2.0) * i / np.float32(head_dim))).astype(np.float32)
    angle = (np.arange(max_len, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return (torch.from_numpy(np.cos(angle).astype(np.float32)).to(DEV),
            torch.from_numpy(np.sin(angle).astype(np.float32)).to(DEV))


def rope(K, x, cos, sin, offset):
    # infernum-cuda/src/inner/cuda/ops/rope.rs:205-207; x is (seq, heads, head_dim)
    T, nh, hd = x.shape
    out = torch.empty_like(x)
    K.launch("rope.cu", "rope_f32", (T, nh), (hd // 2,), 0, [out, x.contiguous(), cos, sin, T, nh, hd, offset])
    return out


def attention(K, q, k, v, offset, window=-1):
    # infernum-cuda/src/inner/cuda/ops/fused_attention.rs:568-605: BR = 4, BC = 32, 128 threads
    T, nh, hd = q.shape
    total, nkv, _ = k.shape
    out = torch.empty_like(q)
    shared = 4 * (4 * hd + 32 * hd + 4 * 32)
    K.launch("flash_prefill_attention_v2.cu", "flash_prefill_attention_v2_f32", (nh, (T + 3) // 4), (128,), shared,
             [out, q.contiguous(), k.contiguous(), v.contiguous(), 1.0 / math.sqrt(hd), 0.0, total, nh, nkv, hd, T,
              offset, window])
    return out


def silu_mul(K, gate, up):
    # infernum-cuda/src/inner/cuda/ops/silu.rs:143-149
    n = gate.numel()
    out = torch.empty_like(gate)
    K.launch("silu.cu", "silu_mul_f32", ((n + 255) // 256,), (256,), 0, [out, gate.contiguous(), up.contiguous(), n])
    return out


def forward(K, cfg, W, tokens):
    """The prefill graph of infernum-llama/src/graph_builder.rs:442-536 for all
    rows: the reference's kernels for everything but the matrix products."""
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    T = len(tokens)
    cos, sin = rope_tables(cfg["max_position_embeddings"], hd, cfg["rope_theta"])
    mm = lambda a, name: torch.mm(a, W[name].t())  # noqa: E731
    h = embedding(K, W["model.embed_tokens.weight"], torch.tensor(tokens, device=DEV))
    x = rmsnorm(K, h, W["model.layers.0.input_layernorm.weight"], eps)
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}."
        q = rope(K, mm(x, p + "self_attn.q_proj.weight").view(T, nh, hd), cos, sin, 0)
        k = rope(K, mm(x, p + "self_attn.k_proj.weight").view(T, nkv, hd), cos, sin, 0)
        v = mm(x, p + "self_attn.v_proj.weight").view(T, nkv, hd)
        a = mm(attention(K, q, k, v, 0).view(T, nh * hd), p + "self_attn.o_proj.weight")
        h, x = add_rmsnorm(K, h, a, W[p + "post_attention_layernorm.weight"], eps)
        act = silu_mul(K, mm(x, p + "mlp.gate_proj.weight"), mm(x, p + "mlp.up_proj.weight"))
        d = mm(act, p + "mlp.down_proj.weight")
        nxt = f"model.layers.{n + 1}.input_layernorm.weight" if n + 1 < cfg["num_hidden_layers"] else "model.norm.weight"
        h, x = add_rmsnorm(K, h, d, W[nxt], eps)
    head = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings") else "lm_head.weight"
    return mm(x, head)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--kernels", required=True, help="the reference's infernum-cuda/kernels folder")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_kernels.safetensors"))
    args = ap.parse_args()
    from safetensors.torch import save_file

    torch.backends.cuda.matmul.allow_tf32 = False
    K = Kernels(args.kernels)
    g = torch.Generator().manual_seed(1234)
    rnd = lambda *shape: torch.randn(*shape, generator=g).to(DEV)  # noqa: E731
    out = {}
    meta = {}

    x, w = rnd(5, 96), 1.0 + 0.1 * rnd(96)
    out.update({"rmsnorm.x": x, "rmsnorm.w": w, "rmsnorm.out": rmsnorm(K, x, w, 3e-6)})
    meta["rmsnorm.eps"] = 3e-6

    r, d = rnd(4, 160), rnd(4, 160)
    w = 1.0 + 0.1 * rnd(160)
    total, normed = add_rmsnorm(K, r, d, w, 1e-5)
    out.update({"add_rmsnorm.residual": r, "add_rmsnorm.x": d, "add_rmsnorm.w": w,
                "add_rmsnorm.sum": total, "add_rmsnorm.out": normed})
    meta["add_rmsnorm.eps"] = 1e-5

    x = rnd(6, 3, 48)
    cos, sin = rope_tables(64, 48, 50000.0)
    out.update({"rope.x": x, "rope.out": rope(K, x, cos, sin, 5)})
    meta.update({"rope.theta": 50000.0, "rope.offset": 5})

    q, k, v = rnd(9, 6, 32), rnd(20, 2, 32), rnd(20, 2, 32)
    out.update({"attention.q": q, "attention.k": k, "attention.v": v,
                "attention.out": attention(K, q, k, v, 11), "attention.out_window7": attention(K, q, k, v, 11, 7)})
    meta["attention.offset"] = 11

    gate, up = 3.0 * rnd(7, 33), rnd(7, 33)
    out.update({"silu_mul.gate": gate, "silu_mul.up": up, "silu_mul.out": silu_mul(K, gate, up)})

    table = rnd(50, 24)
    ids = torch.tensor([3, 49, 0, 3, 17], device=DEV)
    out.update({"embedding.table": table, "embedding.ids": ids.to(torch.int32), "embedding.out": embedding(K, table, ids)})

    # a whole tiny model: the first of the test suite's configurations, weights from the package's
    # seeded writer (bfloat16 values widened to float32, as a float32 engine would hold them)
    sys.path.insert(0, os.path.dirname(HERE))
    from helpers import TINY_A, random_tokens
    from infernum_b200.weights.random_init import model_specs_for, random_tensors

    _, _, specs = model_specs_for(TINY_A)
    W = random_tensors(specs, 4321, DEV, torch.float32)
    tokens = random_tokens(21, TINY_A["vocab_size"], 99)
    out["model.logits"] = forward(K, TINY_A, W, tokens)
    meta.update({"model.config": "TINY_A", "model.seed": 4321, "model.tokens": tokens})

    save_file({k: v.detach().cpu().contiguous() for k, v in out.items()}, args.out,
              metadata={"meta": json.dumps(meta), "made_by": "tests/golden/make_golden.py",
                        "kernels": "infernum-rs/infernum infernum-cuda/kernels (float32 variants), unchanged"})
    print(f"wrote {args.out}: {len(out)} tensors")
    return 0


if __name__ == "__main__":
    sys.exit(main())
