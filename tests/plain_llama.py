"""A plain, slow implementation of the Llama dense decoder, written from the
reference's formulas.  Whole sequences, no cache, one function per part, CPU
tensors only.  It shares no code with the package under test: it parses
config.json by itself and reads the checkpoint with the ``safetensors``
library.

The reference is a Rust workspace and neither cargo nor rustc exists here, so
its model code cannot be compiled or imported as a whole.  Its CUDA kernels
can: ``tests/golden/make_golden.py`` compiled the reference's unchanged ``.cu``
files and ran their float32 variants once on a GPU - each part, and a whole
forward pass of a tiny random model with the reference's kernels for everything
but the matrix products - and ``tests/test_golden.py`` holds the functions
below against those outputs.  What the reference does not have (llama3
frequency scaling) rests on the formula alone.  Each function cites the
reference file and lines it restates.

Precision: weights are taken as stored (bfloat16 values widened exactly) and
all arithmetic runs in ``dtype`` (float64 by default), except rotation angles,
which are formed the way the engine and the reference form them: a float32
product of the integer position and a float32 frequency.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------
# configuration (infernum-llama/src/config.rs:19-126: keys and defaults)
# --------------------------------------------------------------------------
def read_config(folder_or_dict) -> dict:
    if isinstance(folder_or_dict, dict):
        raw = dict(folder_or_dict)
    else:
        with open(os.path.join(folder_or_dict, "config.json")) as fh:
            raw = json.load(fh)
    c = {
        "vocab_size": raw["vocab_size"],
        "hidden_size": raw["hidden_size"],
        "intermediate_size": raw["intermediate_size"],
        "num_hidden_layers": raw["num_hidden_layers"],
        "num_attention_heads": raw["num_attention_heads"],
    }
    c["num_key_value_heads"] = raw.get("num_key_value_heads") or c["num_attention_heads"]  # config.rs:258-260
    c["head_dim"] = raw.get("head_dim") or c["hidden_size"] // c["num_attention_heads"]  # config.rs:264-266
    c["rms_norm_eps"] = raw.get("rms_norm_eps", 1e-5)  # config.rs:112-114
    c["rope_theta"] = raw.get("rope_theta", 10000.0)  # config.rs:116-118
    c["rope_scaling"] = raw.get("rope_scaling")
    c["tie_word_embeddings"] = raw.get("tie_word_embeddings", False)
    return c


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    out = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            out.update(load_file(os.path.join(folder, name)))
    return out


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h[t, :] = E[id_t, :], no scaling (infernum-cuda/kernels/embed.cu:36-50)."""
    return table[torch.tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """(x * rsqrt(mean(x^2) + eps)) * w (infernum-cuda/kernels/rmsnorm.cu:64-94)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * inv) * w


def rope_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_j = theta^(-2j/hd) (infernum/src/rope.rs:24-27); llama3 scaling is the
    three-band ramp of the reference's YaRN branch (infernum/src/rope.rs:91-120)
    with configurable bounds and without its magnitude factor.  Returned as
    float32, the precision frequencies have on the device."""
    half = head_dim // 2
    f = [theta ** (-(2.0 * j) / head_dim) for j in range(half)]
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
        orig = scaling["original_max_position_embeddings"]
        low_wavelen, high_wavelen = orig / low, orig / high
        g = []
        for fj in f:
            wavelen = 2 * math.pi / fj
            if wavelen < high_wavelen:
                g.append(fj)
            elif wavelen > low_wavelen:
                g.append(fj / factor)
            else:
                ramp = (orig / wavelen - low) / (high - low)
                g.append((1 - ramp) * fj / factor + ramp * fj)
        f = g
    return torch.tensor(f, dtype=torch.float64).to(torch.float32)


def rope(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, heads, hd]; pairs (j, j+hd/2): y_j = x_j c - x_{j+hd/2} s,
    y_{j+hd/2} = x_j s + x_{j+hd/2} c (infernum-cuda/kernels/rope.cu:25-41);
    angle = (pos as f32) * f_j in f32 (infernum/src/rope.rs:25-29)."""
    half = x.shape[-1] // 2
    angle = positions.to(torch.float32)[:, None] * freqs[None, :]  # float32 product
    c = torch.cos(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    s = torch.sin(angle.to(torch.float64)).to(x.dtype)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """q [T, nh, hd], k, v [T, nkv, hd] of one whole sequence.  Head a reads kv
    head a / (nh / nkv); scores (q.k)/sqrt(hd); keys j <= p (and, with a
    window, j > p - window); softmax with max subtraction; sum of P v
    (infernum-cuda/kernels/flash_prefill_attention_v2.cu:82-95,149-192;
    infernum-cuda/kernels/paged_decode_attention.cu:540-644)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window > 0:
        allowed &= pos[None, :] > pos[:, None] - window
    for a in range(nh):
        g = a // group
        s = (q[:, a, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, a, :] = p @ v[:, g, :]
    return out


def swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g))
    (infernum-llama/src/graph_builder.rs:498-501; infernum-cuda/kernels/silu.cu:105-116)."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1 + torch.exp(-g))) * u) @ wd.T


# --------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
            dtype: torch.dtype = torch.float64, collect: Optional[dict] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (infernum-llama/src/graph_builder.rs:442-536,
    for all rows instead of the last one)."""
    W = lambda name: weights[name].to(dtype)  # noqa: E731
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    T = len(tokens)
    positions = torch.arange(T)
    freqs = rope_frequencies(hd, cfg["rope_theta"], cfg["rope_scaling"])
    h = embedding(W("model.embed_tokens.weight"), tokens)
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}."
        x = rms_norm(h, W(p + "input_layernorm.weight"), eps)
        q = (x @ W(p + "self_attn.q_proj.weight").T).view(T, nh, hd)
        k = (x @ W(p + "self_attn.k_proj.weight").T).view(T, nkv, hd)
        v = (x @ W(p + "self_attn.v_proj.weight").T).view(T, nkv, hd)
        q, k = rope(q, positions, freqs), rope(k, positions, freqs)
        a = attention(q, k, v).reshape(T, nh * hd) @ W(p + "self_attn.o_proj.weight").T
        h = h + a
        m = rms_norm(h, W(p + "post_attention_layernorm.weight"), eps)
        h = h + swiglu(m, W(p + "mlp.gate_proj.weight"), W(p + "mlp.up_proj.weight"),
                       W(p + "mlp.down_proj.weight"))
        if collect is not None:
            collect[f"layer{n}"] = h.clone()
    f = rms_norm(h, W("model.norm.weight"), eps)
    head = "model.embed_tokens.weight" if (cfg["tie_word_embeddings"]
                                           or "lm_head.weight" not in weights) else "lm_head.weight"
    return f @ W(head).T


# --------------------------------------------------------------------------
# sampling (infernum-cuda/src/inner/cuda/ops/sample.rs:86-160)
# --------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> int:
    """The first maximum wins (infernum-cpu/src/logits.rs:40-53)."""
    best, idx = None, 0
    for i, v in enumerate(logits.tolist()):
        if best is None or v > best:
            best, idx = v, i
    return idx


def sample_probabilities(logits: torch.Tensor, temperature: float, top_p: float,
                         penalty: float, recent: Sequence[int]) -> torch.Tensor:
    """The distribution the reference samples from: repetition penalty once per
    occurrence (sample.rs:96-110), temperature (:113), softmax (:116-119),
    nucleus = shortest prefix of the descending order whose mass reaches top_p
    (:123-136), renormalised (:139-141).  Returns probabilities over the
    vocabulary with zeros outside the nucleus."""
    x = logits.to(torch.float64).clone()
    if abs(penalty - 1.0) > 1e-7:
        for t in recent:
            if 0 <= t < x.numel():
                x[t] = x[t] / penalty if x[t] > 0 else x[t] * penalty
    x = x / temperature
    p = torch.exp(x - x.max())
    p = p / p.sum()
    order = torch.argsort(p, descending=True, stable=True)
    cum = torch.cumsum(p[order], dim=0)
    end = int(torch.searchsorted(cum, torch.tensor(top_p, dtype=cum.dtype)).item()) + 1 \
        if top_p < 1.0 else p.numel()
    end = min(end, p.numel())
    kept = torch.zeros_like(p)
    kept[order[:end]] = p[order[:end]]
    return kept / kept.sum()


def sample_index_order(probs: torch.Tensor, u: float) -> int:
    """Inverse CDF over the kept tokens walked in order of index."""
    acc = 0.0
    last = 0
    for i, p in enumerate(probs.tolist()):
        if p > 0:
            last = i
            acc += p
            if u < acc:
                return i
    return last


def uniform_number(seed: int, n_generated: int) -> float:
    """The uniform number of a request's next token: state = seed ^ tokens
    generated so far (infernum-runtime/src/engine.rs:283,406), one xorshift64
    round (engine.rs:491-494), then + 1 and four more rounds, u = state / 2^64
    (infernum-cuda/src/inner/cuda/ops/sample.rs:143-149)."""
    mask = (1 << 64) - 1

    def xorshift(s: int) -> int:
        s ^= (s << 13) & mask
        s ^= s >> 7
        s ^= (s << 17) & mask
        return s & mask

    s = xorshift((int(seed) ^ int(n_generated)) & mask)
    s = (s + 1) & mask
    for _ in range(4):
        s = xorshift(s)
    return s / float(1 << 64)


def greedy_generate(cfg: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int],
                    n_new: int, dtype=torch.float64) -> List[int]:
    """Recomputes the whole sequence for every new token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, weights, seq, dtype)
        t = argmax(logits[-1])
        out.append(t)
        seq.append(t)
    return out
