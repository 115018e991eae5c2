"""Token selection on the device, and the uniform numbers it consumes.

Greedy: argmax, lowest index among equal logits.  Sampling: the reference's
pipeline - repetition penalty over the recent window, temperature, softmax,
nucleus (top-p), inverse CDF (infernum-cuda/src/inner/cuda/ops/sample.rs:86-160)
- as one kernel per batch of rows.

The uniform number of a token is a function of (seed, number of tokens the
request has generated so far), as in the reference: state = seed ^ n_generated
(infernum-runtime/src/engine.rs:283,406), one xorshift64 round
(engine.rs:484-506), then +1 and four more rounds, u = state / 2^64
(sample.rs:143-149).  So a request's stream does not depend on the batch it is
in, nor on having been preempted and recomputed.
"""

from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..ops import core
from .params import SamplingParams

_M64 = (1 << 64) - 1


def _xorshift64(s: int) -> int:
    s ^= (s << 13) & _M64
    s ^= s >> 7
    s ^= (s << 17) & _M64
    return s & _M64


def uniform_for(seed: int, n_generated: int) -> float:
    """The uniform number in [0, 1) for a request's next token."""
    s = (int(seed) ^ int(n_generated)) & _M64
    s = _xorshift64(s)
    s = (s + 1) & _M64
    for _ in range(4):
        s = _xorshift64(s)
    u = s / float(1 << 64)
    return min(u, 1.0 - 2.0 ** -24)  # stays below 1 after rounding to float32


def recent_window(tokens: Sequence[int], params: Optional[SamplingParams]) -> Sequence[int]:
    """The last ``repetition_penalty_window`` tokens (engine.rs:508-512)."""
    w = params.repetition_penalty_window if params else 0
    return tokens[len(tokens) - w:] if w else []


def pack_choices(choices: Sequence[Optional[tuple]], width: Optional[int] = None):
    """Host tensors for the sampling kernel: params [R, 6] float32 (temperature,
    top_p, penalty, u, count of recent tokens as int bits, pad), recent tokens
    [R, width] int32, and which rows sample at all."""
    R = len(choices)
    if width is None:
        width = max([len(c[2]) for c in choices if c is not None] + [1])
    # (filled through numpy: a row costs a microsecond, not the ten of tensor indexing)
    params = np.zeros((R, core.SAMPLE_PARAM_FLOATS), dtype=np.float32)
    recent = np.zeros((R, width), dtype=np.int32)
    n_recent = np.zeros(R, dtype=np.int32)
    mask = np.zeros(R, dtype=np.bool_)
    for i, c in enumerate(choices):
        if c is None:
            params[i, :3] = 1.0
            continue
        sp, n_gen, rec = c
        params[i, :4] = (sp.temperature, sp.top_p, sp.repetition_penalty, uniform_for(sp.seed, n_gen))
        if len(rec):
            rec = list(rec)[-width:]
            recent[i, : len(rec)] = rec
            n_recent[i] = len(rec)
        mask[i] = True
    params.view(np.int32)[:, 4] = n_recent
    return torch.from_numpy(params), torch.from_numpy(recent), torch.from_numpy(mask)


class Sampler:
    """Selects one token per logits row.  ``choices[i]`` is None for greedy or
    a tuple (SamplingParams, n_generated, recent tokens)."""

    def __init__(self, device):
        self.device = device

    def select(self, logits: torch.Tensor, choices: Sequence[Optional[tuple]]) -> torch.Tensor:
        """Returns int32 token ids [R] on the device."""
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        core.argmax(logits, out)
        if all(c is None for c in choices):
            return out
        params, recent, mask = pack_choices(choices)
        dev = logits.device
        sampled = torch.empty(R, dtype=torch.int32, device=dev)
        core.sample(logits, params.to(dev), recent.to(dev), sampled)
        return torch.where(mask.to(dev), sampled, out)
