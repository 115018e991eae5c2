"""Sampling and generation options, with the reference's names, meanings and
defaults (infernum/src/sampling.rs:4-60): ``SamplingParams`` for nucleus
sampling, ``GenerateOptions`` for the generation loop; ``sampling=None`` means
greedy decoding.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.9
    seed: int = 42
    repetition_penalty: float = 1.0
    repetition_penalty_window: int = 64

    def __post_init__(self):
        if not self.temperature > 0:
            raise ConfigError("temperature must be > 0 (use sampling=None for greedy decoding)")
        if not 0 < self.top_p <= 1:
            raise ConfigError("top_p must be in (0, 1]")
        if not self.repetition_penalty > 0:
            raise ConfigError("repetition_penalty must be > 0")
        if self.repetition_penalty_window < 0:
            raise ConfigError("repetition_penalty_window must be >= 0")


@dataclass(frozen=True)
class GenerateOptions:
    max_new_tokens: int = 100
    eos_token_id: Optional[int] = None
    sampling: Optional[SamplingParams] = None
    use_kv_cache: bool = True  # kept for the reference's option set; the cache is always used
    ignore_eos: bool = False  # benchmarks: run to max_new_tokens
