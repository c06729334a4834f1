"""Sampling options of one request, with the reference's names, meanings and defaults
(crates/vipera-sampler/src/lib.rs:36-70; the command line sets temperature 0 by default,
bins/vipera/src/main.rs:554-560)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


@dataclass
class SamplingParams:
    max_new_tokens: int = 32           # --max-tokens
    temperature: float = 0.0           # 0 selects greedy and skips every other filter
    top_k: int = 40                    # 0: no cut
    top_p: float = 0.95
    min_p: float = 0.05
    repetition_penalty: float = 1.0    # 1.0: off
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Optional[Sequence[Tuple[int, float]]] = None  # at most 16 (id, bias) pairs
    seed: int = 0
    eos_ids: Optional[Sequence[int]] = None  # None: the model configuration's end tokens
    recent_window: int = 128           # tokens the penalties look back over
    # None: no log-probabilities.  n >= 0: every generated token comes with its log-probability
    # under the distribution it was drawn from (penalties and temperature applied, no cut), and
    # with the n most likely tokens and theirs (crates/vipera-sampler/src/lib.rs:302-378).
    logprobs: Optional[int] = None

    def to_native(self, default_eos: Sequence[int] = ()) -> dict:
        return {
            "max_new_tokens": int(self.max_new_tokens),
            "temperature": float(self.temperature),
            "top_k": int(self.top_k),
            "top_p": float(self.top_p),
            "min_p": float(self.min_p),
            "repetition_penalty": float(self.repetition_penalty),
            "presence_penalty": float(self.presence_penalty),
            "frequency_penalty": float(self.frequency_penalty),
            "logit_bias": None if self.logit_bias is None else [(int(i), float(b)) for i, b in self.logit_bias],
            "seed": int(self.seed),
            "eos_ids": list(default_eos if self.eos_ids is None else self.eos_ids),
            "recent_window": int(self.recent_window),
        }
