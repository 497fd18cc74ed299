"""Per-request options, with the reference's names, defaults and meanings
(src/DotLLM.Core/Configuration/InferenceOptions.cs:8-71)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class InferenceOptions:
    temperature: float = 0.7            # <= 0: greedy argmax
    top_k: int = 0                      # 0: off
    top_p: float = 1.0                  # 1.0: off
    min_p: float = 0.0                  # 0: off
    repetition_penalty: float = 1.0     # 1.0: off
    repetition_penalty_window: int = 0  # 0: the whole generated history
    max_tokens: int = 2048              # cap on generated tokens, the first one included
    seed: Optional[int] = None          # None: drawn from the system's entropy per call
    stop_token_ids: Optional[Sequence[int]] = None   # None: the model's own end-of-sequence ids
    sampler_steps: Optional[Sequence] = None         # explicit chain of SamplerStep objects
    logit_processors: Optional[Sequence] = None      # explicit list of LogitProcessor objects
    stop_conditions: Optional[Sequence] = None       # explicit list of StopCondition objects

    def validate(self):
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must lie in [0, 1]")
        if self.top_p <= 0.0:
            raise ValueError("top_p must be positive")
        if self.top_k < 0:
            raise ValueError("top_k must not be negative")
        return self
