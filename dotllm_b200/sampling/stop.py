"""Stop conditions, checked after each generated token is appended
(src/DotLLM.Engine/TextGenerator.cs:248-262, 904-915)."""
from __future__ import annotations

from enum import Enum


class StopResult(Enum):
    """src/DotLLM.Core/Sampling/StopResult.cs:6-16"""
    CONTINUE = 0
    STOP = 1            # stop and drop the token just generated
    STOP_INCLUDE = 2    # stop and keep it


class FinishReason(str, Enum):
    """src/DotLLM.Engine/FinishReason.cs:6-16"""
    STOP = "stop"
    LENGTH = "length"


class StopCondition:
    def should_stop(self, token_id, generated):
        raise NotImplementedError


class EosStopCondition(StopCondition):
    """A stop token ends generation and is not part of the output
    (src/DotLLM.Engine/Samplers/StopConditions/EosStopCondition.cs:9-25).  Takes a set of ids:
    Llama 3 checkpoints list several."""

    def __init__(self, token_ids):
        self.token_ids = frozenset(int(t) for t in token_ids)

    def should_stop(self, token_id, generated):
        return StopResult.STOP if token_id in self.token_ids else StopResult.CONTINUE


class MaxTokensStopCondition(StopCondition):
    """The token that reaches the cap is kept
    (src/DotLLM.Engine/Samplers/StopConditions/MaxTokensStopCondition.cs:9-25)."""

    def __init__(self, max_tokens):
        self.max_tokens = int(max_tokens)

    def should_stop(self, token_id, generated):
        return StopResult.STOP_INCLUDE if len(generated) >= self.max_tokens else StopResult.CONTINUE


def check_stop_conditions(conditions, token_id, generated):
    """First condition that does not say CONTINUE wins (TextGenerator.cs:904-915)."""
    for c in conditions:
        r = c.should_stop(token_id, generated)
        if r != StopResult.CONTINUE:
            return r
    return StopResult.CONTINUE
