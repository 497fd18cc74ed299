"""Sampling: options, the sampler pipeline over device kernels, stop conditions, RNG."""
from .options import InferenceOptions  # noqa: F401
from .pipeline import (CategoricalSampler, LogitProcessor, MinPSampler, RepetitionPenaltyProcessor,  # noqa: F401
                       SamplerPipeline, SamplerStep, TemperatureSampler, TopKSampler, TopPSampler)
from .rng import uniform  # noqa: F401
from .stop import (EosStopCondition, FinishReason, MaxTokensStopCondition, StopCondition, StopResult,  # noqa: F401
                   check_stop_conditions)
