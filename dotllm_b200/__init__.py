"""dotllm_b200: a small inference library for one NVIDIA B200, with the shape of kkokosa/dotLLM.

    from dotllm_b200 import Model, InferenceOptions
    model = Model.load("model_dir", dtype="bfloat16")
    out = model.generate([1, 2, 3], InferenceOptions(temperature=0, max_tokens=16))
"""
from .errors import (CacheError, CacheFullError, ConfigError, DotLlmError, KernelError, StepError,  # noqa: F401
                     WeightsError)
from .sampling.options import InferenceOptions  # noqa: F401
from .engine.step import StepEntry  # noqa: F401
from .model import Model, ModelLoader  # noqa: F401

__version__ = "0.1.0"
