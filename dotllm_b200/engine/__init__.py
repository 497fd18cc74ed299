"""The step function, the generation loop above it, and trace replay."""
from .generate import InferenceResponse, InferenceTimings, TextGenerator, plan_batches  # noqa: F401
from .step import AttentionPlan, StepContext, StepEntry, plan_step, run_step  # noqa: F401
