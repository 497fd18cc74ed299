"""Typed configurations, the architecture registry and the model description."""
from .llama import Llama3RopeScaling, LlamaConfig  # noqa: F401
from .registry import (build_spec, config_from_dict, load_config, register_architecture,  # noqa: F401
                       registered_architectures, resolve_architecture)
from .spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, pre_norm_layer  # noqa: F401
