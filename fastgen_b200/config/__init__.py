from .model_args import (
    ConfigError,
    LayerSpec,
    ModelArgs,
    PartSpec,
    ScheduleEntry,
)
from .registry import (
    architectures,
    load_model_args,
    model_args_from_config,
    read_config,
    register_architecture,
)
from . import llama as _llama  # registers LlamaForCausalLM
from . import sinorax as _sinorax  # registers Sinorax
from . import zeladra as _zeladra  # registers Zeladra
from . import tanupel as _tanupel  # registers Tanupel
from . import palulorn as _palulorn  # registers Palulorn

__all__ = [
    "ConfigError",
    "LayerSpec",
    "ModelArgs",
    "PartSpec",
    "ScheduleEntry",
    "architectures",
    "load_model_args",
    "model_args_from_config",
    "read_config",
    "register_architecture",
]
