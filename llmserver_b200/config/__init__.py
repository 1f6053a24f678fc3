from .errors import UnsupportedModelError, WeightLoadError
from .spec import PartSpec, LayerSpec, ScheduleEntry, ModelSpec
from .registry import ARCHITECTURES, Architecture, register_architecture, architecture_of, read_config
from .qwen3 import Qwen3Config, FULL_ATTENTION, SLIDING_ATTENTION
from .gefarax import GefaraxConfig
from .dikusun import DikusunConfig
from .vibepel import VibepelConfig
from .zeridra import ZeridraConfig

__all__ = ["UnsupportedModelError", "WeightLoadError", "PartSpec", "LayerSpec", "ScheduleEntry", "ModelSpec",
           "ARCHITECTURES", "Architecture", "register_architecture", "architecture_of", "read_config",
           "Qwen3Config", "GefaraxConfig", "DikusunConfig", "VibepelConfig", "ZeridraConfig", "FULL_ATTENTION", "SLIDING_ATTENTION"]
