"""Typed configuration, the architecture registry and the named shapes."""
from .furesun import ARCHITECTURE as FURESUN_ARCHITECTURE
from .furesun import MODEL_TYPE as FURESUN_MODEL_TYPE
from .furesun import FuresunConfig, build_furesun_spec
from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .pavisun import ARCHITECTURE as PAVISUN_ARCHITECTURE
from .pavisun import MODEL_TYPE as PAVISUN_MODEL_TYPE
from .pavisun import PavisunConfig, build_pavisun_spec
from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .qwen2 import MODEL_TYPE as QWEN2_MODEL_TYPE
from .qwen2 import Qwen2Config, build_qwen2_spec, read_config_json
from .registry import (Architecture, register_architecture, registered_architectures, resolve,
                       spec_from_config_dict, unregister_architecture)
from .rirudra import ARCHITECTURE as RIRUDRA_ARCHITECTURE
from .rirudra import MODEL_TYPE as RIRUDRA_MODEL_TYPE
from .rirudra import RirudraConfig, build_rirudra_spec
from .shapes import named_shape, shape_names
from .zodosun import ARCHITECTURE as ZODOSUN_ARCHITECTURE
from .zodosun import MODEL_TYPE as ZODOSUN_MODEL_TYPE
from .zodosun import ZodosunConfig, build_zodosun_spec

register_architecture(
    Architecture(QWEN2_ARCHITECTURE, QWEN2_MODEL_TYPE, Qwen2Config, build_qwen2_spec), replace=True)

register_architecture(
    Architecture(ZODOSUN_ARCHITECTURE, ZODOSUN_MODEL_TYPE, ZodosunConfig, build_zodosun_spec), replace=True)

register_architecture(
    Architecture(RIRUDRA_ARCHITECTURE, RIRUDRA_MODEL_TYPE, RirudraConfig, build_rirudra_spec), replace=True)

register_architecture(
    Architecture(PAVISUN_ARCHITECTURE, PAVISUN_MODEL_TYPE, PavisunConfig, build_pavisun_spec), replace=True)

register_architecture(
    Architecture(FURESUN_ARCHITECTURE, FURESUN_MODEL_TYPE, FuresunConfig, build_furesun_spec), replace=True)

__all__ = [
    "FuresunConfig", "build_furesun_spec",
    "PavisunConfig", "build_pavisun_spec",
    "RirudraConfig", "build_rirudra_spec",
    "Architecture", "ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "Qwen2Config", "ScheduleEntry",
    "ZodosunConfig", "build_zodosun_spec",
    "build_qwen2_spec", "named_shape", "read_config_json", "register_architecture",
    "registered_architectures", "resolve", "shape_names", "spec_from_config_dict", "unregister_architecture",
]
