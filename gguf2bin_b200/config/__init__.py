"""Configuration: typed specs, the Qwen3 reader and the architecture registry."""
from .specs import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE, Qwen3Config
from .registry import (model_spec_from_dict, model_spec_from_folder, read_config_json,
                       read_generation_stop_ids,
                       register_architecture, registered_architectures)

from .senotar import ARCHITECTURE as SENOTAR_ARCHITECTURE, senotar_model_spec

register_architecture(QWEN3_ARCHITECTURE, lambda d: Qwen3Config.from_dict(d).to_model_spec(d))
from .levolix import ARCHITECTURE as LEVOLIX_ARCHITECTURE, levolix_model_spec

from .sominex import ARCHITECTURE as SOMINEX_ARCHITECTURE, sominex_model_spec

from .mopitar import ARCHITECTURE as MOPITAR_ARCHITECTURE, mopitar_model_spec

register_architecture(SENOTAR_ARCHITECTURE, senotar_model_spec)
register_architecture(MOPITAR_ARCHITECTURE, mopitar_model_spec)
register_architecture(SOMINEX_ARCHITECTURE, sominex_model_spec)
register_architecture(LEVOLIX_ARCHITECTURE, levolix_model_spec)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "Qwen3Config",
           "QWEN3_ARCHITECTURE", "SENOTAR_ARCHITECTURE", "senotar_model_spec", "LEVOLIX_ARCHITECTURE", "levolix_model_spec", "SOMINEX_ARCHITECTURE", "sominex_model_spec", "MOPITAR_ARCHITECTURE", "mopitar_model_spec", "model_spec_from_dict", "model_spec_from_folder",
           "read_config_json", "read_generation_stop_ids", "register_architecture", "registered_architectures"]
