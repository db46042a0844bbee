from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep
from .qwen3 import ARCHITECTURE, QwenConfig, read_config_json
from .registry import (config_class_for, config_from_dict, config_from_model_dir,
                       register_architecture, registered_architectures, unregister_architecture)

register_architecture(ARCHITECTURE, QwenConfig)
