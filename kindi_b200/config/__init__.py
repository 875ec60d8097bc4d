from .model_config import ConfigError, ConfigReader, HARMLESS_KEYS, architecture_name, read_config_json
from .registry import (architecture, architectures, model_from_config, model_from_dir, part_class,
                       register_architecture, register_part)
from .runtime import EngineConfig, GREEDY, SamplingParams
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
