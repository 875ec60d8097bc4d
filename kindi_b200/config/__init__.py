from .model_config import ConfigError, ModelConfig
from .registry import (architecture, architectures, part_class, register_architecture, register_part)
from .runtime import EngineConfig, GREEDY, SamplingParams
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
