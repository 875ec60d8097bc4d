"""kindi_b200: a small text-generation library for one NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) or seeded random weights to generated token ids, for the
Llama-arch dense Nanbeige decoder: a typed configuration and a registry, a model assembled from parts, a paged
cache with a slot per sequence, one step function, a generation loop with the reference's sampling options, a
command line (``python -m kindi_b200``) and trace replay (``bin/trace_run``). Every hot operation is a CUDA kernel
of this package; there is no CPU or library fallback.

    from kindi_b200 import Engine
    eng = Engine("model_dir", ctx=8192)                 # dtype="bfloat16" | "float32"
    eng.generate([1, 2, 3], 16)                          # 16 greedy tokens
    eng.generate_batch([[1, 2, 3], [4, 5]], temperature=0.7, top_p=0.8, top_k=20, max_tokens=64, seed=1)
"""
__version__ = "0.1.0"

from .config import (ConfigError, ConfigReader, EngineConfig, GREEDY, LayerSpec, ModelSpec, PartSpec, SamplingParams,
                     ScheduleEntry, model_from_config, model_from_dir, register_architecture, register_part)


def __getattr__(name):
    # the engine needs torch + CUDA; keep `import kindi_b200` light for tools that only read configurations
    if name in ("Engine", "StepEntry", "EngineError"):
        from .engine import engine as _e, batch as _b
        return {"Engine": _e.Engine, "StepEntry": _b.StepEntry, "EngineError": _e.EngineError}[name]
    if name == "write_random_model":
        from .weights.random_init import write_random_model
        return write_random_model
    raise AttributeError(name)
