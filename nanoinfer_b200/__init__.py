"""nanoinfer_b200: a small, whole LLM inference engine for one B200 (sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed configuration
and registry, weight loader, composable parts, paged cache manager, one step function for
mixed batches, scheduler, sampling - with every forward-path kernel hand-written CUDA.

    from nanoinfer_b200 import Engine, SamplingParams
    engine = Engine.from_model_dir("path/to/model", dtype="bfloat16")
    out = engine.generate([[1, 5, 9]], max_new_tokens=16, sampling_params=SamplingParams.greedy())
"""
from .engine import Engine, EngineConfig
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["Engine", "EngineConfig", "SamplingParams"]
