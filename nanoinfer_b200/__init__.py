"""nanoinfer_b200: a small, whole LLM inference engine for one B200 (sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed configuration
and registry, weight loader, composable parts, paged cache manager, one step function for
mixed batches, scheduler, sampling - with every forward-path kernel hand-written CUDA.
"""
__version__ = "0.1.0"
