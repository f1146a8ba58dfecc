"""kvcm: a small, whole, single-GPU inference engine for the Llama dense decoder on B200
(sm_100a), with the capabilities of the kvpage reference: typed config and registry, weights
from safetensors, layers put together from parts, a paged cache manager, one step function for
mixed batches, a continuous-batching scheduler with chunked prefill, sampling, hand-written CUDA
kernels, a true float32 path and trace replay.

    import kvcm
    eng = kvcm.Engine.from_folder("model_dir", kvcm.EngineConfig(dtype="bfloat16"))
    rid = eng.add_request([1, 5, 9], max_new_tokens=16)
    while not eng.idle():
        eng.step()
    print(eng.take_finished()[0].generated())
"""
from . import config, models, parts, weights
from .config import (ConfigError, EngineConfig, KVManagerConfig, LlamaConfig, SchedulerConfig,
                     load_config, register_architecture, registered_architectures)
from .weights import WeightError, write_random_model


def __getattr__(name):
    # Engine pieces import torch.cuda-facing modules; resolve them lazily so that configuration,
    # weights and the CPU core can be used without touching a GPU.
    if name in ("Engine", "ModelRunner", "load_model", "generate"):
        from . import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)


__all__ = ["config", "models", "parts", "weights", "ConfigError", "EngineConfig",
           "KVManagerConfig", "LlamaConfig", "SchedulerConfig", "load_config",
           "register_architecture", "registered_architectures", "WeightError",
           "write_random_model", "Engine", "ModelRunner", "load_model", "generate"]
