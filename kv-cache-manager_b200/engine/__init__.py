"""Engine: model loading, the step function, the request loop above the scheduler."""
from .model_io import load_model, model_from_tensors, torch_dtype
from .runner import ModelRunner

__all__ = ["load_model", "model_from_tensors", "torch_dtype", "ModelRunner", "Engine", "generate"]


def __getattr__(name):
    if name in ("Engine", "generate", "FinishedRequest", "StepInfo"):
        from . import engine as _e
        return getattr(_e, name)
    raise AttributeError(name)
