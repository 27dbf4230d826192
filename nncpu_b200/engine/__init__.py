"""Engine: the model, the step function, generation."""
from .model import Model, parameter_list, resolve_dtype
from .step import Engine, StepContext

__all__ = ["Model", "parameter_list", "resolve_dtype", "Engine", "StepContext"]
