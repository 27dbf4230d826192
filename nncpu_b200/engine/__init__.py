"""Engine: the model, the step function, generation."""
from .model import Model, parameter_list, resolve_dtype
from .step import Engine, StepContext, make_context

__all__ = ["Model", "parameter_list", "resolve_dtype", "Engine", "StepContext", "make_context"]
