from .batch import StepContext, StepEntry, build_context
from .runner import ModelRunner, OutOfPages, parse_dtype
