from .batch import StepContext, StepEntry, build_context
from .engine import Engine, load_engine
from .runner import ModelRunner, OutOfPages, parse_dtype
from .scheduler import PlannedEntry, Request, Scheduler, StepPlan
