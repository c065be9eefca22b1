from .engine import Engine
from .step import StepContext, StepEntry, StepError, StepRunner, Workspace
