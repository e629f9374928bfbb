from .engine import Engine
from .step import StepContext, StepItem, Stepper
