from ..sampling.params import GenParams, GenStats
from .engine import Engine, TokenStream
from .scheduler import Event, Request, Scheduler, plan_batch
from .step import StepContext, StepItem, Stepper
