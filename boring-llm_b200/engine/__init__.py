from .runner import ModelRunner, StepEntry, OutOfPages, StepError
from .scheduler import Scheduler, Request, ScheduledStep, AdmissionError
from .engine import Engine, generate
from ..sampling.params import SamplingParams

__all__ = ["ModelRunner", "StepEntry", "OutOfPages", "StepError", "Scheduler", "Request", "ScheduledStep",
           "AdmissionError", "Engine", "generate", "SamplingParams"]
