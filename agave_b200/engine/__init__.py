from .batch import DECODE, PREFILL, StepContext
from .generate import GenerationPlan, RequestState
from .step import Runner, StepError

__all__ = ["DECODE", "PREFILL", "StepContext", "GenerationPlan", "RequestState", "Runner",
           "StepError"]
