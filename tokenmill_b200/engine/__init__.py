from .batch import StepEntry
from .llm_engine import LLMEngine, RequestRejected
from .request import Phase, Request, RequestOutput
from .runner import ModelRunner
from .scheduler import PlanItem, Scheduler, StepPlan

__all__ = ["StepEntry", "LLMEngine", "RequestRejected", "ModelRunner", "PlanItem", "Scheduler", "StepPlan",
           "Phase", "Request", "RequestOutput"]
