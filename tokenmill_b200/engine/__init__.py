from .batch import StepEntry
from .llm_engine import LLMEngine, RequestRejected
from .runner import ModelRunner
from .scheduler import PlanItem, Scheduler, StepPlan
from .sequence import RequestOutput, Sequence, Status

__all__ = ["StepEntry", "LLMEngine", "RequestRejected", "ModelRunner", "PlanItem", "Scheduler", "StepPlan",
           "RequestOutput", "Sequence", "Status"]
