from .runtime import Runtime, parse_dtype
from .context import StepContext
from .runner import DeviceFault, ModelRunner, StepEntry
from .scheduler import PlanItem, Scheduler, SeqStatus
from .engine import Engine, LoadedModel
from .llm import LLM, GenerationConfig, read_eos_id

__all__ = ["Runtime", "parse_dtype", "StepContext", "DeviceFault", "ModelRunner", "StepEntry",
           "PlanItem", "Scheduler", "SeqStatus", "Engine", "LoadedModel", "LLM",
           "GenerationConfig", "read_eos_id"]
