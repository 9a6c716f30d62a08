"""A small, whole inference engine for the Qwen2 dense decoder on one NVIDIA B200."""

from .config import Qwen2Config, load_config, register_architecture
from .engine import (LLM, Engine, GenerationConfig, LoadedModel, ModelRunner, SeqStatus,
                     StepEntry)
from .sampling import SamplingParams
from .weights import write_random_model

__version__ = "0.1.0"

__all__ = ["Qwen2Config", "load_config", "register_architecture", "LLM", "Engine",
           "GenerationConfig", "LoadedModel", "ModelRunner", "SeqStatus", "StepEntry",
           "SamplingParams", "write_random_model", "__version__"]
