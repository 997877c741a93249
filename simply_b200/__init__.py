"""simply_b200: a single-GPU inference engine for the Gemma 2 dense decoder on NVIDIA B200."""

from simply_b200.config import EngineConfig, load_config, preset
from simply_b200.engine import Engine, GenerationResult, StepEntry
from simply_b200.sampling import SamplingParams

__all__ = ["Engine", "EngineConfig", "GenerationResult", "SamplingParams", "StepEntry",
           "load_config", "preset"]
__version__ = "0.1.0"
