from .batch import StepEntry, StepPlan, plan_step
from .engine import Engine
from .generate import Backend, EngineBackend, Stats, run_generation
from .model import DecoderModel, expected_tensors_for_config, model_for_config
from .profile import StepProfile

__all__ = ["Backend", "DecoderModel", "Engine", "EngineBackend", "Stats", "StepEntry", "StepProfile", "StepPlan", "expected_tensors_for_config",
           "model_for_config", "plan_step", "run_generation"]
