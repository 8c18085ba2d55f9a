"""nanoinfer_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a)."""
from .api import Model, generate, load_model
from .config import EngineConfig
from .engine.scheduler import Request, Scheduler
from .sampling.params import SamplingParams

__version__ = "0.1.0"
__all__ = ["Model", "generate", "load_model", "EngineConfig", "Request", "Scheduler", "SamplingParams"]
