from .engine import Engine, StepEntry

__all__ = ["Engine", "StepEntry"]
