"""Model assembly, the step function, the scheduler and the entry point."""
from .model import CausalLM
from .step import Engine, StepEntry, StepContext

__all__ = ["CausalLM", "Engine", "StepEntry", "StepContext"]
