"""glint_b200: a Gemma 2 inference engine for one B200, in the shape of HamadAndrabi/glint.

``LLM`` is the Python entry point (the reference's ``GlintLLM``, src/python.rs:30-148);
``python -m glint_b200`` is the command line (src/main.rs:35-287).
"""
from .errors import (GlintError, ConfigError, WeightsError, PagePoolExhausted, SlotsExhausted, KernelError,
                     RequestError)

__version__ = "0.1.0"


def __getattr__(name):
    # heavy imports (torch, the engine) only when asked for
    if name in ("LLM", "GlintLLM", "SamplingParams"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)
