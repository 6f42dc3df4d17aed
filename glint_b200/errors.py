"""Error types of the engine.

The reference reports every failure as one typed value, ``GlintError``
(src/error.rs:12-86); the classes here keep its cases that an engine without
GGUF, server or tokenizer still meets.
"""
from __future__ import annotations


class GlintError(Exception):
    """Base of all engine errors."""


class ConfigError(GlintError):
    """config.json is unreadable, lacks a required key, or asks for something unsupported
    (reference: HfInvalidJson, HfMissingConfigField, HfUnsupported)."""


class WeightsError(GlintError):
    """The weight file is malformed or does not fit the model.

    ``missing``, ``unexpected`` and ``wrong_shape`` list every offending tensor at once
    (reference: TensorNotFound, InvalidTensorShape, SafeTensorsMalformed,
    SafeTensorsUnsupportedDtype raise on the first one found).
    """

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


class PagePoolExhausted(GlintError):
    """Not enough free cache pages (reference: KvPagePoolExhausted{needed, available, capacity},
    src/error.rs:78-82).  Recoverable: nothing was taken."""

    def __init__(self, group, needed, available, capacity):
        super().__init__(
            f"cache pages exhausted in group '{group}': needed {needed}, available {available}, "
            f"capacity {capacity}")
        self.group, self.needed, self.available, self.capacity = group, needed, available, capacity


class SlotsExhausted(GlintError):
    """No free per-request state slot."""


class KernelError(GlintError):
    """The CUDA extension is missing, failed to build, refused a size, or a launch failed."""


class RequestError(GlintError):
    """A request is invalid: empty prompt, token id out of range, context exceeded."""
