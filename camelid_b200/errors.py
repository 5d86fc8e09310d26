"""Typed errors of the library. Every error is raised before any device work is queued,
so a failed call leaves the cache as it was (the reference asserts the same in
tests/inference_session.rs:409-543; its typed errors are in src/error.rs:3-69)."""


class CamelidError(Exception):
    """Base class of every error this library raises on purpose."""


class ConfigError(CamelidError):
    """A key of config.json, a parameter of a part or an option is missing, of the wrong
    type or outside its range. ``key`` names it."""

    def __init__(self, key: str, message: str):
        self.key = key
        super().__init__(f"configuration: {key}: {message}")


class UnknownArchitectureError(CamelidError):
    """config.json names an architecture that no model is registered for."""


class WeightsError(CamelidError):
    """The tensors of a model folder do not fit the model: one error lists everything."""

    def __init__(self, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, expected, got)
        self.other = list(other)
        lines = ["model weights do not fit the configuration:"]
        if self.missing:
            lines.append("  missing tensors: " + ", ".join(self.missing))
        if self.unexpected:
            lines.append("  unexpected tensors: " + ", ".join(self.unexpected))
        for name, expected, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name}: expected {list(expected)}, got {list(got)}")
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


class SafetensorsError(CamelidError):
    """A safetensors file is malformed."""


class CacheError(CamelidError):
    """No free slot or page, an unknown slot, a slot freed twice, or a sequence too long."""


class StepError(CamelidError):
    """A step's input is not acceptable (empty, token id outside the vocabulary, a wanted
    place outside the step's tokens, mixed phases)."""


class KernelError(CamelidError):
    """A CUDA kernel refused a size, the extension is missing, or a launch failed."""


class SamplingError(CamelidError):
    """A sampling option is outside its range, or the logits are not finite."""
