from .engine import Engine, StepError, resolve_dtype  # noqa: F401
