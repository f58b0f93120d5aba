from .params import SamplingParams, XorShift64  # noqa: F401
