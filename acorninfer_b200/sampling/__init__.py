from .params import SamplingParams  # noqa: F401
