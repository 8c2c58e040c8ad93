"""In-house sampler: paged KV cache, continuous batching, sampling with log-prob capture."""
from .params import SamplingParams  # noqa: F401
