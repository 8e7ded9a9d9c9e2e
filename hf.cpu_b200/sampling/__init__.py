from .host import logprob, sample_host, top_logprobs
from .params import SamplingParams
from .rng import Rng, next_state, seed_state, uniform_of_state

__all__ = ["SamplingParams", "Rng", "sample_host", "logprob", "top_logprobs", "seed_state", "next_state",
           "uniform_of_state"]
from . import device  # noqa: E402,F401
