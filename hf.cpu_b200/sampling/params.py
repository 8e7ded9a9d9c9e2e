"""Sampling options with the reference's names, defaults and ranges (src/opts.c:57-63, :104-108)."""
from dataclasses import dataclass


@dataclass
class SamplingParams:
    temp: float = 0.8          # <= 0: greedy
    top_k: int = 40            # 0 = off
    top_p: float = 0.95        # 1 = off
    min_p: float = 0.05        # 0 = off
    seed: int = 0
    max_tokens: int = 512
    logprobs: int = 0          # top-N log-probabilities per token, at most 64

    def validate(self) -> None:
        if not 0 <= self.temp <= 5:
            raise ValueError("--temp must lie in [0, 5]")
        if not 0 <= self.top_k <= 1_000_000:
            raise ValueError("--top-k must lie in [0, 1000000]")
        if not 0 <= self.top_p <= 1 or not 0 <= self.min_p <= 1:
            raise ValueError("--top-p and --min-p must lie in [0, 1]")
        if not 1 <= self.max_tokens <= 1 << 24:
            raise ValueError("--max-tokens must lie in [1, 2^24]")
        if not 0 <= self.logprobs <= 100:
            raise ValueError("--logprobs must lie in [0, 100]")

    @property
    def greedy(self) -> bool:
        return self.temp <= 0
