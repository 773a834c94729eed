"""Sampling parameters of a request, with the reference's names, meanings and defaults
(Tokenomos api/llm.py:36-46)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_tokens: int = 256
    # 0: greedy (the first maximum)
    temperature: float = 0.0
    top_p: float = 1.0
    # 0: off
    top_k: int = 0
    min_p: float = 0.0
    seed: int = 0
    stop_token_ids: tuple[int, ...] = ()

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens {self.max_tokens}: a reply has at least one token")
        if self.temperature < 0:
            raise ValueError(f"temperature {self.temperature} is negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p {self.top_p} outside (0, 1]")
        if self.top_k < 0:
            raise ValueError(f"top_k {self.top_k} is negative")
        if not 0.0 <= self.min_p < 1.0:
            raise ValueError(f"min_p {self.min_p} outside [0, 1)")
