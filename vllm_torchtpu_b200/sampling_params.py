"""Per-request sampling parameters (the subset of the OpenAI/vLLM surface the
engine honours: greedy and random sampling with temperature, top-k, top-p,
min-p free; logprobs; stop conditions; structured output)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

GREEDY_EPS = 1e-5


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0                      # 0 / -1 = off
    top_p: float = 1.0
    max_tokens: int = 16
    min_tokens: int = 0
    ignore_eos: bool = False
    stop_token_ids: list = field(default_factory=list)
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None
    seed: Optional[int] = None
    structured: Optional[dict] = None   # {"regex": ...} | {"json": schema} | {"choice": [...]}
    lora_name: Optional[str] = None
    pooling: Optional[str] = None        # last | mean | max | cls | all: return pooled hidden state(s) of the prompt

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_EPS

    def verify(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1:
            raise ValueError("top_k must be >= -1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
