"""Per-request sampling parameters (the subset of the OpenAI/vLLM surface the
engine honours: greedy and random sampling with temperature, top-k, top-p and
min-p; presence / frequency / repetition penalties, logit bias and allowed
tokens; logprobs; stop tokens and stop strings; n samples per prompt;
structured output)."""
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
    n: int = 1                          # completions per prompt (expanded into n requests by the entry points)
    stop: list = field(default_factory=list)        # stop strings (matched on the detokenised text)
    include_stop_str_in_output: bool = False
    min_p: float = 0.0                  # drop tokens whose probability is below min_p x the top probability
    presence_penalty: float = 0.0       # subtracted once from every token generated so far
    frequency_penalty: float = 0.0      # subtracted per occurrence among the generated tokens
    repetition_penalty: float = 1.0     # > 1 shrinks the logits of tokens seen in prompt or output
    logit_bias: Optional[dict] = None   # {token id: additive bias}
    allowed_token_ids: Optional[list] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_EPS

    @property
    def has_penalties(self) -> bool:
        return bool(self.presence_penalty or self.frequency_penalty or self.repetition_penalty != 1.0)

    @property
    def has_logit_adjust(self) -> bool:
        """True when the logits of this request are edited in front of the sampler."""
        return bool(self.has_penalties or self.logit_bias or self.allowed_token_ids
                    or (self.min_p > 0.0 and not self.greedy))

    def verify(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1:
            raise ValueError("top_k must be >= -1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.n < 1:
            raise ValueError("n must be >= 1")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError("presence_penalty must be in [-2, 2]")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError("frequency_penalty must be in [-2, 2]")
        if not 0.0 < self.repetition_penalty <= 2.0:
            raise ValueError("repetition_penalty must be in (0, 2]")
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        if any(not isinstance(s, str) or not s for s in self.stop):
            raise ValueError("stop strings must be non-empty strings")
        if self.logit_bias:
            try:
                self.logit_bias = {int(k): float(v) for k, v in self.logit_bias.items()}
            except (TypeError, ValueError):
                raise ValueError("logit_bias maps token ids to numbers")
            if any(not -100.0 <= v <= 100.0 for v in self.logit_bias.values()):
                raise ValueError("logit_bias values must be in [-100, 100]")
        if self.allowed_token_ids is not None and not len(self.allowed_token_ids):
            raise ValueError("allowed_token_ids must not be empty")
