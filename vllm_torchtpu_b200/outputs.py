"""Result objects returned by ``LLM.generate`` and the server."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class CompletionOutput:
    index: int
    token_ids: list
    text: Optional[str] = None
    finish_reason: Optional[str] = None
    logprobs: Optional[list] = None
    stop_reason: Optional[str] = None      # the stop string that ended the text, if one did


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list
    outputs: list = field(default_factory=list)
    finished: bool = True
    num_cached_tokens: int = 0
    ttft_s: Optional[float] = None
    latency_s: Optional[float] = None
    kv_transfer_params: Optional[dict] = None
    error: Optional[str] = None
    pooled: Optional[list] = None          # embedding of the prompt for pooling requests
    prompt_logprobs: Optional[list] = None  # [None, entry, ...] per prompt token when requested

    @staticmethod
    def from_request(req, detokenize=None) -> "RequestOutput":
        shown = req.output_token_ids
        sp = req.sampling_params
        if req.status.value == "stop" and shown and not getattr(sp, "include_stop_str_in_output", False) and \
                (shown[-1] in sp.stop_token_ids or shown[-1] == req.eos_token_id):
            shown = shown[:-1]              # the token that ended the completion is not part of its text
        text = detokenize(shown) if detokenize else None
        ttft = (req.first_token_time - req.arrival_time) if req.first_token_time else None
        lat = (req.finish_time - req.arrival_time) if req.finish_time else None
        return RequestOutput(
            req.request_id, req.prompt_token_ids,
            [CompletionOutput(0, list(req.output_token_ids), text, req.status.value,
                              req.logprobs or None)],
            req.status.finished, req.num_cached_tokens, ttft, lat, req.kv_transfer_params, req.error,
            getattr(req, "pooled", None), getattr(req, "prompt_logprobs", None) or None)
