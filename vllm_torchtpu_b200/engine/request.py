"""Request state tracked by the scheduler."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional

from ..sampling_params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    WAITING_FOR_REMOTE_KVS = "waiting_for_remote_kvs"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED_STOPPED = "stop"
    FINISHED_LENGTH = "length"
    FINISHED_ABORTED = "abort"
    FINISHED_ERROR = "error"

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list
    sampling_params: SamplingParams
    eos_token_id: Optional[int] = None
    arrival_time: float = field(default_factory=time.monotonic)
    kv_transfer_params: Optional[dict] = None
    priority: int = 0

    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list = field(default_factory=list)
    num_computed_tokens: int = 0        # tokens whose KV is in the cache
    num_cached_tokens: int = 0          # prefix-cache hits at admission
    block_ids: list = field(default_factory=list)
    spec_token_ids: list = field(default_factory=list)
    scheduled_time: Optional[float] = None     # first admission to the running set
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    error: Optional[str] = None
    pooled: Optional[list] = None          # pooled final hidden state (pooling requests)
    logprobs: list = field(default_factory=list)
    prompt_logprobs: list = field(default_factory=list)
    num_preemptions: int = 0
    # tokens sampled on the device that the host has not seen yet (async scheduling)
    num_output_placeholders: int = 0

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_tokens_with_placeholders(self) -> int:
        return self.num_tokens + self.num_output_placeholders

    @property
    def all_token_ids(self) -> list:
        return self.prompt_token_ids + self.output_token_ids

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    @property
    def is_prefill(self) -> bool:
        return self.num_computed_tokens < self.num_prompt_tokens

    def check_stop(self) -> bool:
        """Update status from the last appended token; True if finished."""
        sp = self.sampling_params
        n_out = len(self.output_token_ids)
        if n_out >= sp.min_tokens and n_out > 0:
            last = self.output_token_ids[-1]
            if not sp.ignore_eos and self.eos_token_id is not None and last == self.eos_token_id:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
            if last in sp.stop_token_ids:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
        if n_out >= sp.max_tokens:
            self.status = RequestStatus.FINISHED_LENGTH
            return True
        return False
