"""Per-step batch description handed to every attention layer.

Same fields as the reference's metadata
(reference: src/vllm_torchtpu/layers/core/attention_metadata.py:83-141):
the batch is ordered ``[decode][spec-verify][prefill/mixed]`` and
``request_distribution = (decode_end, verify_end, num_reqs)``.  Padded requests
have ``q_len == 0`` because the padded tail of ``query_start_loc`` repeats the
last valid value (reference: src/vllm_torchtpu/runner/tpu_runner.py:3513-3519).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class AttentionMetadata:
    positions: torch.Tensor            # [T] int32/int64
    slot_mapping: torch.Tensor         # [T] int32, -1 = padding
    block_tables: torch.Tensor         # [R, max_blocks] int32
    seq_lens: torch.Tensor             # [R] int32
    query_start_loc: torch.Tensor      # [R+1] int32
    num_reqs: int                      # real requests (host value)
    num_tokens: int                    # real tokens (host value)
    num_decode_reqs: int = 0           # leading requests with q_len == 1
    max_query_len: int = 1
    max_seq_len: int = 0
    logits_indices: Optional[torch.Tensor] = None   # [R] rows whose logits are needed
    request_distribution: tuple = (0, 0, 0)
    # context-parallel extras
    dcp_rank: int = 0
    dcp_size: int = 1
    dcp_interleave: int = 1
    global_seq_lens: Optional[torch.Tensor] = None   # [R] true lengths when seq_lens are a rank's local share
    # state slots for linear-attention layers (one per request)
    state_slots: Optional[torch.Tensor] = None
    # verification step on a hybrid: recurrent layers hand their snapshots and inputs to this object
    state_rollback: Optional[object] = None
    pcp: Optional[object] = None          # PcpStepPlan of a step whose prefill chunks are split over PCP ranks
    # padded sizes when running inside a captured graph
    padded_num_reqs: Optional[int] = None
    padded_num_tokens: Optional[int] = None
    # host copies for kernels that plan work on the CPU
    seq_lens_cpu: Optional[torch.Tensor] = None
    query_start_loc_cpu: Optional[torch.Tensor] = None

    @property
    def is_decode_only(self) -> bool:
        return self.num_decode_reqs == self.num_reqs
