"""Device communicator for vLLM process groups: NCCL through ``torch.distributed`` for everything,
except small bf16 all-reduces of the tensor-parallel group, which run as one kernel over the
symmetric NVLink heap (two-shot, bounded flag waits) the way the native engine's decode path does.
Same role as the reference's communicator (reference: src/vllm_torchtpu/distributed/tpu_communicator.py:35-93)."""
from __future__ import annotations

from typing import Optional

import torch
from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase

from .. import envs
from ..logger import init_logger
from ..parallel.state import Group

logger = init_logger(__name__)


class B200Communicator(DeviceCommunicatorBase):
    def __init__(self, cpu_group, device: Optional[torch.device] = None, device_group=None, unique_name: str = "",
                 **kwargs):
        super().__init__(cpu_group, device, device_group, unique_name, **kwargs)
        self.heap = None
        self._heap_failed = False
        self.peer_all_reduce_max_bytes = int(envs.B200_TP_ONE_SHOT_BYTES)

    def _ensure_heap(self):
        """Symmetric heap of this group, created on first use (tensor-parallel groups on GPUs only)."""
        if self.heap is not None or self._heap_failed:
            return self.heap
        if (self.world_size == 1 or self.world_size > 8 or self.unique_name.split(":")[0] != "tp"
                or not torch.cuda.is_available() or envs.B200_TP_COMM == "nccl"):
            self._heap_failed = True
            return None
        try:
            from ..parallel.symm_heap import SymmetricHeap
            grp = Group("tp", list(self.ranks), self.rank_in_group, self.device_group, self.cpu_group)
            self.heap = SymmetricHeap.create(grp, 96 * 2**20)
        except Exception as e:                              # noqa: BLE001 - fall back to NCCL
            logger.warning("peer-memory all-reduce unavailable (%r): using NCCL", e)
            self._heap_failed = True
        return self.heap

    def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
        if (input_.is_cuda and input_.dtype == torch.bfloat16 and input_.is_contiguous()
                and 0 < input_.numel() * 2 <= self.peer_all_reduce_max_bytes
                and not torch.cuda.is_current_stream_capturing()):
            heap = self._ensure_heap()
            if heap is not None:
                from ..ops import cuda
                out = input_.clone()
                return cuda.p2p_all_reduce(out, heap)
        out = input_.clone()
        torch.distributed.all_reduce(out, group=self.device_group)
        return out
