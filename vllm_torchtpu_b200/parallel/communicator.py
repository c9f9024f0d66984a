"""Device communicator: collectives over a process group with three data planes.

* ``nccl`` – ``torch.distributed`` (NCCL on GPUs, gloo in CPU tests); the
  baseline and the fallback.
* ``p2p``  – hand-written kernels over a symmetric heap of peer-mapped buffers
  (NVLink loads/stores + flag waits with an iteration limit).
* ``multimem`` – as ``p2p`` but reductions go through NVSwitch multicast.

The MoE ``dispatch``/``combine`` pair has the reference's semantics
(reference: src/vllm_torchtpu/distributed/tpu_communicator.py:35-93): dispatch
all-gathers hidden states, top-k weights and ids over the group, combine
reduce-scatters the expert output back; the fused EP kernel replaces both.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import envs
from ..logger import init_logger
from .state import Group, get_state

logger = init_logger(__name__)


class DeviceCommunicator:
    def __init__(self, group: Group, symm_heap=None):
        self.group = group
        self.heap = symm_heap
        self.plane = envs.B200_TP_COMM if symm_heap is not None else "nccl"

    @property
    def size(self) -> int:
        return self.group.size

    @property
    def rank(self) -> int:
        return self.group.rank_in_group

    # ---- plain collectives ---------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if (self.heap is not None and self.plane != "nccl" and x.is_cuda and x.dtype == torch.bfloat16
                and x.numel() * 2 <= self.heap.ar_stage_bytes):
            # small tensors: one kernel over the peer heap; larger ones exceed its staging buffer
            from ..ops import cuda_ops
            return cuda_ops().p2p_all_reduce(x, self.heap)
        dist.all_reduce(x, group=self.group.device_group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.size == 1:
            return x
        dim = dim % x.dim()
        # the concatenated output form is accepted by NCCL and gloo alike
        flat = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x.contiguous(), group=self.group.device_group)
        out = flat.view((self.size,) + tuple(x.shape))
        if dim == 0:
            return out.reshape((self.size * x.shape[0],) + tuple(x.shape[1:]))
        out = out.movedim(0, dim)
        shape = list(x.shape)
        shape[dim] *= self.size
        return out.reshape(shape)

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        if self.size == 1:
            return x
        x = x.movedim(dim, 0).contiguous()
        assert x.shape[0] % self.size == 0
        if not x.is_cuda:
            # gloo has no reduce-scatter: reduce everything, keep this rank's slice
            dist.all_reduce(x, group=self.group.device_group)
            n = x.shape[0] // self.size
            return x[self.rank * n:(self.rank + 1) * n].movedim(0, dim)
        out = torch.empty((x.shape[0] // self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=self.group.device_group)
        return out.movedim(0, dim)

    def all_to_all(self, x: torch.Tensor, split_dim: int = 0, concat_dim: int = 0) -> torch.Tensor:
        """Split ``split_dim`` into group-size pieces, exchange, concatenate on ``concat_dim``
        (the head<->token exchange of linear-attention layers under context parallelism,
        reference: src/vllm_torchtpu/distributed/collectives.py:24-31)."""
        if self.size == 1:
            return x
        pieces = [p.contiguous() for p in x.chunk(self.size, dim=split_dim)]
        if not x.is_cuda:
            # gloo: gather everybody's pieces, keep the ones addressed to this rank
            stacked = torch.stack(pieces, 0)
            every = torch.empty((self.size * self.size,) + tuple(pieces[0].shape), dtype=x.dtype)
            dist.all_gather_into_tensor(every, stacked, group=self.group.device_group)
            every = every.view((self.size, self.size) + tuple(pieces[0].shape))
            return torch.cat([every[src, self.rank] for src in range(self.size)], dim=concat_dim)
        outs = [torch.empty_like(pieces[0]) for _ in range(self.size)]
        dist.all_to_all(outs, pieces, group=self.group.device_group)
        return torch.cat(outs, dim=concat_dim)

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.size > 1:
            dist.broadcast(x, self.group.ranks[src], group=self.group.device_group)
        return x

    def cpu_all_reduce_max(self, values: list) -> list:
        """Host-side MAX agreement (DP lockstep); stays on gloo."""
        if self.size == 1 or self.group.cpu_group is None:
            return list(values)
        t = torch.tensor(values, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group.cpu_group)
        return t.tolist()

    # ---- collectives that return before they finish (pipelined MoE plane) --------
    def all_gather_start(self, x: torch.Tensor):
        """Rows of every rank, concatenated on dim 0: (output tensor, handle); the output is valid after
        ``handle.wait()``."""
        out = torch.empty((self.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        work = dist.all_gather_into_tensor(out, x.contiguous(), group=self.group.device_group, async_op=True)
        return out, work

    def reduce_scatter_start(self, x: torch.Tensor):
        """Sum over the ranks, this rank's slice of dim 0: (getter, handle); ``getter()`` after
        ``handle.wait()`` gives the slice."""
        x = x.contiguous()
        assert x.shape[0] % self.size == 0
        n = x.shape[0] // self.size
        if not x.is_cuda:
            work = dist.all_reduce(x, group=self.group.device_group, async_op=True)     # gloo has no reduce-scatter
            return (lambda: x[self.rank * n:(self.rank + 1) * n]), work
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        work = dist.reduce_scatter_tensor(out, x, group=self.group.device_group, async_op=True)
        return (lambda: out), work

    # ---- MoE data plane ---------------------------------------------------------
    def dispatch(self, hidden, topk_w, topk_ids):
        if self.size == 1:
            return hidden, topk_w, topk_ids
        return (self.all_gather(hidden, 0), self.all_gather(topk_w, 0), self.all_gather(topk_ids, 0))

    def combine(self, expert_out):
        return self.reduce_scatter(expert_out, 0)


_tp_comm: Optional[DeviceCommunicator] = None
_ep_comm: Optional[DeviceCommunicator] = None
_dcp_comm: Optional[DeviceCommunicator] = None


def get_tp_comm() -> DeviceCommunicator:
    global _tp_comm
    st = get_state()
    if _tp_comm is None or _tp_comm.group is not st.tp:
        _tp_comm = DeviceCommunicator(st.tp, _heap_for(st.tp))
    return _tp_comm


def get_ep_comm() -> DeviceCommunicator:
    global _ep_comm
    st = get_state()
    if _ep_comm is None or _ep_comm.group is not st.ep:
        _ep_comm = DeviceCommunicator(st.ep, _heap_for(st.ep))
    return _ep_comm


_pcp_comm: Optional[DeviceCommunicator] = None


def get_pcp_comm() -> DeviceCommunicator:
    global _pcp_comm
    st = get_state()
    if _pcp_comm is None or _pcp_comm.group is not st.pcp:
        _pcp_comm = DeviceCommunicator(st.pcp, None)
    return _pcp_comm


def get_dcp_comm() -> DeviceCommunicator:
    global _dcp_comm
    st = get_state()
    if _dcp_comm is None or _dcp_comm.group is not st.dcp:
        _dcp_comm = DeviceCommunicator(st.dcp, None)
    return _dcp_comm


_heaps: dict = {}
_heap_min_bytes = 0


def ensure_tp_heap(max_tokens: int, max_n: int):
    """Create the TP group's symmetric heap sized for the fused row-parallel GEMMs (GPU, tp > 1)."""
    global _heap_min_bytes
    st = get_state()
    if st.tp.size == 1 or not torch.cuda.is_available() or envs.B200_TP_COMM == "nccl":
        return None
    from ..ops import cuda
    _heap_min_bytes = cuda.FusedTP.heap_bytes(max_tokens, max_n, st.tp.size) + 64 * 2**20
    comm = get_tp_comm()
    if comm.heap is not None and envs.B200_FUSED_TP:
        comm.heap.configure_fused_tp(max_tokens, max_n)
    return comm.heap


def ensure_ep_heap(max_tokens: int, top_k: int, hidden: int, inter: int, num_experts: int):
    """Create the EP group's symmetric heap with the regions of the fused dispatch/combine plane."""
    global _heap_min_bytes
    st = get_state()
    if (st.ep.size == 1 or not torch.cuda.is_available() or envs.B200_TP_COMM == "nccl"
            or not envs.B200_MOE_FUSED_EP):
        return None
    from ..ops import cuda_moe
    factor = envs.B200_MOE_EP_CAPACITY_FACTOR
    need = cuda_moe.EpState.heap_bytes(max_tokens, top_k, hidden, num_experts, st.ep.size, factor) + 16 * 2**20
    _heap_min_bytes = max(_heap_min_bytes, need)
    comm = get_ep_comm()
    if comm.heap is not None and getattr(comm.heap, "ep_state", None) is None:
        comm.heap.ep_state = cuda_moe.EpState(comm.heap, max_tokens, top_k, hidden, inter, num_experts, factor)
    return comm.heap


def _heap_for(group: Group):
    """Symmetric heap of a group, created on first use on GPUs when fused collectives are on."""
    if group.size == 1 or not torch.cuda.is_available() or envs.B200_TP_COMM == "nccl":
        return None
    key = (group.name, tuple(group.ranks))
    if key not in _heaps:
        from .symm_heap import SymmetricHeap
        _heaps[key] = SymmetricHeap.create(group, max(envs.B200_SYMM_HEAP_MB * 2**20, _heap_min_bytes))
    return _heaps[key]


def reset() -> None:
    global _tp_comm, _ep_comm, _dcp_comm
    _tp_comm = _ep_comm = _dcp_comm = None
    _heaps.clear()
