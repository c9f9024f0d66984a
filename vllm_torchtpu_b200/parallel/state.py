"""Process-group bookkeeping for the TP / PP / DP / EP / PCP / DCP layout.

World rank order is ``dp`` outermost, then ``pp``, then ``pcp``, then ``tp``
innermost, so the ranks of one TP group are consecutive GPUs.  NVSwitch makes
every peer equidistant, so none of the reference's topology-ordering logic
(reference: src/vllm_torchtpu/distributed/ep_mesh.py:155-195,
pcp_rank_order.py) is needed: groups are plain arithmetic on the rank.

Every group has a device communicator (NCCL, or gloo in CPU tests) and a CPU
(gloo) twin for host-side agreement such as the DP lockstep all-reduce
(reference: src/vllm_torchtpu/runner/tpu_runner.py:4132-4180).
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from ..logger import init_logger

logger = init_logger(__name__)


@dataclass
class Group:
    name: str
    ranks: list
    rank_in_group: int
    device_group: Optional[object] = None
    cpu_group: Optional[object] = None

    @property
    def size(self) -> int:
        return len(self.ranks)

    @property
    def is_first(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last(self) -> bool:
        return self.rank_in_group == self.size - 1

    @property
    def next_rank(self) -> int:
        return self.ranks[(self.rank_in_group + 1) % self.size]

    @property
    def prev_rank(self) -> int:
        return self.ranks[(self.rank_in_group - 1) % self.size]


def _single(name: str, rank: int = 0) -> Group:
    return Group(name, [rank], 0)


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    local_rank: int = 0
    tp: Group = field(default_factory=lambda: _single("tp"))
    pp: Group = field(default_factory=lambda: _single("pp"))
    dp: Group = field(default_factory=lambda: _single("dp"))
    ep: Group = field(default_factory=lambda: _single("ep"))
    pcp: Group = field(default_factory=lambda: _single("pcp"))
    dcp: Group = field(default_factory=lambda: _single("dcp"))
    world: Group = field(default_factory=lambda: _single("world"))
    expert_parallel: bool = False
    initialized_dist: bool = False


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def tp_size() -> int:
    return _STATE.tp.size


def tp_rank() -> int:
    return _STATE.tp.rank_in_group


def layout_ranks(world: int, tp: int, pp: int, dp: int, pcp: int = 1) -> dict:
    """All groups of every kind as lists of world ranks (pure function; unit-tested)."""
    assert world == tp * pp * dp * pcp, (world, tp, pp, dp, pcp)
    import numpy as np
    grid = np.arange(world).reshape(dp, pp, pcp, tp)
    groups = {
        "tp": [grid[d, p, c, :].tolist() for d in range(dp) for p in range(pp) for c in range(pcp)],
        "pcp": [grid[d, p, :, t].tolist() for d in range(dp) for p in range(pp) for t in range(tp)],
        "pp": [grid[d, :, c, t].tolist() for d in range(dp) for c in range(pcp) for t in range(tp)],
        "dp": [grid[:, p, c, t].tolist() for p in range(pp) for c in range(pcp) for t in range(tp)],
        # experts shard over dp x tp of one pipeline stage
        "ep": [grid[:, p, c, :].reshape(-1).tolist() for p in range(pp) for c in range(pcp)],
    }
    return groups


def dcp_groups(tp_group: list, dcp: int) -> list:
    """DCP groups are consecutive sub-ranges of a TP group (dcp divides tp)."""
    return [tp_group[i:i + dcp] for i in range(0, len(tp_group), dcp)]


def init_distributed(parallel_config, backend: Optional[str] = None,
                     timeout_s: float = 600.0) -> ParallelState:
    """Initialise torch.distributed (if world_size > 1) and build all groups."""
    global _STATE
    pc = parallel_config
    world = int(os.environ.get("WORLD_SIZE", pc.world_size))
    rank = int(os.environ.get("RANK", pc.rank))
    local_rank = int(os.environ.get("LOCAL_RANK", pc.local_rank))
    st = ParallelState(rank=rank, world_size=world, local_rank=local_rank)
    st.expert_parallel = pc.enable_expert_parallel
    if world == 1:
        _STATE = st
        return st
    backend = backend or pc.backend
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    st.initialized_dist = True
    lay = layout_ranks(world, pc.tensor_parallel_size, pc.pipeline_parallel_size,
                       pc.data_parallel_size, pc.prefill_context_parallel_size)

    def build(kind: str, all_groups: list) -> Group:
        mine = None
        for ranks in all_groups:
            dev = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
            cpu = dist.new_group(ranks, backend="gloo") if len(ranks) > 1 else None
            if rank in ranks:
                mine = Group(kind, ranks, ranks.index(rank), dev, cpu)
        assert mine is not None
        return mine

    st.tp = build("tp", lay["tp"])
    st.pp = build("pp", lay["pp"])
    st.dp = build("dp", lay["dp"])
    st.pcp = build("pcp", lay["pcp"])
    st.ep = build("ep", lay["ep"]) if pc.enable_expert_parallel else _single("ep", rank)
    if pc.decode_context_parallel_size > 1:
        alld = [g for tpg in lay["tp"] for g in dcp_groups(tpg, pc.decode_context_parallel_size)]
        st.dcp = build("dcp", alld)
    else:
        st.dcp = _single("dcp", rank)
    st.world = Group("world", list(range(world)), rank, dist.group.WORLD,
                     dist.new_group(list(range(world)), backend="gloo"))
    _STATE = st
    logger.info("rank %d/%d: tp=%s pp=%s dp=%s ep=%s", rank, world, st.tp.ranks, st.pp.ranks,
                st.dp.ranks, st.ep.ranks)
    return st


def set_state_for_test(**kw) -> ParallelState:
    global _STATE
    _STATE = ParallelState(**kw)
    return _STATE


def leave_process(code: int = 0) -> None:
    """End a multi-rank process without tearing the communicators down.

    Captured CUDA graphs hold NCCL kernels, and destroying a communicator under them can block; so
    ranks of a multi-GPU job skip the interpreter's teardown.  The registered at-exit handlers (coverage
    and library-load recorders among them) still run first, and the standard streams are flushed."""
    import atexit
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    try:
        atexit._run_exitfuncs()
    finally:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(code)


def destroy() -> None:
    global _STATE
    if dist.is_initialized():
        dist.destroy_process_group()
    _STATE = ParallelState()
