"""Mixture-of-experts layer: router, expert ownership, dispatch / experts / combine.

Routing follows the reference (scoring → optional bias / grouped top-k → top-k →
renormalise → scale, reference: src/vllm_torchtpu/layers/adapter/moe_routing.py:161-343).
Expert ownership under expert parallelism is linear by ``experts_start``
(reference: src/vllm_torchtpu/layers/core/fused_moe_gmm.py:749-753) or a static
permutation (``expert_placement``).  Three data planes, as in the reference
(reference: src/vllm_torchtpu/layers/adapter/custom_ops/moe_runner.py:41-169):

* no EP: every rank holds all experts with the intermediate dim sharded over TP;
* EP, all-gather/reduce-scatter plane: ``DeviceCommunicator.dispatch`` gathers
  tokens, every rank runs its experts on all tokens, ``combine`` reduce-scatters;
* EP, fused plane: the dispatch/combine all-to-all runs inside the expert kernel
  over NVLink peer memory (``ops.cuda.moe_experts_ep``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import envs, ops
from ..parallel.communicator import get_ep_comm, get_tp_comm
from ..parallel.state import get_state
from ..quantization import get_moe_method
from .linear import ReplicatedLinear


_step_num_valid = None       # device int32[1]: rows of the current step that are real tokens (None: all)


def set_step_valid_tokens(t) -> None:
    """The runner names, per step, the device word that holds the number of real token rows; rows behind it
    (bucket padding, lockstep padding) are masked out of the routing."""
    global _step_num_valid
    _step_num_valid = t


def expert_placement(num_experts: int, ep_size: int, policy: str = "linear",
                     static_perm: Optional[list] = None) -> list:
    """``owner[e]`` = (rank, local index) for every global expert id."""
    per = num_experts // ep_size
    if policy == "linear":
        return [(e // per, e % per) for e in range(num_experts)]
    if policy == "round_robin":
        return [(e % ep_size, e // ep_size) for e in range(num_experts)]
    if policy == "static":
        assert static_perm is not None and sorted(static_perm) == list(range(num_experts))
        pos = {e: i for i, e in enumerate(static_perm)}
        return [(pos[e] // per, pos[e] % per) for e in range(num_experts)]
    raise ValueError(policy)


PIPELINED_CALLS = 0          # calls of the pipelined all-gather plane (tests and diagnostics)

class FusedMoE:
    def __init__(self, name: str, cfg, device, quant_config=None):
        st = get_state()
        self.name = name
        self.cfg = cfg
        self.device = device
        self.dtype = cfg.dtype
        self.hidden_size = cfg.hidden_size
        self.num_experts = cfg.num_experts
        self.activation = getattr(cfg, "hidden_act", "silu")
        self.top_k = cfg.num_experts_per_tok
        self.use_ep = st.expert_parallel and st.ep.size > 1
        self.ep_size = st.ep.size if self.use_ep else 1
        self.ep_rank = st.ep.rank_in_group if self.use_ep else 0
        self.tp_size = 1 if self.use_ep else st.tp.size
        self.tp_rank = 0 if self.use_ep else st.tp.rank_in_group
        self.intermediate_size = cfg.moe_intermediate_size // self.tp_size
        self.num_local_experts = self.num_experts // self.ep_size
        lo = self.ep_rank * self.num_local_experts
        self.expert_range = (lo, lo + self.num_local_experts)
        self.has_bias = bool(getattr(cfg, "moe_bias", False))      # router and expert biases (GPT-OSS)
        self.gate = ReplicatedLinear(f"{name}.gate", cfg.hidden_size, cfg.num_experts, dtype=cfg.dtype,
                                     device=device, quant_config=None, bias=self.has_bias)
        self.b13 = self.b2 = None
        self.score_bias = None
        if cfg.moe_score_bias:
            self.score_bias = torch.zeros(cfg.num_experts, dtype=torch.float32, device=device)
        self.method = get_moe_method(quant_config, name)
        self.method.create_weights(self)

    def alloc_biases(self) -> None:
        from ..quantization.unquantized import padded_hidden
        E, I = self.num_local_experts, self.intermediate_size
        self.b13 = torch.zeros(E, 2 * I, dtype=self.dtype, device=self.device)
        self.b2 = torch.zeros(E, padded_hidden(self), dtype=self.dtype, device=self.device)

    def load_expert_bias(self, local_e: int, gate_b, up_b, down_b) -> None:
        """Unsharded bias vectors of one expert (gate [I_full], up [I_full], down [H]); under tensor parallelism
        the gate / up slices follow the weight rows and the down bias is split evenly (the ranks' partial
        outputs are summed)."""
        if self.b13 is None:
            self.alloc_biases()
        I, r = self.intermediate_size, self.tp_rank
        self.b13[local_e, :I] = gate_b[r * I:(r + 1) * I].to(self.b13.dtype)
        self.b13[local_e, I:] = up_b[r * I:(r + 1) * I].to(self.b13.dtype)
        self.b2[local_e, :self.hidden_size] = (down_b.float() / self.tp_size).to(self.b2.dtype)

    def init_dummy(self, std: float, seed: int) -> None:
        # router logits come from N(0,1) gate weights so that routing is well spread
        self.gate.init_dummy(1.0, seed)
        self.method.init_dummy(self, std, seed)
        if self.has_bias:
            from .linear import seeded_normal
            self.alloc_biases()
            I, H = self.intermediate_size, self.hidden_size
            lo = self.expert_range[0]
            for e in range(self.num_local_experts):
                self.b13[e] = seeded_normal(f"{self.name}.experts.{lo + e}.b13", (2 * I,), 0.05, self.dtype,
                                            self.device, seed)
                self.b2[e, :H] = seeded_normal(f"{self.name}.experts.{lo + e}.b2", (H,), 0.05, self.dtype,
                                               self.device, seed) / self.tp_size
            self.gate.bias = seeded_normal(f"{self.name}.gate.bias", (self.num_experts,), 0.1, self.dtype,
                                           self.device, seed)
        if self.score_bias is not None:
            from .linear import seeded_normal
            self.score_bias = seeded_normal(f"{self.name}.bias", (self.num_experts,), 0.01, torch.float32,
                                            self.device, seed)

    def weight_bytes(self) -> int:
        return self.method.weight_bytes(self) + self.gate.weight_bytes()

    def route(self, x: torch.Tensor):
        logits = self.gate(x)
        c = self.cfg
        ids, w = ops.moe_route(logits, self.top_k, scoring=c.moe_scoring, renormalize=c.moe_renormalize,
                               routed_scaling=c.moe_routed_scaling, score_bias=self.score_bias,
                               n_group=c.moe_n_group, topk_group=c.moe_topk_group)
        sim = envs.B200_MOE_ROUTING_SIM
        nv = _step_num_valid
        if nv is not None and nv.device != ids.device:
            nv = None
        if sim or nv is not None:
            # padded rows take no expert; a routing simulation (benchmarks with random-init routers) replaces
            # the router's choice by a balanced or hashed one
            post = ops.cuda_ops().moe_route_post if ids.is_cuda else ops.ref.moe_route_post
            ids, w = post(ids, w, self.num_experts, nv, sim)
        return ids, w

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        topk_ids, topk_w = self.route(x)
        if not self.use_ep:
            y = self.method.apply(self, x, topk_ids, topk_w)
            if self.tp_size > 1:
                y = get_tp_comm().all_reduce(y)
            return y
        comm = get_ep_comm()
        if (x.is_cuda and envs.B200_MOE_FUSED_EP and comm.heap is not None and self.activation == "silu"
                and getattr(comm.heap, "ep_state", None) is not None
                and x.shape[0] >= envs.B200_MOE_FUSED_EP_MIN_TOKENS and hasattr(self.method, "apply_fused_ep")):
            return self._forward_fused_ep(x, topk_ids, topk_w, comm)
        chunks = envs.B200_MOE_PIPELINE_CHUNKS
        if chunks > 1 and x.shape[0] >= chunks * envs.B200_MOE_PIPELINE_MIN_CHUNK_TOKENS and comm.size > 1 and \
                not (x.is_cuda and torch.cuda.is_current_stream_capturing()):
            return self._forward_pipelined(x, topk_ids, topk_w, comm, chunks)
        # all-gather / reduce-scatter plane: rows must be equal on every rank (DP lockstep pads them)
        hx, hw, hi = comm.dispatch(x, topk_w, topk_ids)
        y = self.method.apply(self, hx, hi, hw)
        return comm.combine(y)

    def _forward_pipelined(self, x, topk_ids, topk_w, comm, chunks: int):
        """All-gather -> grouped expert GEMMs -> reduce-scatter over token chunks, with the collectives of the
        neighbouring chunks in flight while a chunk's experts run: the gather of chunk i + 1 is started before
        the experts of chunk i, the reduce-scatter of chunk i runs under the experts of chunk i + 1.  The
        collectives are issued in the same order on every rank (the chunk bounds follow from the common row
        count) and run on the process group's own stream; ``wait`` orders them against this stream.
        (reference: src/vllm_torchtpu/layers/adapter/pipelined_fused_moe.py:14-60 - chunked all-gather and
        reduce-scatter overlapped with the grouped matmuls)"""
        global PIPELINED_CALLS
        PIPELINED_CALLS += 1
        T = x.shape[0]
        step = -(-T // chunks)
        bounds = [(lo, min(T, lo + step)) for lo in range(0, T, step)]

        def start(i):
            lo, hi = bounds[i]
            return [comm.all_gather_start(t[lo:hi]) for t in (x, topk_w, topk_ids)]
        pending = start(0)
        tails = []
        for i in range(len(bounds)):
            nxt = start(i + 1) if i + 1 < len(bounds) else None
            for _, work in pending:
                work.wait()
            hx, hw, hi_ = (t for t, _ in pending)
            y = self.method.apply(self, hx, hi_, hw)
            tails.append(comm.reduce_scatter_start(y))
            pending = nxt
        outs = []
        for get, work in tails:
            work.wait()
            outs.append(get())
        return torch.cat(outs, 0)

    def _forward_fused_ep(self, x, topk_ids, topk_w, comm):
        """Fused dispatch/combine plane.  The ranks of a TP group hold identical tokens, so each
        dispatches one contiguous slice of them and the slices are all-gathered afterwards (the
        sequence-parallel MoE dataflow of the reference, models/vllm/qwen3_5_patch.py:95-141)."""
        st = get_state()
        tp = st.tp.size
        if tp == 1:
            return self._fused_ep_calls(x, topk_ids, topk_w, comm)
        T = x.shape[0]
        chunk = -(-T // tp)
        lo = min(T, st.tp.rank_in_group * chunk)
        hi = min(T, lo + chunk)
        y = self._fused_ep_calls(x[lo:hi], topk_ids[lo:hi], topk_w[lo:hi], comm, rows=chunk)
        if hi - lo < chunk:
            y = torch.cat([y, y.new_zeros(chunk - (hi - lo), y.shape[1])], 0)
        return get_tp_comm().all_gather(y, 0)[:T]

    def _fused_ep_calls(self, x, topk_ids, topk_w, comm, rows=None):
        """One call of the plane per ``max_tokens`` rows.  Every rank of the EP group makes the same number
        of calls: ``rows`` is the row count the ranks agree on (a TP slice may be shorter on the last
        rank; replicas in lockstep pad their steps to one length)."""
        step = comm.heap.ep_state.max_tokens
        T = x.shape[0]
        n_calls = max(1, -(-(rows if rows is not None else T) // step))
        if n_calls == 1:
            return self.method.apply_fused_ep(self, x, topk_ids, topk_w, comm)
        outs = []
        for i in range(n_calls):
            lo, hi = min(T, i * step), min(T, (i + 1) * step)
            outs.append(self.method.apply_fused_ep(self, x[lo:hi], topk_ids[lo:hi], topk_w[lo:hi], comm))
        return torch.cat(outs, 0)
