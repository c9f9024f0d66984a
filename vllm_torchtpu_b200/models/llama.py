"""Dense decoder family: Llama 3.x, Mistral, Qwen2 (qkv bias), Qwen3 (q/k norm).

Per layer: fused add+RMSNorm → packed qkv GEMM → RoPE + KV write + ragged paged
attention → o_proj (row parallel, reduced across TP inside the GEMM kernel) →
fused add+RMSNorm → gate_up GEMM → SiLU·mul → down_proj (row parallel).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..layers.attention import PagedAttention
from ..layers.linear import ColumnParallelLinear, RowParallelLinear, seeded_normal
from ..parallel.communicator import get_tp_comm
from ..parallel.state import get_state
from ..quantization import QuantConfig


def pad_q_heads(t: torch.Tensor, dim: int, num_kv_heads: int, g: int, g_padded: int, head_dim: int):
    """Zero-pad the query heads of every KV group from ``g`` to ``g_padded`` along ``dim`` of a weight
    whose extent there is ``num_kv_heads * g * head_dim``; the head -> KV-head mapping is unchanged
    (reference: src/vllm_torchtpu/gqa_head_padding.py — zero-pad Q heads when heads % tp != 0)."""
    t = t.movedim(dim, 0)
    rest = t.shape[1:]
    t = t.reshape(num_kv_heads, g, head_dim, -1)
    out = t.new_zeros((num_kv_heads, g_padded, head_dim, t.shape[-1]))
    out[:, :g] = t
    return out.reshape((num_kv_heads * g_padded * head_dim,) + tuple(rest)).movedim(0, dim)


class QKVParallelLinear(ColumnParallelLinear):
    """q/k/v packed; KV heads are replicated when there are fewer than TP ranks.  ``unpadded_q`` > 0:
    checkpoints hold that many query heads and ``num_q_heads`` is the zero-padded count."""

    def __init__(self, name, hidden, num_q_heads, num_kv_heads, head_dim, unpadded_q: int = 0, **kw):
        st = get_state()
        tp, r = st.tp.size, st.tp.rank_in_group
        self.total_q, self.total_kv, self.hd = num_q_heads, num_kv_heads, head_dim
        self.unpadded_q = unpadded_q if unpadded_q and unpadded_q != num_q_heads else 0
        self.q_per_rank = num_q_heads // tp
        self.kv_per_rank = max(1, num_kv_heads // tp)
        self.kv_replicas = max(1, tp // num_kv_heads)
        super().__init__(name, hidden, [num_q_heads * head_dim, num_kv_heads * head_dim,
                                        num_kv_heads * head_dim], **kw)
        self.shard_sizes = [self.q_per_rank * head_dim, self.kv_per_rank * head_dim,
                            self.kv_per_rank * head_dim]
        if self.out_features != sum(self.shard_sizes):
            self.out_features = sum(self.shard_sizes)
        self._r = r
        if self.unpadded_q:
            # random-init and checkpoint weights both come with the checkpoint's head count
            self.full_out = (self.unpadded_q + 2 * num_kv_heads) * head_dim

    def shard_of(self, full_weight):
        hd = self.hd
        if self.unpadded_q and full_weight.shape[0] == (self.unpadded_q + 2 * self.total_kv) * hd:
            q = pad_q_heads(full_weight[: self.unpadded_q * hd], 0, self.total_kv,
                            self.unpadded_q // self.total_kv, self.total_q // self.total_kv, hd)
            full_weight = torch.cat([q, full_weight[self.unpadded_q * hd:]], 0)
        q = full_weight[: self.total_q * hd]
        k = full_weight[self.total_q * hd:(self.total_q + self.total_kv) * hd]
        v = full_weight[(self.total_q + self.total_kv) * hd:]
        r = self._r
        kv_idx = r // self.kv_replicas
        qs = q[r * self.q_per_rank * hd:(r + 1) * self.q_per_rank * hd]
        ks = k[kv_idx * self.kv_per_rank * hd:(kv_idx + 1) * self.kv_per_rank * hd]
        vs = v[kv_idx * self.kv_per_rank * hd:(kv_idx + 1) * self.kv_per_rank * hd]
        return torch.cat([qs, ks, vs], 0)


class OProjParallelLinear(RowParallelLinear):
    """Row-parallel output projection whose input features are query heads; pads the checkpoint's
    columns when the query heads were zero-padded for tensor parallelism."""

    def __init__(self, name, num_q_heads, num_kv_heads, head_dim, hidden, unpadded_q: int = 0, **kw):
        super().__init__(name, num_q_heads * head_dim, hidden, **kw)
        self.q_pad = None
        if unpadded_q and unpadded_q != num_q_heads:
            self.q_pad = (num_kv_heads, unpadded_q // num_kv_heads, num_q_heads // num_kv_heads, head_dim)
            self.full_in = unpadded_q * head_dim

    def shard_of(self, full_weight):
        if self.q_pad is not None and full_weight.shape[1] == self.q_pad[0] * self.q_pad[1] * self.q_pad[3]:
            full_weight = pad_q_heads(full_weight, 1, *self.q_pad)
        return super().shard_of(full_weight)


class LlamaMLP:
    def __init__(self, name, cfg: ModelConfig, intermediate_size: int, device, quant, reduce_results=True):
        kw = dict(dtype=cfg.dtype, device=device, quant_config=quant)
        self.gate_up = ColumnParallelLinear(f"{name}.gate_up_proj", cfg.hidden_size,
                                            [intermediate_size, intermediate_size], **kw)
        self.down = RowParallelLinear(f"{name}.down_proj", intermediate_size, cfg.hidden_size,
                                      reduce_results=reduce_results, **kw)
        self.act = getattr(cfg, "hidden_act", "silu")

    def linears(self):
        return [self.gate_up, self.down]

    def init_dummy(self, std, seed):
        for lin in self.linears():
            lin.init_dummy(std, seed)

    def weight_bytes(self):
        return sum(lin.weight_bytes() for lin in self.linears())

    def forward(self, x):
        gu = self.gate_up
        if self.act != "silu":
            # other gated activations (GELU-tanh, clamped and OAI-style SwiGLU, SiTU): GEMM, activation kernel, GEMM
            h = self.gate_up(x)
            return self.down(ops.gated_act_and_mul(h.reshape(-1, h.shape[-1]), self.act).reshape(
                *x.shape[:-1], h.shape[-1] // 2))
        if (x.is_cuda and gu.bias is None and getattr(gu.method, "supports_fused_reduce", False)
                and not gu.lora_targets):
            # gate and up tiles share the activation tile; SiLU*mul happens in the GEMM epilogue
            return self.down(ops.cuda_ops().gemm_swiglu(x, gu.weight))
        if (x.is_cuda and x.dtype == torch.bfloat16 and hasattr(self.down.method, "apply_quantised")
                and not self.down.lora_targets and type(self.down.method) is type(gu.method)):
            # block-scaled fp8: SiLU*mul runs inside the quantisation kernel of the down projection's input
            h = self.gate_up(x)
            h2 = h.reshape(-1, h.shape[-1])
            xq, xs = ops.cuda_ops().quant_rows_1x128(h2, h2.shape[1] // 2, swiglu=True)
            y = self.down.forward_quantised(xq, xs)
            return y if not isinstance(y, torch.Tensor) else y.reshape(*x.shape[:-1], y.shape[-1])
        return self.down(ops.silu_and_mul(self.gate_up(x)))


class LlamaAttention:
    def __init__(self, name, cfg: ModelConfig, device, quant):
        kw = dict(dtype=cfg.dtype, device=device, quant_config=quant)
        self.qkv = QKVParallelLinear(f"{name}.qkv_proj", cfg.hidden_size, cfg.num_q_heads,
                                     cfg.num_kv_heads, cfg.head_dim, unpadded_q=cfg.num_q_heads_unpadded,
                                     bias=cfg.attention_bias, **kw)
        self.o = OProjParallelLinear(f"{name}.o_proj", cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim,
                                     cfg.hidden_size, unpadded_q=cfg.num_q_heads_unpadded,
                                     bias=getattr(cfg, "attention_out_bias", False), **kw)
        self.q_norm_w = self.k_norm_w = None
        if cfg.qk_norm:
            self.q_norm_w = torch.ones(cfg.head_dim, dtype=cfg.dtype, device=device)
            self.k_norm_w = torch.ones(cfg.head_dim, dtype=cfg.dtype, device=device)
        inv_freq = ops.ref.rope_inv_freq(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling).to(device)
        af = ops.ref.rope_attention_factor(cfg.rope_scaling)      # YaRN: cos / sin carry it on q and k
        self.attn = PagedAttention(self.qkv.q_per_rank, self.qkv.kv_per_rank, cfg.head_dim, inv_freq,
                                   scale=cfg.head_dim ** -0.5 * af * af, rope_interleaved=cfg.rope_interleaved, q_norm_w=self.q_norm_w,
                                   k_norm_w=self.k_norm_w, eps=cfg.rms_norm_eps,
                                   sliding_window=cfg.sliding_window, softcap=cfg.logit_softcap)

    def linears(self):
        return [self.qkv, self.o]

    def forward(self, x, kv_cache, meta):
        qkv = self.qkv(x)
        o = self.attn.forward(qkv, kv_cache, meta)
        return self.o(o)


class LlamaDecoderLayer:
    def __init__(self, idx: int, cfg: ModelConfig, device, quant):
        name = f"model.layers.{idx}"
        self.idx = idx
        self.eps = cfg.rms_norm_eps
        self.input_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.post_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.self_attn = LlamaAttention(f"{name}.self_attn", cfg, device, quant)
        self.mlp = self._make_ffn(name, cfg, device, quant)
        # both row-parallel outputs of this layer feed an add + RMSNorm directly
        self.self_attn.o.defer_reduce = True
        if isinstance(self.mlp, LlamaMLP):
            self.mlp.down.defer_reduce = True

    def _make_ffn(self, name, cfg, device, quant):
        return LlamaMLP(f"{name}.mlp", cfg, cfg.intermediate_size, device, quant)

    def forward(self, hidden, residual, kv_cache, meta):
        if residual is None:
            residual = hidden
            h = ops.rms_norm(hidden, self.input_ln, self.eps)
        else:
            h, residual = ops.fused_add_rms_norm(hidden, residual, self.input_ln, self.eps)
        h = self.self_attn.forward(h, kv_cache, meta)
        h, residual = ops.fused_add_rms_norm(h, residual, self.post_ln, self.eps)
        h = self.mlp.forward(h)
        return h, residual


class LlamaForCausalLM:
    layer_cls = LlamaDecoderLayer

    def __init__(self, cfg: ModelConfig, device="cpu", layer_range: Optional[tuple] = None):
        self.cfg = cfg
        self.device = device
        st = get_state()
        self.pp_first = st.pp.is_first
        self.pp_last = st.pp.is_last
        quant = QuantConfig(cfg.quantization, cfg.weight_block_size,
                            ignored_layers=("lm_head", "embed", "gate.") + tuple(getattr(cfg, "quant_ignored", ()))) \
            if cfg.quantization else None
        lo, hi = layer_range if layer_range else (0, cfg.num_layers)
        self.layer_range = (lo, hi)
        self.layers = [self.layer_cls(i, cfg, device, quant) for i in range(lo, hi)]
        self.embed = None
        self.norm = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.lm_head = None
        self.vocab_shard = cfg.vocab_size // st.tp.size if cfg.vocab_size % st.tp.size == 0 else None
        self.decode_mega = None          # persistent decode kernel (ops/cuda_mega.py), set up with the KV cache
        self.decode_mega_reason = "not set up"
        self.aux_layers: tuple = ()      # layers whose input (hidden + residual) an Eagle-3 drafter reads
        self.aux_hidden: list = []

    # ---- weights -------------------------------------------------------------
    def named_linears(self):
        for l in self.layers:
            for lin in l.self_attn.linears():
                yield lin
            for lin in l.mlp.linears():
                yield lin

    def init_dummy(self) -> None:
        cfg, st = self.cfg, get_state()
        std, seed = cfg.init_std, cfg.seed
        if self.pp_first or cfg.tie_word_embeddings:
            self.embed = seeded_normal("model.embed_tokens", (cfg.vocab_size, cfg.hidden_size), std,
                                       cfg.dtype, self.device, seed)
        if self.pp_last:
            full = self.embed if cfg.tie_word_embeddings else seeded_normal(
                "lm_head", (cfg.vocab_size, cfg.hidden_size), std, cfg.dtype, self.device, seed)
            self.lm_head = self._shard_vocab(full)
        for l in self.layers:
            for lin in l.self_attn.linears():
                lin.init_dummy(std, seed)
            l.mlp.init_dummy(std, seed)

    def _shard_vocab(self, full):
        st = get_state()
        if st.tp.size == 1 or self.vocab_shard is None:
            return full
        r = st.tp.rank_in_group
        return full[r * self.vocab_shard:(r + 1) * self.vocab_shard].contiguous()

    def weight_bytes(self) -> int:
        n = 0
        for t in (self.embed, self.lm_head):
            if t is not None:
                n += t.numel() * t.element_size()
        if self.cfg.tie_word_embeddings and self.embed is not None and self.lm_head is self.embed:
            n -= self.embed.numel() * self.embed.element_size()
        for l in self.layers:
            for lin in l.self_attn.linears():
                n += lin.weight_bytes()
            n += l.mlp.weight_bytes()
        return n

    # ---- forward -------------------------------------------------------------
    def setup_decode_fusion(self, kv_caches) -> None:
        """(Re)build the persistent decode kernel's descriptors for these KV caches; models or layouts
        it does not cover keep the per-layer kernels (the reason is kept for the log)."""
        self.decode_mega = None
        if not kv_caches or not torch.is_tensor(kv_caches[0]) or not kv_caches[0].is_cuda:
            self.decode_mega_reason = "not on a GPU"
            return
        from ..ops.cuda_mega import DecodeMega
        heap = get_tp_comm().heap if get_state().tp.size > 1 else None
        why = DecodeMega.why_not(self, kv_caches, heap)
        self.decode_mega_reason = why or ""
        if why is None:
            self.decode_mega = DecodeMega.build(self, kv_caches, kv_caches[0].device, heap)

    def _use_decode_mega(self, meta, hidden, residual) -> bool:
        m = self.decode_mega
        if m is None or hidden is None or residual is not None or self.aux_layers:
            return False
        T = hidden.shape[0]
        if T > m.maxt or meta.num_decode_reqs != meta.num_reqs or meta.max_query_len > 1:
            return False
        if meta.dcp_size > 1 or (meta.padded_num_reqs or meta.num_reqs) != T:
            return False
        from ..lora import wiring
        return not wiring.active()

    def forward(self, input_ids, meta, kv_caches, *, hidden=None, residual=None):
        """Returns (hidden, residual) of the last local layer; the caller applies
        ``finalize`` on the last pipeline stage."""
        if hidden is None:
            hidden = ops.embedding(input_ids, self.embed)
        if self._use_decode_mega(meta, hidden, residual):
            # decode-only step: every layer in one persistent kernel; (0, residual stream) comes back
            return self.decode_mega.run(hidden.contiguous(), meta, hidden.shape[0])
        self.aux_hidden = []
        for i, layer in enumerate(self.layers):
            if i in self.aux_layers:
                hidden = ops.materialize(hidden)
                self.aux_hidden += [hidden if residual is None else hidden + residual] * self.aux_layers.count(i)
            hidden, residual = layer.forward(hidden, residual, kv_caches[i], meta)
        return ops.materialize(hidden), residual

    def finalize(self, hidden, residual):
        if residual is None:
            return ops.rms_norm(hidden, self.norm, self.cfg.rms_norm_eps)
        h, _ = ops.fused_add_rms_norm(hidden, residual, self.norm, self.cfg.rms_norm_eps)
        return h

    def enable_dp_vocab(self, dp_vocab) -> None:
        """Keep only this data-parallel replica's rows of the embedding table and the lm_head
        (``parallel/dp_vocab.py``); idempotent, called again after the weights are replaced."""
        tied = self.lm_head is self.embed
        if self.embed is not None:
            self.embed = dp_vocab.shard_rows(self.embed)
        if self.lm_head is not None:
            self.lm_head = self.embed if tied else dp_vocab.shard_rows(self.lm_head)
        self.dp_vocab = dp_vocab

    def compute_logits(self, hidden_rows):
        """hidden_rows [R, H] → logits [R, V] (all-gathered over the vocab shards)."""
        if getattr(self, "dp_vocab", None) is not None:
            return self.dp_vocab.logits(hidden_rows, self.lm_head)
        logits = ops.gemm(hidden_rows, self.lm_head)
        comm = get_tp_comm()
        if comm.size > 1 and self.vocab_shard is not None:
            logits = comm.all_gather(logits, dim=-1)
        return logits

    def local_logits(self, hidden_rows):
        return ops.gemm(hidden_rows, self.lm_head)

    # ---- KV geometry -----------------------------------------------------------
    def kv_cache_shape(self, num_blocks: int, block_size: int) -> tuple:
        a = self.layers[0].self_attn.attn
        return (num_blocks, 2, a.num_kv_heads, block_size, a.head_dim)

    def kv_bytes_per_block(self, block_size: int, kv_dtype: torch.dtype) -> int:
        a = self.layers[0].self_attn.attn
        return len(self.layers) * 2 * a.num_kv_heads * block_size * a.head_dim * \
            torch.empty((), dtype=kv_dtype).element_size()
