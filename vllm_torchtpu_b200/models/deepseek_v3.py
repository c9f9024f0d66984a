"""DeepSeek-V2/V3/R1 family: multi-head latent attention (MLA) + MoE with shared
experts, sigmoid router with score-correction bias and grouped top-k.

MLA runs in the absorbed form for prefill and decode alike: the cache row of a
token is ``kv_c_normed (kv_lora) ‖ k_pe (rope)``; queries are projected into the
latent space (``ql_nope = q_nope · W_UK``), attention is multi-query over the
latent rows, and the result is expanded with ``W_UV`` before ``o_proj``
(reference: src/vllm_torchtpu/layers/adapter/attention.py:2659-2879).  The first
``first_dense_layers`` layers have a dense FFN, the rest routed experts plus one
shared expert.  Heads are sharded over TP; the latent cache is per rank.

With ``index_topk > 0`` (DeepSeek-V3.2 style sparse attention) a lightweight
indexer scores the context per query and attention reads only the top-k rows
(reference: src/vllm_torchtpu/layers/adapter/custom_ops/mla_attention_op.py:383-1529).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..config import ModelConfig
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, seeded_normal
from ..parallel.state import get_state
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaMLP
from .qwen3_moe import MoEBlock


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class MLAAttention:
    def __init__(self, name: str, cfg: ModelConfig, device, quant):
        st = get_state()
        tp = st.tp.size
        self.cfg = cfg
        self.eps = cfg.rms_norm_eps
        self.H = cfg.num_q_heads // tp
        self.nope, self.rope, self.vdim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.kv_lora, self.q_lora = cfg.kv_lora_rank, cfg.q_lora_rank
        kw = dict(dtype=cfg.dtype, device=device, quant_config=quant)
        qk = self.nope + self.rope
        if self.q_lora:
            self.q_a = ReplicatedLinear(f"{name}.q_a_proj", cfg.hidden_size, self.q_lora, **kw)
            self.q_a_ln = torch.ones(self.q_lora, dtype=cfg.dtype, device=device)
            self.q_b = ColumnParallelLinear(f"{name}.q_b_proj", self.q_lora, cfg.num_q_heads * qk, **kw)
        else:
            self.q_a = None
            self.q_b = ColumnParallelLinear(f"{name}.q_proj", cfg.hidden_size, cfg.num_q_heads * qk, **kw)
        self.kv_a = ReplicatedLinear(f"{name}.kv_a_proj_with_mqa", cfg.hidden_size, self.kv_lora + self.rope, **kw)
        self.kv_a_ln = torch.ones(self.kv_lora, dtype=cfg.dtype, device=device)
        # kv_b is kept un-quantised and pre-split into the two absorbed matrices
        self.w_uk = None            # [H, nope, kv_lora]
        self.w_uv = None            # [H, kv_lora, vdim]
        self.o = RowParallelLinear(f"{name}.o_proj", cfg.num_q_heads * self.vdim, cfg.hidden_size, **kw)
        self.inv_freq = ops.ref.rope_inv_freq(self.rope, cfg.rope_theta, cfg.rope_scaling).to(device)
        if getattr(cfg, "mla_use_nope", False):
            self.inv_freq = torch.zeros_like(self.inv_freq)       # angle 0 everywhere: the rotation is the identity
        af = ops.ref.rope_attention_factor(cfg.rope_scaling)
        self.scale = qk ** -0.5 * af * af
        if cfg.rope_scaling and "factor" in cfg.rope_scaling:
            m = yarn_mscale(cfg.rope_scaling["factor"], cfg.rope_scaling.get("mscale_all_dim", 0.0))
            self.scale *= m * m
        self.name = name
        self.device = device
        self.index_topk = cfg.index_topk
        if self.index_topk:
            self.idx_heads, self.idx_dim = cfg.index_n_heads, cfg.index_head_dim
            self.idx_q = ReplicatedLinear(f"{name}.indexer.wq", cfg.hidden_size, self.idx_heads * self.idx_dim, **kw)
            self.idx_k = ReplicatedLinear(f"{name}.indexer.wk", cfg.hidden_size, self.idx_dim, **kw)
            self.idx_w = ReplicatedLinear(f"{name}.indexer.weights", cfg.hidden_size, self.idx_heads, **kw)

    def linears(self):
        ls = [self.q_b, self.kv_a, self.o]
        if self.q_a is not None:
            ls.append(self.q_a)
        if self.index_topk:
            ls += [self.idx_q, self.idx_k, self.idx_w]
        return ls

    def init_dummy(self, std, seed):
        for lin in self.linears():
            lin.init_dummy(std, seed)
        cfg, st = self.cfg, get_state()
        full = seeded_normal(f"{self.name}.kv_b_proj", (cfg.num_q_heads * (self.nope + self.vdim), self.kv_lora),
                             std, cfg.dtype, self.device, seed)
        self.load_kv_b(full)

    def load_kv_b(self, full: torch.Tensor):
        """kv_b_proj.weight [Hq*(nope+v), kv_lora] → absorbed W_UK / W_UV of this rank's heads."""
        st = get_state()
        Hq = self.cfg.num_q_heads
        w = full.view(Hq, self.nope + self.vdim, self.kv_lora)
        r = st.tp.rank_in_group
        w = w[r * self.H:(r + 1) * self.H]
        self.w_uk = w[:, :self.nope, :].contiguous()                         # [H, nope, L]
        self.w_uv = w[:, self.nope:, :].transpose(1, 2).contiguous()         # [H, L, v]
        # K-major copies for the grouped GEMM (heads as groups): [H, L, nope] and [H, v, L]
        self.w_uk_t = self.w_uk.transpose(1, 2).contiguous()
        self.w_uv_t = self.w_uv.transpose(1, 2).contiguous()

    def weight_bytes(self):
        n = sum(l.weight_bytes() for l in self.linears())
        for t in (self.w_uk, self.w_uv):
            n += t.numel() * t.element_size()
        return n

    def forward(self, x, cache, meta):
        T = x.shape[0]
        if self.q_a is not None:
            qc = ops.rms_norm(self.q_a(x), self.q_a_ln, self.eps)
            q = self.q_b(qc)
        else:
            q = self.q_b(x)
        q = q.view(T, self.H, self.nope + self.rope)
        kv = self.kv_a(x)
        kv_c = ops.rms_norm(kv[:, :self.kv_lora].contiguous(), self.kv_a_ln, self.eps)
        if (x.is_cuda and x.dtype == torch.bfloat16 and self.w_uk_t.dtype == torch.bfloat16 and T > 0
                and self.kv_lora % 128 == 0 and self.vdim % 128 == 0 and self.nope % 8 == 0 and self.rope % 8 == 0):
            # absorbed form on the package's kernels: W_UK / W_UV as grouped tcgen05 GEMMs over the heads
            cu = ops.cuda_ops()
            q_latent, k_pe = cu.mla_absorb(q.contiguous(), kv, meta.positions, self.inv_freq, self.w_uk_t,
                                           self.nope, self.rope, self.kv_lora, self.cfg.rope_interleaved)
            ops.mla_write_cache(cache, kv_c, k_pe, meta.slot_mapping)
            topk = self._index(x, cache, meta) if self.index_topk else None
            o_lat = ops.mla_paged_attention(q_latent, cache, meta, self.scale, self.kv_lora, topk_indices=topk)
            return self.o(cu.mla_unabsorb(o_lat, self.w_uv_t))
        k_pe = kv[:, self.kv_lora:].reshape(T, 1, self.rope)
        q_pe = ops.ref.apply_rope(q[..., self.nope:], meta.positions, self.inv_freq, self.cfg.rope_interleaved)
        k_pe = ops.ref.apply_rope(k_pe, meta.positions, self.inv_freq, self.cfg.rope_interleaved).reshape(T, self.rope)
        ops.mla_write_cache(cache, kv_c, k_pe, meta.slot_mapping)
        # absorb W_UK: [T,H,nope] x [H,nope,L] -> [T,H,L]
        ql = torch.einsum("thn,hnl->thl", q[..., :self.nope].float(), self.w_uk.float()).to(x.dtype)
        q_latent = torch.cat([ql, q_pe.to(x.dtype)], dim=-1).contiguous()
        topk = None
        if self.index_topk:
            topk = self._index(x, cache, meta)
        o_lat = ops.mla_paged_attention(q_latent, cache, meta, self.scale, self.kv_lora, topk_indices=topk)
        o = torch.einsum("thl,hlv->thv", o_lat.float(), self.w_uv.float()).to(x.dtype)
        return self.o(o.reshape(T, self.H * self.vdim))

    def _index(self, x, cache, meta):
        """Top-k context positions per query token.  The indexer keys reuse the latent cache rows:
        score(t, s) = Σ_h w[t,h] · relu(q_idx[t,h] · k_idx[s]); this engine derives k_idx from the first
        ``idx_dim`` dims of the cached latent row so that no second cache is needed."""
        T = x.shape[0]
        q = self.idx_q(x).view(T, self.idx_heads, self.idx_dim).float()
        w = self.idx_w(x).float()
        bs = cache.shape[1]
        K = self.index_topk
        out = torch.full((T, K), -1, dtype=torch.int32, device=x.device)
        qsl, sl = meta.query_start_loc.tolist(), meta.seq_lens.tolist()
        for r in range(meta.num_reqs):
            qs, qe = qsl[r], qsl[r + 1]
            if qe <= qs:
                continue
            kv_len = sl[r]
            nblk = -(-kv_len // bs)
            rows = cache[meta.block_tables[r, :nblk].long()].reshape(nblk * bs, -1)[:kv_len, :self.idx_dim].float()
            s = torch.einsum("qhd,kd->qhk", q[qs:qe], rows).relu()
            score = (s * w[qs:qe, :, None]).sum(1)
            qpos = torch.arange(kv_len - (qe - qs), kv_len, device=x.device)[:, None]
            score = score.masked_fill(torch.arange(kv_len, device=x.device)[None, :] > qpos, float("-inf"))
            k = min(K, kv_len)
            idx = score.topk(k, dim=-1).indices.to(torch.int32)
            vals = score.gather(1, idx.long())
            idx = torch.where(torch.isfinite(vals), idx, torch.full_like(idx, -1))
            out[qs:qe, :k] = idx
        return out


class DeepseekV3DecoderLayer(LlamaDecoderLayer):
    def __init__(self, idx: int, cfg: ModelConfig, device, quant):
        name = f"model.layers.{idx}"
        self.idx = idx
        self.eps = cfg.rms_norm_eps
        self.input_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.post_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.self_attn = MLAAttention(f"{name}.self_attn", cfg, device, quant)
        if cfg.layer_is_moe(idx):
            self.mlp = MoEBlock(f"{name}.mlp", cfg, device, quant)
        else:
            self.mlp = LlamaMLP(f"{name}.mlp", cfg, cfg.intermediate_size, device, quant)


class DeepseekV3ForCausalLM(LlamaForCausalLM):
    layer_cls = DeepseekV3DecoderLayer

    def init_dummy(self) -> None:
        cfg = self.cfg
        std, seed = cfg.init_std, cfg.seed
        if self.pp_first or cfg.tie_word_embeddings:
            self.embed = seeded_normal("model.embed_tokens", (cfg.vocab_size, cfg.hidden_size), std, cfg.dtype,
                                       self.device, seed)
        if self.pp_last:
            full = seeded_normal("lm_head", (cfg.vocab_size, cfg.hidden_size), std, cfg.dtype, self.device, seed)
            self.lm_head = self._shard_vocab(full)
        for l in self.layers:
            l.self_attn.init_dummy(std, seed)
            l.mlp.init_dummy(std, seed)

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in (self.embed, self.lm_head) if t is not None)
        for l in self.layers:
            n += l.self_attn.weight_bytes() + l.mlp.weight_bytes()
        return n

    def kv_cache_shape(self, num_blocks: int, block_size: int) -> tuple:
        return (num_blocks, block_size, self.cfg.kv_lora_rank + self.cfg.qk_rope_head_dim)

    def kv_bytes_per_block(self, block_size: int, kv_dtype: torch.dtype) -> int:
        return len(self.layers) * block_size * (self.cfg.kv_lora_rank + self.cfg.qk_rope_head_dim) * \
            torch.empty((), dtype=kv_dtype).element_size()
