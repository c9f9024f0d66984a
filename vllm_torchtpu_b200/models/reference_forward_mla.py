"""Dense, cache-free forward of the MLA + MoE family in the NON-absorbed form
(per-head keys and values are materialised from the latent), used to check the
absorbed paged implementation."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import reference as ref
from .reference_forward import _rms


@torch.no_grad()
def dense_mla_logits(model, token_ids: list) -> torch.Tensor:
    cfg = model.cfg
    ids = torch.tensor(token_ids, dtype=torch.long, device=model.embed.device)
    S = ids.numel()
    pos = torch.arange(S, device=ids.device)
    x = model.embed[ids].float()
    for layer in model.layers:
        a = layer.self_attn
        h = _rms(x, layer.input_ln, cfg.rms_norm_eps)
        if a.q_a is not None:
            qc = _rms(h @ a.q_a.weight.float().t(), a.q_a_ln, cfg.rms_norm_eps)
            q = qc @ a.q_b.weight.float().t()
        else:
            q = h @ a.q_b.weight.float().t()
        q = q.view(S, a.H, a.nope + a.rope)
        kv = h @ a.kv_a.weight.float().t()
        kv_c = _rms(kv[:, :a.kv_lora], a.kv_a_ln, cfg.rms_norm_eps)
        k_pe = ref.apply_rope(kv[:, a.kv_lora:].reshape(S, 1, a.rope), pos, a.inv_freq, cfg.rope_interleaved)
        q_pe = ref.apply_rope(q[..., a.nope:], pos, a.inv_freq, cfg.rope_interleaved)
        k_nope = torch.einsum("sl,hnl->shn", kv_c, a.w_uk.float())
        v = torch.einsum("sl,hlv->shv", kv_c, a.w_uv.float())
        qf = torch.cat([q[..., :a.nope], q_pe], -1)
        kf = torch.cat([k_nope, k_pe.expand(S, a.H, a.rope)], -1)
        s = torch.einsum("qhd,khd->hqk", qf, kf) * a.scale
        mask = torch.ones(S, S, dtype=torch.bool, device=ids.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
        o = torch.einsum("hqk,khv->qhv", torch.softmax(s, -1), v).reshape(S, a.H * a.vdim)
        x = x + o @ a.o.weight.float().t()
        h = _rms(x, layer.post_ln, cfg.rms_norm_eps)
        if hasattr(layer.mlp, "gate_up"):
            gu = h @ layer.mlp.gate_up.weight.float().t()
            I = gu.shape[-1] // 2
            x = x + (F.silu(gu[:, :I]) * gu[:, I:]) @ layer.mlp.down.weight.float().t()
        else:
            x = x + layer.mlp.forward(h.to(cfg.dtype)).float()
    x = _rms(x, model.norm, cfg.rms_norm_eps)
    return x @ model.lm_head.float().t()
