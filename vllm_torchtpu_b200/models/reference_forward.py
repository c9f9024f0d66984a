"""Dense, cache-free PyTorch forward of the decoder families, used as the
correctness oracle for the paged engine: it recomputes the whole sequence with
ordinary causal attention and knows nothing about pages, buckets or batching."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import reference as ref


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def dense_weight(lin) -> torch.Tensor:
    """fp32 weight of a linear layer whatever its storage (block-scaled fp8 is dequantised)."""
    scale = getattr(lin, "weight_scale_inv", None)
    if scale is not None:
        from ..quantization.fp8 import dequantize_weight_block
        return dequantize_weight_block(lin.weight, scale).float()
    return lin.weight.float()


@torch.no_grad()
def dense_llama_hidden(model, token_ids: list) -> torch.Tensor:
    """Final-norm hidden states [S, H] of one sequence (fp32 math)."""
    return dense_llama_logits(model, token_ids, return_hidden=True)


def dense_llama_logits(model, token_ids: list, return_hidden: bool = False) -> torch.Tensor:
    """Logits [S, V] of one sequence for a single-rank LlamaForCausalLM (fp32 math)."""
    cfg = model.cfg
    ids = torch.tensor(token_ids, dtype=torch.long, device=model.embed.device)
    S = ids.numel()
    pos = torch.arange(S, device=ids.device)
    x = model.embed[ids].float()
    Hq, Hkv, D = cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    for layer in model.layers:
        a = layer.self_attn
        h = _rms(x, layer.input_ln, cfg.rms_norm_eps)
        qkv = h @ dense_weight(a.qkv).t()
        if a.qkv.bias is not None:
            qkv = qkv + a.qkv.bias.float()
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], -1)
        q, k, v = q.view(S, Hq, D), k.view(S, Hkv, D), v.view(S, Hkv, D)
        if a.q_norm_w is not None:
            q, k = _rms(q, a.q_norm_w, cfg.rms_norm_eps), _rms(k, a.k_norm_w, cfg.rms_norm_eps)
        q = ref.apply_rope(q, pos, a.attn.inv_freq, cfg.rope_interleaved)
        k = ref.apply_rope(k, pos, a.attn.inv_freq, cfg.rope_interleaved)
        G = Hq // Hkv
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) * (D ** -0.5)
        mask = torch.ones(S, S, dtype=torch.bool, device=ids.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(S, Hq * D)
        x = x + o @ dense_weight(a.o).t()
        h = _rms(x, layer.post_ln, cfg.rms_norm_eps)
        if hasattr(layer.mlp, "gate_up"):
            gu = h @ dense_weight(layer.mlp.gate_up).t()
            I = gu.shape[-1] // 2
            x = x + (F.silu(gu[:, :I]) * gu[:, I:]) @ dense_weight(layer.mlp.down).t()
        else:
            x = x + layer.mlp.forward(h.to(cfg.dtype)).float()
    x = _rms(x, model.norm, cfg.rms_norm_eps)
    if return_hidden:
        return x
    return x @ model.lm_head.float().t()


@torch.no_grad()
def dense_greedy_generate(model, prompt: list, max_new_tokens: int) -> tuple[list, torch.Tensor]:
    toks = list(prompt)
    step_logits = []
    for _ in range(max_new_tokens):
        lg = dense_llama_logits(model, toks)[-1]
        step_logits.append(lg)
        toks.append(int(lg.argmax()))
    return toks[len(prompt):], torch.stack(step_logits)
