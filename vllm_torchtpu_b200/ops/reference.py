"""Plain-PyTorch statements of every op, computed in fp32.

These are the oracles the CUDA kernels are tested against, and the code path
the engine runs on CPU tensors (unit tests, the CPU plumbing configuration).
Nothing here is tuned for speed.

KV cache layout (one tensor per layer): ``[num_blocks, 2, kv_heads, block_size,
head_dim]``; ``[:, 0]`` is K, ``[:, 1]`` is V.  A token's slot is
``block_id * block_size + offset``.

Batch description for attention, as in the reference's metadata
(reference: src/vllm_torchtpu/layers/core/attention_metadata.py:83-141):
``seq_lens[r]`` is the KV length of request r including this step's tokens,
``query_start_loc[r]:query_start_loc[r+1]`` are its rows in the packed token
dimension, ``block_tables[r]`` its pages.  New K/V are written at positions
``[seq_len - q_len, seq_len)`` before attention
(reference: src/vllm_torchtpu/kernels/ragged_paged_attention/v3/kernel.py:155-168).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def fused_add_rms_norm(x, residual, weight, eps):
    """residual' = round_to_dtype(x + residual); y = rms_norm(residual').
    The sum is rounded to the activation dtype before normalising
    (reference: src/vllm_torchtpu/layers/adapter/ir_ops.py:50-88)."""
    r = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(r, weight, eps), r


GATED_ACTS = ("silu", "gelu", "gelu_tanh", "swigluoai", "silu_clamp", "situ")


def parse_gated_act(spec: str) -> tuple:
    """"silu" | "gelu" | "gelu_tanh" | "swigluoai[:alpha:limit]" | "silu_clamp[:limit]" | "situ:beta[:linear_beta]"
    -> (index into GATED_ACTS, a, b)."""
    parts = str(spec).split(":")
    name = {"silu_and_mul_with_clamp": "silu_clamp"}.get(parts[0], parts[0])
    if name not in GATED_ACTS:
        raise ValueError(f"unknown gated activation {spec!r}; known: {GATED_ACTS}")
    nums = [float(p) if p not in ("", "none") else 0.0 for p in parts[1:]]
    if name == "swigluoai":
        a, b = (nums + [1.702, 7.0][len(nums):])[:2]
    elif name == "silu_clamp":
        a, b = 0.0, (nums + [10.0])[0]
    elif name == "situ":
        if not nums:
            raise ValueError("situ needs its beta: 'situ:<beta>[:<linear_beta>]'")
        a, b = nums[0], (nums[1] if len(nums) > 1 else 0.0)
    else:
        a, b = 0.0, 0.0
    return GATED_ACTS.index(name), a, b


def gated_act_and_mul(x: torch.Tensor, spec: str = "silu") -> torch.Tensor:
    """x [..., 2I] (gate columns first) -> act(gate, up) [..., I] in fp32 then the input dtype
    (reference: src/vllm_torchtpu/kernels/megablox/gmm_v2.py:30-58)."""
    act, a, b = parse_gated_act(spec)
    I = x.shape[-1] // 2
    g, u = x[..., :I].float(), x[..., I:].float()
    if act == 0:
        y = F.silu(g) * u
    elif act == 1:
        y = F.gelu(g) * u
    elif act == 2:
        y = F.gelu(g, approximate="tanh") * u
    elif act == 3:
        gc, uc = g.clamp(max=b), u.clamp(-b, b)
        y = (uc + 1.0) * gc * torch.sigmoid(a * gc)
    elif act == 4:
        y = F.silu(g.clamp(max=b)) * u.clamp(-b, b)
    else:
        y = a * torch.tanh(g / a) * torch.sigmoid(g) * (b * torch.tanh(u / b) if b > 0 else u)
    return y.to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (F.silu(g) * u).to(x.dtype)


def gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[T,N] = x[T,K] @ w[N,K]^T (+ bias), fp32 accumulate."""
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None,
                  rotary_dim: Optional[int] = None) -> torch.Tensor:
    rd = rotary_dim or head_dim
    inv = 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float64) / rd))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        smooth = (old / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor,
                             torch.where(wavelen < old / hi, inv,
                                         (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "linear":
        inv = inv / scaling["factor"]
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "yarn":
        # YaRN: dimensions that turn often inside the original context keep their frequency, slow ones are
        # interpolated by `factor`, with a linear ramp between the two correction dimensions
        factor = float(scaling["factor"])
        old = float(scaling.get("original_max_position_embeddings", 4096))
        fast, slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

        def corr_dim(rot):
            return rd * math.log(old / (rot * 2 * math.pi)) / (2 * math.log(theta))
        lo, hi = corr_dim(fast), corr_dim(slow)
        if scaling.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rd - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(rd // 2, dtype=torch.float64) - lo) / (hi - lo)).clamp(0, 1)
        keep = 1.0 - ramp
        inv = inv / factor * (1.0 - keep) + inv * keep
    return inv.float()


def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def rope_attention_factor(scaling: Optional[dict]) -> float:
    """Multiplier of cos / sin under YaRN (both q and k carry it, so attention logits scale by its square)."""
    if not scaling or scaling.get("rope_type", scaling.get("type")) != "yarn":
        return 1.0
    if scaling.get("attention_factor") is not None:
        return float(scaling["attention_factor"])
    factor = float(scaling["factor"])
    if scaling.get("mscale") and scaling.get("mscale_all_dim"):
        return yarn_mscale(factor, scaling["mscale"]) / yarn_mscale(factor, scaling["mscale_all_dim"])
    return yarn_mscale(factor)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
               interleaved: bool = False) -> torch.Tensor:
    """x: [T, H, D]; rotates the first 2*len(inv_freq) dims in fp32
    (reference: src/vllm_torchtpu/layers/adapter/rotary_embedding.py:14-44)."""
    rd = inv_freq.numel() * 2
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xr = x[..., :rd].float()
    if interleaved:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).flatten(-2)
    else:
        x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
        o = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
    out = x.clone()
    out[..., :rd] = o.to(x.dtype)
    return out


def head_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head RMSNorm over the last dim of [T, H, D] (Qwen3 q/k norm)."""
    return rms_norm(x, weight, eps)


def write_kv_cache(kv_cache: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   slot_mapping: torch.Tensor) -> None:
    """k, v: [T, Hkv, D]; slot < 0 skips the token (padding)."""
    bs = kv_cache.shape[3]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    blk, off = slots // bs, slots % bs
    kv_cache[blk, 0, :, off] = k[valid].to(kv_cache.dtype)
    kv_cache[blk, 1, :, off] = v[valid].to(kv_cache.dtype)


def rope_and_cache(qkv, positions, inv_freq, kv_cache, slot_mapping, num_q_heads, num_kv_heads,
                   head_dim, interleaved=False, q_norm_w=None, k_norm_w=None, eps=1e-6,
                   k_scale: float = 1.0, v_scale: float = 1.0):
    """Split packed qkv, optional per-head q/k RMSNorm, RoPE on q and k, write k/v
    to the paged cache.  Returns q [T, Hq, D]."""
    T = qkv.shape[0]
    q, k, v = qkv.split([num_q_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * head_dim], -1)
    q = q.reshape(T, num_q_heads, head_dim)
    k = k.reshape(T, num_kv_heads, head_dim)
    v = v.reshape(T, num_kv_heads, head_dim)
    if q_norm_w is not None:
        q = head_rms_norm(q, q_norm_w, eps)
        k = head_rms_norm(k, k_norm_w, eps)
    q = apply_rope(q, positions, inv_freq, interleaved)
    k = apply_rope(k, positions, inv_freq, interleaved)
    if kv_cache is not None:
        if kv_cache.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            write_kv_cache(kv_cache, k.float() / k_scale, v.float() / v_scale, slot_mapping)
        else:
            write_kv_cache(kv_cache, k, v, slot_mapping)
    return q.contiguous()


def paged_attention(q, kv_cache, block_tables, seq_lens, query_start_loc, scale, *,
                    num_reqs: Optional[int] = None, sliding_window: Optional[int] = None,
                    softcap: Optional[float] = None, sinks: Optional[torch.Tensor] = None,
                    k_scale: float = 1.0, v_scale: float = 1.0, return_lse: bool = False,
                    global_seq_lens=None, dcp_size: int = 1, dcp_rank: int = 0, dcp_interleave: int = 1):
    """Causal attention of packed ragged queries over the paged cache.

    q: [T, Hq, D]; returns [T, Hq, D] (rows beyond query_start_loc[num_reqs] are zero).
    Query j of request r sits at absolute position seq_len - q_len + j.

    Under decode context parallelism (``dcp_size`` > 1) the cache holds the positions p with
    ``(p // dcp_interleave) % dcp_size == dcp_rank``, ``seq_lens`` are local lengths and
    ``global_seq_lens`` the true ones: a query at global position g sees the local keys whose global
    position is <= g.
    """
    T, Hq, D = q.shape
    Hkv, bs = kv_cache.shape[2], kv_cache.shape[3]
    G = Hq // Hkv
    out = torch.zeros_like(q)
    lse = torch.full((T, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    R = int(num_reqs if num_reqs is not None else seq_lens.shape[0])
    qsl = query_start_loc.tolist()
    sl = seq_lens.tolist()
    for r in range(R):
        qs, qe = qsl[r], qsl[r + 1]
        q_len, kv_len = qe - qs, sl[r]
        if q_len <= 0 or kv_len <= 0:
            continue
        gl = int(global_seq_lens[r]) if dcp_size > 1 else kv_len
        nblk = -(-kv_len // bs)
        blocks = block_tables[r, :nblk].long()
        k = kv_cache[blocks, 0].float() * k_scale        # [nblk, Hkv, bs, D]
        v = kv_cache[blocks, 1].float() * v_scale
        k = k.permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :kv_len]
        v = v.permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :kv_len]
        qr = q[qs:qe].float().permute(1, 0, 2).reshape(Hkv, G, q_len, D)
        s = torch.einsum("hgqd,hkd->hgqk", qr, k) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        kpos = torch.arange(kv_len, device=q.device)[None, :]
        if dcp_size > 1:
            g = torch.arange(gl - q_len, gl, device=q.device) + 1          # keys at global positions < g
            period = dcp_interleave * dcp_size
            vis = (g // period) * dcp_interleave + (g % period - dcp_rank * dcp_interleave).clamp(0, dcp_interleave)
            qpos = (vis - 1)[:, None]
        else:
            qpos = torch.arange(kv_len - q_len, kv_len, device=q.device)[:, None]
        mask = kpos <= qpos
        if sliding_window:
            mask &= kpos > qpos - sliding_window
        s = s.masked_fill(~mask, float("-inf"))
        if sinks is not None:
            sink = sinks.float().reshape(Hkv, G, 1, 1).expand(Hkv, G, q_len, 1)
            s_all = torch.cat([s, sink], dim=-1)
            l = torch.logsumexp(s_all, dim=-1)
        else:
            l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - torch.where(torch.isfinite(l), l, torch.zeros_like(l))[..., None])
        p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))      # rows that see no key stay zero
        o = torch.einsum("hgqk,hkd->hgqd", p, v)
        out[qs:qe] = o.reshape(Hq, q_len, D).permute(1, 0, 2).to(q.dtype)
        lse[qs:qe] = l.reshape(Hq, q_len).t()
    if return_lse:
        return out, lse
    return out


def merge_attn_states(outs: list, lses: list):
    """Combine partial attention results by their log-sum-exp
    (reference: src/vllm_torchtpu/distributed/dcp_comm.py:23-46)."""
    lse = torch.stack(lses).float()                      # [P, T, H]
    m = lse.max(0).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w = torch.exp(lse - m)
    w = torch.where(torch.isfinite(lse), w, torch.zeros_like(w))
    denom = w.sum(0)
    o = sum(torch.where(w[i][..., None] > 0, outs[i].float() * w[i][..., None],
                        torch.zeros_like(outs[i], dtype=torch.float32)) for i in range(len(outs)))
    o = o / denom.clamp_min(1e-38)[..., None]
    return o.to(outs[0].dtype), m + torch.log(denom.clamp_min(1e-38))


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table[ids.long()]


# ---- sampling ------------------------------------------------------------------
def apply_top_k_top_p(logits: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor) -> torch.Tensor:
    """Mask logits outside each row's top-k / nucleus to -inf.  top_k<=0 and top_p>=1 are off."""
    logits = logits.float().clone()
    V = logits.shape[-1]
    sorted_logits, idx = logits.sort(dim=-1, descending=True)
    k = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k).clamp(max=V).long()
    ranks = torch.arange(V, device=logits.device)[None, :]
    keep = ranks < k[:, None]
    probs = torch.softmax(sorted_logits.masked_fill(~keep, float("-inf")), dim=-1)
    cum = probs.cumsum(-1)
    keep &= (cum - probs) < top_p[:, None].float()
    keep[:, 0] = True
    masked = sorted_logits.masked_fill(~keep, float("-inf"))
    out = torch.empty_like(logits)
    out.scatter_(1, idx, masked)
    return out


def gumbel_from_uniform(u: torch.Tensor) -> torch.Tensor:
    return -torch.log(-torch.log(u.clamp(1e-20, 1.0 - 1e-7)))


def sample(logits, temperature, top_k, top_p, uniform: Optional[torch.Tensor] = None):
    """Greedy where temperature <= 1e-5, else Gumbel-max over the masked, tempered
    logits (reference: src/vllm_torchtpu/runner/tpu_runner.py:9240-9274)."""
    logits = logits.float()
    greedy = logits.argmax(-1)
    if uniform is None or bool((temperature <= 1e-5).all()):
        return greedy
    t = temperature.clamp_min(1e-5)[:, None].float()
    masked = apply_top_k_top_p(logits / t, top_k, top_p)
    noisy = masked + gumbel_from_uniform(uniform.float())
    rnd = noisy.argmax(-1)
    return torch.where(temperature <= 1e-5, greedy, rnd)


def gather_logprobs(logits, token_ids, k: int):
    """fp32 log-softmax; returns (logprob of token_ids, top-k logprobs, top-k ids, rank)."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    tok = lp.gather(1, token_ids.long()[:, None]).squeeze(1)
    topv, topi = lp.topk(k, dim=-1) if k > 0 else (lp[:, :0], token_ids[:, None][:, :0])
    rank = (lp > tok[:, None]).sum(-1) + 1
    return tok, topv, topi, rank


# ---- MoE ------------------------------------------------------------------------
def moe_route(router_logits, top_k: int, scoring: str = "softmax", renormalize: bool = True,
              routed_scaling: float = 1.0, score_bias: Optional[torch.Tensor] = None,
              n_group: int = 1, topk_group: int = 1):
    """scoring → (bias / grouped top-k) → top-k → renormalise → scale
    (reference: src/vllm_torchtpu/layers/adapter/moe_routing.py:161-343)."""
    x = router_logits.float()
    scores = torch.softmax(x, dim=-1) if scoring == "softmax" else torch.sigmoid(x)
    choice = scores if score_bias is None else scores + score_bias.float()[None, :]
    T, E = scores.shape
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        if score_bias is not None:
            gs = g.topk(2, dim=-1).values.sum(-1)
        else:
            gs = g.max(-1).values
        gidx = gs.topk(topk_group, dim=-1).indices
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=x.device).scatter_(1, gidx, True)
        choice = choice.masked_fill(~gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E),
                                    float("-inf"))
    ids = choice.topk(top_k, dim=-1).indices
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    return ids.to(torch.int32), (w * routed_scaling).float()


def moe_route_post(ids, w, num_experts: int, num_valid=None, sim: str = ""):
    """Padding mask and routing simulation after the router (same rules as the CUDA kernel)."""
    T, k = ids.shape
    if sim == "uniform":
        ids.copy_((torch.arange(T * k, device=ids.device) % num_experts).view(T, k).to(ids.dtype))
        w.fill_(1.0 / k)
    elif sim == "hash":
        t = torch.arange(T, device=ids.device, dtype=torch.int64)
        h = (t * 2654435761) & 0xFFFFFFFF
        h = h ^ (h >> 15)
        h = (h * 2246822519) & 0xFFFFFFFF
        h = h ^ (h >> 13)
        stride = max(1, num_experts // k)
        j = torch.arange(k, device=ids.device, dtype=torch.int64)
        ids.copy_(((h % num_experts)[:, None] + j[None, :] * stride) % num_experts)
        w.fill_(1.0 / k)
    if num_valid is not None:
        n = int(num_valid[0])
        ids[n:] = -1
        w[n:] = 0
    return ids, w


def moe_experts(x, w13, w2, topk_ids, topk_w, expert_offset: int = 0, act: str = "silu", b13=None, b2=None):
    """Σ_k w_k · FFN_e(x) over the experts this rank owns.  w13: [E_local, 2I, H] (gate rows first),
    w2: [E_local, H, I] (rows beyond H, padding for the kernels' tile width, are ignored); ``act``: gated
    activation (``parse_gated_act``); optional expert biases b13 [E_local, 2I], b2 [E_local, H]."""
    T, H = x.shape
    E_local = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(E_local):
        sel = (topk_ids == e + expert_offset)
        rows = sel.any(-1).nonzero().squeeze(-1)
        if rows.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[rows]
        h = xf[rows] @ w13[e].float().t()
        if b13 is not None:
            h = (h.to(x.dtype).float() + b13[e].float())
        a = gated_act_and_mul(h, act).to(x.dtype).float()
        y = (a @ w2[e, :H].float().t()).to(x.dtype).float()
        if b2 is not None:
            y = (y + b2[e, :H].float()).to(x.dtype).float()
        out[rows] += y * wt[:, None]
    return out.to(x.dtype)


# ---- MLA -------------------------------------------------------------------------
def mla_write_cache(cache: torch.Tensor, kv_c: torch.Tensor, k_pe: torch.Tensor,
                    slot_mapping: torch.Tensor) -> None:
    """cache: [num_blocks, block_size, kv_lora + rope]; row = kv_c_normed ‖ k_pe
    (reference: src/vllm_torchtpu/layers/adapter/attention.py:2718-2727)."""
    bs = cache.shape[1]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    row = torch.cat([kv_c[valid], k_pe[valid]], dim=-1).to(cache.dtype)
    cache[slots // bs, slots % bs] = row


def mla_paged_attention(q_latent, cache, block_tables, seq_lens, query_start_loc, scale, kv_lora_rank: int,
                        *, num_reqs: Optional[int] = None, topk_indices: Optional[torch.Tensor] = None,
                        return_lse: bool = False):
    """Absorbed-query MLA: q_latent [T, H, kv_lora + rope] against latent rows; the value of a
    row is its first ``kv_lora_rank`` dims.  Returns [T, H, kv_lora_rank].
    ``topk_indices`` [T, K] (sparse MLA): each query attends only the listed positions (-1 = unused)."""
    T, H, Dq = q_latent.shape
    bs = cache.shape[1]
    out = torch.zeros(T, H, kv_lora_rank, dtype=q_latent.dtype, device=q_latent.device)
    lse = torch.full((T, H), float("-inf"), dtype=torch.float32, device=q_latent.device)
    R = int(num_reqs if num_reqs is not None else seq_lens.shape[0])
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    for r in range(R):
        qs, qe = qsl[r], qsl[r + 1]
        q_len, kv_len = qe - qs, sl[r]
        if q_len <= 0 or kv_len <= 0:
            continue
        nblk = -(-kv_len // bs)
        rows = cache[block_tables[r, :nblk].long()].reshape(nblk * bs, Dq)[:kv_len].float()
        s = torch.einsum("qhd,kd->hqk", q_latent[qs:qe].float(), rows) * scale
        qpos = torch.arange(kv_len - q_len, kv_len, device=s.device)[:, None]
        kpos = torch.arange(kv_len, device=s.device)[None, :]
        mask = kpos <= qpos
        if topk_indices is not None:
            sel = torch.zeros(q_len, kv_len, dtype=torch.bool, device=s.device)
            idx = topk_indices[qs:qe].long()
            ok = (idx >= 0) & (idx < kv_len)
            qrow = torch.arange(q_len, device=s.device)[:, None].expand_as(idx)
            sel[qrow[ok], idx[ok]] = True           # unused (-1) and out-of-range entries select nothing
            mask = mask & sel
        s = s.masked_fill(~mask[None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None])
        p = torch.where(torch.isfinite(l)[..., None], p, torch.zeros_like(p))
        o = torch.einsum("hqk,kd->qhd", p, rows[:, :kv_lora_rank])
        out[qs:qe] = o.to(out.dtype)
        lse[qs:qe] = l.t()
    if return_lse:
        return out, lse
    return out


def encoder_attention(q, k, v, cu_seqlens, scale=None):
    """Bidirectional attention inside each sequence of a ragged batch (fp32 oracle).
    q [T, Hq, D]; k, v [T, Hkv, D]; cu_seqlens: R + 1 offsets."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    sc = float(scale) if scale is not None else D ** -0.5
    out = torch.zeros_like(q)
    for r in range(len(cu_seqlens) - 1):
        a, b = int(cu_seqlens[r]), int(cu_seqlens[r + 1])
        if b <= a:
            continue
        qr = q[a:b].float().permute(1, 0, 2).reshape(Hkv, G, b - a, D)
        kr, vr = k[a:b].float().permute(1, 0, 2), v[a:b].float().permute(1, 0, 2)
        p = torch.softmax(torch.einsum("hgqd,hkd->hgqk", qr, kr) * sc, dim=-1)
        o = torch.einsum("hgqk,hkd->hgqd", p, vr).reshape(Hq, b - a, D).permute(1, 0, 2)
        out[a:b] = o.to(q.dtype)
    return out
