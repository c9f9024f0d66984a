"""Gated DeltaNet (linear attention) in plain PyTorch: causal depth-wise conv1d with a carried
window, and the gated delta-rule recurrence with a carried per-head state.

State per request: ``conv_state [C, kernel-1]`` and ``rec_state [Hv, dk, dv]`` (fp32), stored in
pools indexed by the request's state slot.  A request whose first token of the step has position 0
starts from zero state.  Recurrence for one head (``S`` is [dk, dv])::

    S   <- S * exp(g_t)
    u_t  = (v_t - k_t^T S) * beta_t
    S   <- S + k_t u_t^T
    o_t  = q_t^T S            (q scaled by dk^-1/2, q and k L2-normalised)

(reference math: src/vllm_torchtpu/kernels/gdn/v3/, layers/core/gdn_attention.py; the reference
runs a chunked WY form for prefill and this recurrence for decode; both give the same result)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_conv1d_update(x: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor,
                         bias=None, activation: bool = True):
    """x [T, C] tokens of ONE request in order; conv_state [C, K-1] (updated in place);
    weight [C, K].  Returns [T, C]."""
    T, C = x.shape
    K = weight.shape[1]
    window = torch.cat([conv_state.t().to(x.dtype), x], dim=0)            # [K-1+T, C]
    out = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    for j in range(K):
        out += window[j:j + T].float() * weight[:, j].float()[None, :]
    if bias is not None:
        out += bias.float()
    conv_state.copy_(window[-(K - 1):].t().to(conv_state.dtype))
    if activation:
        out = F.silu(out)
    return out.to(x.dtype)


def gated_delta_rule(q, k, v, g, beta, state):
    """q, k [T, Hk, dk]; v [T, Hv, dv]; g, beta [T, Hv]; state [Hv, dk, dv] fp32 (in place).
    Hk divides Hv (each k head serves Hv/Hk value heads).  Returns o [T, Hv, dv]."""
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf = F.normalize(q.float(), dim=-1).repeat_interleave(rep, dim=1) * (dk ** -0.5)
    kf = F.normalize(k.float(), dim=-1).repeat_interleave(rep, dim=1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    out = torch.empty(T, Hv, dv, dtype=torch.float32, device=q.device)
    S = state
    for t in range(T):
        S.mul_(torch.exp(gf[t])[:, None, None])
        kv_mem = torch.einsum("hkv,hk->hv", S, kf[t])
        u = (vf[t] - kv_mem) * bf[t][:, None]
        S.add_(kf[t][:, :, None] * u[:, None, :])
        out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
    return out.to(q.dtype)


def gdn_forward(mixed_qkv, a, b, z_unused, meta, conv_pool, rec_pool, conv_w, A_log, dt_bias,
                Hk: int, Hv: int, dk: int, dv: int):
    """Whole-batch driver: per request, conv over [q|k|v] channels then the recurrence.
    mixed_qkv [T, 2*Hk*dk + Hv*dv]; a, b [T, Hv]; pools are indexed by meta.state_slots."""
    T = mixed_qkv.shape[0]
    out = torch.zeros(T, Hv, dv, dtype=mixed_qkv.dtype, device=mixed_qkv.device)
    qsl = meta.query_start_loc.tolist()
    sl = meta.seq_lens.tolist()
    slots = meta.state_slots.tolist()
    beta = torch.sigmoid(b.float())
    g = -torch.exp(A_log.float())[None, :] * F.softplus(a.float() + dt_bias.float()[None, :])
    for r in range(meta.num_reqs):
        qs, qe = qsl[r], qsl[r + 1]
        if qe <= qs:
            continue
        slot = slots[r]
        if sl[r] - (qe - qs) == 0:                      # first tokens of the request: fresh state
            conv_pool[slot].zero_()
            rec_pool[slot].zero_()
        x = causal_conv1d_update(mixed_qkv[qs:qe], conv_pool[slot], conv_w)
        qh, kh, vh = x.split([Hk * dk, Hk * dk, Hv * dv], dim=-1)
        out[qs:qe] = gated_delta_rule(qh.reshape(-1, Hk, dk), kh.reshape(-1, Hk, dk), vh.reshape(-1, Hv, dv),
                                      g[qs:qe], beta[qs:qe], rec_pool[slot])
    return out


def kda_gate(a, A_log, dt_bias, lower_bound=None):
    """Raw gate a [T, Hv, dk] -> per-channel log-decay (<= 0); A_log [Hv], dt_bias [Hv, dk]
    (reference: src/vllm_torchtpu/kernels/gdn/v3/compute_kda.py:42-63)."""
    af = a.float() + dt_bias.float()[None]
    ea = torch.exp(A_log.float())[None, :, None]
    if lower_bound is None:
        return -ea * F.softplus(af)
    return lower_bound * torch.sigmoid(ea * af)


def kda_rule(q, k, v, g, beta, state):
    """Kimi Delta Attention recurrence: as gated_delta_rule, but g [T, Hv, dk] decays every key channel
    of the state on its own (reference: compute_kda.py:362-423).  state [Hv, dk, dv] fp32, in place."""
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf = q.float()
    kf = k.float()
    qf = (qf * torch.rsqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, dim=1) * (dk ** -0.5)
    kf = (kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, dim=1)
    vf, gf, bf = v.float(), g.float(), beta.float()
    out = torch.empty(T, Hv, dv, dtype=torch.float32, device=q.device)
    S = state
    for t in range(T):
        S.mul_(torch.exp(gf[t])[:, :, None])
        kv_mem = torch.einsum("hkv,hk->hv", S, kf[t])
        u = (vf[t] - kv_mem) * bf[t][:, None]
        S.add_(kf[t][:, :, None] * u[:, None, :])
        out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
    return out.to(q.dtype)


def kda_forward(q, k, v, a, b, meta, rec_pool, A_log, dt_bias, lower_bound=None):
    """Whole-batch driver of the KDA recurrence over a ragged batch; rec_pool [slots, Hv, dk, dv] fp32."""
    T, Hv, dv = v.shape
    out = torch.zeros(T, Hv, dv, dtype=v.dtype, device=v.device)
    qsl = meta.query_start_loc.tolist()
    sl = meta.seq_lens.tolist()
    slots = meta.state_slots.tolist()
    g = kda_gate(a, A_log, dt_bias, lower_bound)
    beta = torch.sigmoid(b.float())
    for r in range(meta.num_reqs):
        qs, qe = qsl[r], qsl[r + 1]
        if qe <= qs:
            continue
        slot = slots[r]
        if sl[r] - (qe - qs) == 0:
            rec_pool[slot].zero_()
        out[qs:qe] = kda_rule(q[qs:qe], k[qs:qe], v[qs:qe], g[qs:qe], beta[qs:qe], rec_pool[slot])
    return out
