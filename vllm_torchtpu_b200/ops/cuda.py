"""ctypes bindings of the in-tree sm_100a kernel library.

The library is ``csrc/libb200_kernels.so`` (built by ``csrc/build.py``; plain C
ABI, raw device pointers, the caller's CUDA stream).  Importing this module on a
machine with a GPU but without the built library raises: there is no PyTorch
fallback for CUDA tensors.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p
from typing import Optional

import torch

from .. import envs
from . import count_launch

_lib = None
_sms = 148


class _Overlay:
    """Symbols of ``over`` where it defines them, of ``main`` otherwise."""

    def __init__(self, main, over):
        self._main, self._over = main, over

    def __getattr__(self, name):
        try:
            f = getattr(self._over, name)
        except AttributeError:
            f = getattr(self._main, name)
        setattr(self, name, f)
        return f


def bad_index_count() -> int:
    """Out-of-range block ids / page indices seen by the attention kernels since the last call (counted only
    by the bounds-checked library, ``B200_BOUNDS_CHECK=1``)."""
    total = 0
    for name in ("b200_bad_index_count_attention", "b200_bad_index_count_attention_tc",
                 "b200_bad_index_count_attention_mla"):
        v = ctypes.c_uint(0)
        _check(getattr(lib(), name)(ctypes.byref(v)), name)
        total += v.value
    return total


def reload_lib(path: Optional[str] = None) -> str:
    """Forget the loaded kernel library and load it again, from ``path`` or from the in-tree build.  A copy
    under a fresh name is opened, because the dynamic loader hands back the already mapped object for a
    path it knows."""
    global _lib
    import shutil
    import tempfile
    from ..csrc import build as _build
    src = path or envs.B200_KERNEL_LIB or _build.lib_path()
    if not os.path.exists(src):
        raise RuntimeError(f"kernel library {src} is missing")
    fd, tmp = tempfile.mkstemp(prefix="libb200_kernels_", suffix=".so")
    os.close(fd)
    shutil.copyfile(src, tmp)
    # local scope and own symbols first: the copy must not bind to the functions of the library it replaces
    new = ctypes.CDLL(tmp, mode=os.RTLD_LOCAL | os.RTLD_DEEPBIND)
    new.b200_get_last_error.restype = ctypes.c_char_p
    new.b200_attn_decode_scratch_bytes.restype = c_size_t
    _lib = new
    return src


def lib():
    global _lib, _sms
    if _lib is not None:
        return _lib
    from ..csrc import build as _build
    path = envs.B200_KERNEL_LIB or _build.lib_path()
    if not os.path.exists(path):
        raise RuntimeError(f"kernel library {path} is missing; run `python -m vllm_torchtpu_b200.csrc.build`")
    _lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    _lib.b200_get_last_error.restype = ctypes.c_char_p
    _lib.b200_attn_decode_scratch_bytes.restype = c_size_t
    if envs.B200_BOUNDS_CHECK:
        # the attention kernels from the bounds-checked library, everything else from the main one
        checked = _build.checked_lib_path()
        if not os.path.exists(checked):
            raise RuntimeError(f"{checked} is missing; run `python -m vllm_torchtpu_b200.csrc.build`")
        over = ctypes.CDLL(checked)
        over.b200_attn_decode_scratch_bytes.restype = c_size_t
        _lib = _Overlay(_lib, over)
    if torch.cuda.is_available():
        _sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().b200_get_last_error().decode()
        raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


class Workspace:
    """Per-device scratch shared by all launches on the engine's stream."""

    _by_device: dict = {}

    def __init__(self, device):
        self.device = device
        self.gemm_ws = torch.empty(64 * 2**20, dtype=torch.uint8, device=device)
        self.gemm_counters = torch.zeros(16384, dtype=torch.int32, device=device)
        self.attn_scratch = torch.empty(48 * 2**20, dtype=torch.uint8, device=device)
        self.attn_counters = torch.zeros(65536, dtype=torch.int32, device=device)
        self.status = torch.zeros(16, dtype=torch.int32, device=device)
        self.rng_step = torch.zeros(1, dtype=torch.int64, device=device)
        self._attn_out: dict = {}

    def attn_out(self, T: int, Hq: int, D: int) -> torch.Tensor:
        """Attention output buffer for (T, Hq, D): two per shape, used alternately (consecutive layers
        consume the output before the next attention runs on the same stream)."""
        key = (T, Hq, D)
        ring = self._attn_out.get(key)
        if ring is None:
            if torch.cuda.is_current_stream_capturing():
                # memory allocated during capture belongs to that graph: do not keep it
                return torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=self.device)
            ring = self._attn_out[key] = [
                [torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=self.device) for _ in range(2)], 0]
        ring[1] ^= 1
        return ring[0][ring[1]]

    @classmethod
    def get(cls, device) -> "Workspace":
        key = torch.device(device).index or 0
        ws = cls._by_device.get(key)
        if ws is None:
            ws = cls._by_device[key] = Workspace(device)
        return ws


def check_status(device=None) -> int:
    """Read (and clear) the status word that bounded device waits write on timeout."""
    ws = Workspace.get(device or torch.cuda.current_device())
    v = int(ws.status[0].item())
    if v:
        ws.status.zero_()
    return v


# ------------------------------------------------------------------ elementwise
def _require_bf16(*ts):
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"sm_100a kernels take bfloat16 tensors, got {t.dtype}")


def rms_norm(x, weight, eps):
    _require_bf16(x, weight)
    x = x.contiguous()
    y = torch.empty_like(x)
    T, H = x.numel() // x.shape[-1], x.shape[-1]
    _check(lib().b200_rms_norm(_p(x), c_void_p(0), _p(weight), _p(y), c_int(T), c_int(H), c_float(eps),
                               _stream()), "rms_norm")
    count_launch()
    return y


def fused_add_rms_norm(x, residual, weight, eps):
    """In-place on ``residual`` (residual += x), returns (normed, residual)."""
    _require_bf16(x, residual, weight)
    x = x.contiguous()
    assert residual.is_contiguous()
    y = torch.empty_like(x)
    T, H = x.numel() // x.shape[-1], x.shape[-1]
    _check(lib().b200_rms_norm(_p(x), _p(residual), _p(weight), _p(y), c_int(T), c_int(H), c_float(eps),
                               _stream()), "fused_add_rms_norm")
    count_launch()
    return y, residual


def gated_act_and_mul(x, spec: str = "silu"):
    """x [T, 2I] bf16 (gate columns first) -> act(gate, up) [T, I]; ``spec`` as in
    ``ops.reference.parse_gated_act`` (silu, gelu, gelu_tanh, swigluoai, silu_clamp, situ)."""
    from .reference import parse_gated_act
    _require_bf16(x)
    act, a, b = parse_gated_act(spec)
    x = x.contiguous()
    T, I2 = x.shape
    y = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device)
    _check(lib().b200_gated_act(_p(x), _p(y), c_int(T), c_int(I2 // 2), c_int(act), ctypes.c_float(a),
                                ctypes.c_float(b), _stream()), "gated_act")
    count_launch()
    return y


def silu_and_mul(x):
    _require_bf16(x)
    x = x.contiguous()
    T, I2 = x.shape
    y = torch.empty((T, I2 // 2), dtype=x.dtype, device=x.device)
    _check(lib().b200_silu_and_mul(_p(x), _p(y), c_int(T), c_int(I2 // 2), _stream()), "silu_and_mul")
    count_launch()
    return y


def embedding(ids, table, token_src=None, last_tokens=None):
    _require_bf16(table)
    T = ids.numel()
    out = torch.empty((T, table.shape[1]), dtype=table.dtype, device=table.device)
    assert ids.dtype == torch.int32
    _check(lib().b200_embedding(_p(ids), _p(token_src), _p(last_tokens), _p(table), _p(out), c_int(T),
                                c_int(table.shape[1]), c_int(table.shape[0]), _stream()), "embedding")
    count_launch()
    return out


def gather_rows(hidden, residual, idx):
    R, H = idx.numel(), hidden.shape[1]
    oh = torch.empty((R, H), dtype=hidden.dtype, device=hidden.device)
    orr = torch.empty_like(oh) if residual is not None else None
    _check(lib().b200_gather_rows(_p(hidden), _p(residual), _p(idx), _p(oh), _p(orr), c_int(R), c_int(H),
                                  c_int(hidden.shape[0]), _stream()), "gather_rows")
    count_launch()
    return oh, orr


def scatter_tokens(tokens, slots, last_tokens):
    _check(lib().b200_scatter_tokens(_p(tokens), _p(slots), _p(last_tokens), c_int(tokens.numel()),
                                     c_int(last_tokens.numel()), _stream()), "scatter_tokens")
    count_launch()


def rope_and_cache(qkv, positions, inv_freq, kv_cache, slot_mapping, num_q_heads, num_kv_heads, head_dim,
                   interleaved=False, q_norm_w=None, k_norm_w=None, eps=1e-6, k_scale=1.0, v_scale=1.0):
    _require_bf16(qkv, q_norm_w, k_norm_w)
    qkv = qkv.contiguous()
    T = qkv.shape[0]
    q = torch.empty((T, num_q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    rot_pairs = inv_freq.numel()
    if not interleaved and rot_pairs * 2 != head_dim:
        raise NotImplementedError("partial rotary with half-rotation layout")
    if positions.dtype != torch.int32:
        positions = positions.to(torch.int32)
    if kv_cache is not None:
        nb, bs = kv_cache.shape[0], kv_cache.shape[3]
        eb = kv_cache.element_size()
    else:
        nb, bs, eb = 0, 16, 2
    _check(lib().b200_rope_and_cache(
        _p(qkv), _p(positions), _p(inv_freq), c_int(rot_pairs), _p(slot_mapping), _p(q), _p(kv_cache),
        _p(q_norm_w), _p(k_norm_w), c_float(eps), c_int(T), c_int(num_q_heads), c_int(num_kv_heads),
        c_int(head_dim), c_int(bs), c_longlong(nb), c_int(1 if interleaved else 0), c_int(eb),
        c_float(k_scale), c_float(v_scale), _stream()), "rope_and_cache")
    count_launch()
    return q


# ------------------------------------------------------------------------ GEMM
def gemm(x, w, bias=None, out=None, force_splits: int = 0):
    """y[T,N] = x[T,K] @ w[N,K]^T (+bias) on the tcgen05 kernel."""
    _require_bf16(x, w, bias)
    if envs.B200_GEMM_IMPL == "cublas":
        y = torch.nn.functional.linear(x, w, bias)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if x.stride(-1) != 1:
        x = x.contiguous()
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.stride(1) == 1
    y = out if out is not None else torch.empty((T, N), dtype=x.dtype, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    ws = Workspace.get(x.device)
    if force_splits == 0 and 0 < envs.B200_GEMM_2SM_MIN_T <= T:
        _check(lib().b200_gemm_bf16_2sm(
            _p(x2), _p(w), _p(y), _p(bias), c_int(T), c_int(N), c_int(K), c_int(x2.stride(0)),
            c_int(w.stride(0)), c_int(y.stride(0)), _p(ws.status), c_int(_sms), _stream()), "gemm_2sm")
        count_launch()
        return y.reshape(*lead, N)
    _check(lib().b200_gemm_bf16(
        _p(x2), _p(w), _p(y), _p(bias), c_int(T), c_int(N), c_int(K), c_int(x2.stride(0)), c_int(w.stride(0)),
        c_int(y.stride(0)), _p(ws.gemm_ws), c_size_t(ws.gemm_ws.numel()), _p(ws.gemm_counters),
        c_int(ws.gemm_counters.numel()), _p(ws.status), c_int(_sms), c_int(force_splits), _stream()), "gemm")
    count_launch()
    return y.reshape(*lead, N)


def gemm_plan(T, N, K):
    bn, sp, wsb, cn = c_int(), c_int(), c_size_t(), c_int()
    lib().b200_gemm_plan(c_int(T), c_int(N), c_int(K), c_int(_sms), ctypes.byref(bn), ctypes.byref(sp),
                         ctypes.byref(wsb), ctypes.byref(cn))
    return bn.value, sp.value, wsb.value, cn.value


# ------------------------------------------------------------------- attention
def decode_splits(num_reqs: int, num_kv_heads: int) -> int:
    if envs.B200_ATTN_SPLIT_KV > 0:
        return envs.B200_ATTN_SPLIT_KV
    # two CTAs are resident per SM.  Splitting costs a scratch round trip and a second merge, so the
    # (request, kv head) pairs are split only when they cannot fill one wave of resident CTAs.
    slots = 2 * _sms
    pairs = max(1, num_reqs * num_kv_heads)
    if pairs >= slots:
        return 1
    return max(1, min(16, slots // pairs))


def paged_attention(q, kv_cache, meta, scale, *, sliding_window=None, softcap=None, sinks=None,
                    k_scale=1.0, v_scale=1.0, return_lse=False):
    """Ragged paged attention over [decode | prefill/mixed] request ranges of the batch."""
    _require_bf16(q)
    # an e4m3 cache is expanded to bf16 in shared memory by the mma.sync kernels; k_scale joins the
    # logit scale and v_scale the output normalisation (reference: layers/adapter/quantization.py:91)
    kv_fp8 = 1 if kv_cache.dtype == torch.float8_e4m3fn else 0
    if not kv_fp8 and kv_cache.dtype != torch.bfloat16:
        raise NotImplementedError(f"KV cache dtype {kv_cache.dtype}: bf16 or float8_e4m3fn")
    T, Hq, D = q.shape
    nb, _, Hkv, bs, _ = kv_cache.shape
    ws = Workspace.get(q.device)
    if return_lse:
        # callers that merge partial results keep several outputs alive: fresh, fully defined tensors
        out = torch.zeros_like(q)
        lse = torch.full((T, Hq), float("-inf"), dtype=torch.float32, device=q.device)
    else:
        # rows of padded requests are never written; a reused zero-initialised buffer keeps them
        # finite without a fill kernel per layer
        out, lse = ws.attn_out(T, Hq, D), None
    G = Hq // Hkv
    R = meta.num_reqs
    R_launch = meta.padded_num_reqs if meta.padded_num_reqs is not None else R
    nd = meta.num_decode_reqs
    max_blocks = meta.block_tables.shape[1]
    window = int(sliding_window) if sliding_window else 0
    cap = float(softcap) if softcap else 0.0
    L = lib()
    if nd > 0 and G <= 16:
        # decode range; in a padded (graph) step all launched requests are decode-shaped
        n_dec = R_launch if nd == R else nd
        splits = decode_splits(n_dec, Hkv)
        need = L.b200_attn_decode_scratch_bytes(c_int(n_dec), c_int(Hkv), c_int(splits), c_int(D))
        if need > ws.attn_scratch.numel() or n_dec * Hkv > ws.attn_counters.numel():
            splits = 1
        args = (_p(q), _p(kv_cache), _p(out), _p(lse), _p(meta.block_tables), _p(meta.seq_lens),
                _p(meta.query_start_loc), c_int(0), c_int(n_dec), c_int(max_blocks), c_int(bs), c_longlong(nb),
                c_int(Hq), c_int(Hkv), c_int(D), c_float(scale), c_int(window), c_float(cap), _p(sinks),
                c_int(splits), _p(ws.attn_scratch), _p(ws.attn_counters))
        if kv_fp8:
            _check(L.b200_attn_decode_fp8kv(*args, c_float(k_scale), c_float(v_scale), _stream()),
                   "attn_decode_fp8kv")
        else:
            _check(L.b200_attn_decode(*args, _stream()), "attn_decode")
        count_launch()
    else:
        nd = 0
    if R > nd:
        qsl = meta.query_start_loc_cpu
        if qsl is not None:
            ql = (qsl[nd + 1:R + 1] - qsl[nd:R])
            tiles = int(((ql + 63) // 64).sum())
        else:
            tiles = (T + 63) // 64 + (R - nd)
        if meta.dcp_size > 1:
            # the cache holds this rank's share of the positions: local lengths, visibility by global position
            if kv_fp8 or window or sinks is not None:
                raise NotImplementedError("decode context parallelism: bf16 cache, no sliding window, no sinks")
            _check(L.b200_attn_prefill_dcp(
                _p(q), _p(kv_cache), _p(out), _p(lse), _p(meta.block_tables), _p(meta.seq_lens),
                _p(meta.global_seq_lens), _p(meta.query_start_loc), c_int(nd), c_int(R), c_int(tiles),
                c_int(max_blocks), c_int(bs), c_longlong(nb), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale),
                c_float(cap), c_int(meta.dcp_size), c_int(meta.dcp_rank), c_int(meta.dcp_interleave), _stream()),
                "attn_prefill_dcp")
        elif D == 128 and G in (1, 2, 4, 8) and envs.B200_ATTN_PREFILL_IMPL == "tc" and not kv_fp8:
            # tcgen05 kernel: one CTA per (kv head, 128 / G positions), K/V shared by the GQA group
            _check(L.b200_attn_prefill_tc(
                _p(q), _p(kv_cache), _p(out), _p(lse), _p(meta.block_tables), _p(meta.seq_lens),
                _p(meta.query_start_loc), c_int(nd), c_int(R), c_int(tiles), c_int(T), c_int(max_blocks),
                c_int(bs), c_longlong(nb), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale), c_int(window),
                c_float(cap), _p(sinks), _p(ws.status), _stream()), "attn_prefill_tc")
        else:
            args = (_p(q), _p(kv_cache), _p(out), _p(lse), _p(meta.block_tables), _p(meta.seq_lens),
                    _p(meta.query_start_loc), c_int(nd), c_int(R), c_int(tiles), c_int(max_blocks), c_int(bs),
                    c_longlong(nb), c_int(Hq), c_int(Hkv), c_int(D), c_float(scale), c_int(window),
                    c_float(cap), _p(sinks))
            if kv_fp8:
                _check(L.b200_attn_prefill_fp8kv(*args, c_float(k_scale), c_float(v_scale), _stream()),
                       "attn_prefill_fp8kv")
            else:
                _check(L.b200_attn_prefill(*args, _stream()), "attn_prefill")
        count_launch()
    if return_lse:
        return out, lse
    return out


def encoder_attention(q, k, v, cu_seqlens, scale=None):
    """Bidirectional attention over a ragged batch of sequences (vision encoders).  q [T, Hq, D], k / v
    [T, Hkv, D] bf16, ``cu_seqlens`` = list of R + 1 token offsets.  Keys and values are packed into the
    paged layout of the attention kernels and the prefill kernel runs with the causal mask off: the tcgen05
    kernel for 128-wide heads, the mma.sync kernel for 64-wide ones
    (reference: src/vllm_torchtpu/kernels/flash_attention/ — segment-id flash attention;
    kernels/diffusion_attention/kernel.py — dense attention of the diffusion transformers)."""
    _require_bf16(q, k, v)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    bs = 16
    lens = [int(cu_seqlens[i + 1]) - int(cu_seqlens[i]) for i in range(len(cu_seqlens) - 1)]
    R = len(lens)
    nblk = [-(-n // bs) for n in lens]
    max_blocks = max(1, max(nblk) if nblk else 1)
    NB = max(1, sum(nblk))
    dev = q.device
    bt = torch.zeros((R, max_blocks), dtype=torch.int32)
    slots = torch.empty(T, dtype=torch.long)
    off = 0
    for r, n in enumerate(lens):
        bt[r, :nblk[r]] = torch.arange(off, off + nblk[r], dtype=torch.int32)
        slots[int(cu_seqlens[r]):int(cu_seqlens[r + 1])] = off * bs + torch.arange(n)
        off += nblk[r]
    flat = torch.zeros((NB * bs, 2, Hkv, D), dtype=q.dtype, device=dev)
    slots = slots.to(dev)
    flat[slots, 0] = k
    flat[slots, 1] = v
    cache = flat.view(NB, bs, 2, Hkv, D).permute(0, 2, 3, 1, 4).contiguous()
    bt_d = bt.to(dev)
    sl = torch.tensor(lens, dtype=torch.int32, device=dev)
    qsl = torch.tensor([int(c) for c in cu_seqlens], dtype=torch.int32, device=dev)
    out = torch.zeros_like(q)
    tiles = sum(-(-n // 64) for n in lens)
    sc = float(scale) if scale is not None else D ** -0.5
    qc = q.contiguous()
    if D == 128 and Hq // Hkv in (1, 2, 4, 8) and envs.B200_ATTN_PREFILL_IMPL == "tc":
        # the tcgen05 prefill kernel with the causal mask off: one CTA per (kv head, 128 / G positions)
        ws = Workspace.get(dev)
        _check(lib().b200_attn_encoder_tc(
            _p(qc), _p(cache), _p(out), c_void_p(0), _p(bt_d), _p(sl), _p(qsl), c_int(0), c_int(R), c_int(tiles),
            c_int(T), c_int(max_blocks), c_int(bs), c_longlong(NB), c_int(Hq), c_int(Hkv), c_int(D), c_float(sc),
            _p(ws.status), _stream()), "attn_encoder_tc")
    else:
        _check(lib().b200_attn_encoder(
            _p(qc), _p(cache), _p(out), c_void_p(0), _p(bt_d), _p(sl), _p(qsl), c_int(0), c_int(R), c_int(tiles),
            c_int(max_blocks), c_int(bs), c_longlong(NB), c_int(Hq), c_int(Hkv), c_int(D), c_float(sc), _stream()),
            "attn_encoder")
    count_launch()
    return out


# -------------------------------------------------------------------- sampling
def _logit_dtype(t):
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"logits must be bf16 or fp32, got {t.dtype}")


def argmax(logits):
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    _check(lib().b200_argmax(_p(logits), c_int(_logit_dtype(logits)), c_int(R), c_int(V),
                             c_int(logits.stride(0)), _p(out), _stream()), "argmax")
    count_launch()
    return out


def sample(logits, temperature, top_k, top_p, uniform=None, all_greedy=False, seed: int = 0,
           step_tensor=None):
    if all_greedy:
        return argmax(logits)
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    _check(lib().b200_sample(_p(logits), c_int(_logit_dtype(logits)), c_int(R), c_int(V),
                             c_int(logits.stride(0)), _p(temperature), _p(top_k), _p(top_p), _p(uniform),
                             c_ulonglong(seed), c_ulonglong(0), _p(step_tensor), _p(out), _stream()), "sample")
    count_launch()
    return out


def spec_accept(target_tokens, input_ids, query_start_loc, spec_k, R: int, kmax: int):
    """Device-side acceptance of deterministic drafts (see ``spec_accept_kernel``): returns
    (tokens [R, kmax + 1] padded with -1, count [R])."""
    out = torch.empty((R, kmax + 1), dtype=torch.int32, device=target_tokens.device)
    cnt = torch.empty(R, dtype=torch.int32, device=target_tokens.device)
    _check(lib().b200_spec_accept(_p(target_tokens), _p(input_ids), _p(query_start_loc), _p(spec_k), c_int(R),
                                  c_int(kmax), _p(out), _p(cnt), _stream()), "spec_accept")
    count_launch()
    return out, cnt


def rejection_sample(logits, drafts, draft_probs, spec_k, temperature, uniform, resample_uniform):
    """Rejection sampling of sampled drafts on the device.  logits [sum(k_i + 1), V] (rows of request r are
    consecutive), drafts [R, kmax] int32, draft_probs [R, kmax, V] fp32 or None (one-hot), spec_k [R] int32,
    temperature [R], uniform [R, kmax], resample_uniform [R, kmax + 1] -> (tokens [R, kmax + 1], count [R])."""
    R, kmax = drafts.shape
    V = logits.shape[1]
    out = torch.empty((R, kmax + 1), dtype=torch.int32, device=logits.device)
    cnt = torch.empty(R, dtype=torch.int32, device=logits.device)
    _check(lib().b200_rejection_sample(
        _p(logits), c_int(_logit_dtype(logits)), c_int(R), c_int(V), c_int(logits.stride(0)), _p(drafts),
        _p(draft_probs), _p(spec_k), _p(temperature), _p(uniform), _p(resample_uniform), c_int(kmax), _p(out),
        _p(cnt), _stream()), "rejection_sample")
    count_launch()
    return out, cnt


def gather_logprobs(logits, token_ids, k: int):
    R, V = logits.shape
    dev = logits.device
    tok_lp = torch.empty(R, dtype=torch.float32, device=dev)
    top_lp = torch.empty((R, max(k, 1)), dtype=torch.float32, device=dev)
    top_id = torch.empty((R, max(k, 1)), dtype=torch.int32, device=dev)
    rank = torch.empty(R, dtype=torch.int32, device=dev)
    _check(lib().b200_logprobs(_p(logits), c_int(_logit_dtype(logits)), c_int(R), c_int(V),
                               c_int(logits.stride(0)), _p(token_ids.to(torch.int32)), c_int(k), _p(tok_lp),
                               _p(top_lp), _p(top_id), _p(rank), _stream()), "logprobs")
    count_launch()
    return tok_lp, top_lp[:, :k], top_id[:, :k], rank


def philox_uniform(R, V, seed, step, device):
    out = torch.empty((R, V), dtype=torch.float32, device=device)
    _check(lib().b200_philox_uniform(_p(out), c_int(R), c_int(V), c_ulonglong(seed), c_ulonglong(step),
                                     _stream()), "philox_uniform")
    return out


def flush_l2(device=None):
    ws = Workspace.get(device or torch.cuda.current_device())
    if not hasattr(ws, "flush_buf"):
        ws.flush_buf = torch.empty(256 * 2**20, dtype=torch.uint8, device=ws.device)
    _check(lib().b200_flush_l2(_p(ws.flush_buf), c_size_t(ws.flush_buf.numel()), _stream()), "flush_l2")


# ------------------------------------------------- fused compute + collective (NVLink P2P)
class FusedTP:
    """Heap layout and launch state of the fused row-parallel GEMM + reduction.

    Two receive regions and two output buffers alternate between launches, so a rank that runs one
    launch ahead of a peer never overwrites data the peer still reads."""

    MAX_TILES = 8192

    def __init__(self, heap, max_tokens: int, max_n: int):
        self.heap = heap
        self.max_elems = max_tokens * max_n
        self.one_shot_bytes = envs.B200_TP_ONE_SHOT_BYTES
        self.part_bytes = self.region_bytes(max_tokens, max_n, heap.world, self.one_shot_bytes)
        self.parts = [heap.alloc("tp_part0", self.part_bytes), heap.alloc("tp_part1", self.part_bytes)]
        self.outs = [heap.alloc("tp_out0", self.max_elems * 2), heap.alloc("tp_out1", self.max_elems * 2)]
        self.tile_flags = heap.alloc("tp_tile_flags", heap.world * self.MAX_TILES * 4)
        self.done_flags = heap.alloc("tp_done_flags", self.MAX_TILES * 4)
        # all-gather -> GEMM: two full activation matrices [max_tokens, max_n] and their done flags
        self.xfull = [heap.alloc("tp_xfull0", self.max_elems * 2), heap.alloc("tp_xfull1", self.max_elems * 2)]
        self.ag_done = heap.alloc("tp_ag_done", 2 * heap.world * 4)
        self.ag_flip = 0
        self.ctrl = torch.zeros(4, dtype=torch.int32, device=heap.device)
        self.flip = 0

    def can_push(self, T: int, N: int) -> bool:
        """Shapes small enough for the push plane (every rank receives every partial)."""
        return (envs.B200_TP_DEFER_REDUCE and N % 8 == 0 and N <= 16384
                and T * N * 2 * (self.heap.world - 1) <= self.one_shot_bytes)

    @staticmethod
    def region_bytes(max_tokens: int, max_n: int, world: int, one_shot_bytes: int) -> int:
        # via owners: every tile (padded to 128 x 256) lands in exactly one slab, plus one tile of
        # rounding per (owner, source); one-shot: `world` matrices of at most one_shot_bytes/(world-1)
        owners = (max_tokens + 256) * (max_n + 128) * 2 + world * world * 128 * 256 * 2
        one_shot = world * (one_shot_bytes // max(1, world - 1) + 256)
        return (max(owners, one_shot) + 255) // 256 * 256

    @staticmethod
    def heap_bytes(max_tokens: int, max_n: int, world: int) -> int:
        region = FusedTP.region_bytes(max_tokens, max_n, world, envs.B200_TP_ONE_SHOT_BYTES)
        return (2 * region + 4 * max_tokens * max_n * 2 + world * FusedTP.MAX_TILES * 4 +
                FusedTP.MAX_TILES * 4 + (1 << 20))


def gemm_all_reduce(x, w, heap, mode: int = 0):
    """Row-parallel ``x @ w.T`` summed over the ranks of ``heap`` inside one kernel
    (mode 0: the sum lands on every rank; mode 1: only on the owner of each output tile)."""
    _require_bf16(x, w)
    st = heap.fused_tp
    if x.stride(-1) != 1:
        x = x.contiguous()
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = w.shape[0]
    if T * N > st.max_elems:
        raise RuntimeError(f"fused TP buffers hold {st.max_elems} elements, need {T * N}")
    out, part = st.outs[st.flip], st.parts[st.flip]
    st.flip ^= 1
    ws = Workspace.get(x.device)
    _check(lib().b200_gemm_bf16_fused_reduce(
        _p(x2), _p(w), c_int(T), c_int(N), c_int(K), c_int(x2.stride(0)), c_int(w.stride(0)),
        heap.peers_c, c_int(heap.rank), c_int(heap.world), c_int(mode),
        c_ulonglong(part.offset), c_ulonglong(st.part_bytes), c_ulonglong(st.one_shot_bytes),
        c_ulonglong(out.offset), c_ulonglong(st.tile_flags.offset),
        c_ulonglong(st.done_flags.offset), c_int(FusedTP.MAX_TILES), _p(st.ctrl), _p(ws.gemm_ws),
        c_size_t(ws.gemm_ws.numel()), _p(ws.gemm_counters), c_int(ws.gemm_counters.numel()), _p(ws.status),
        c_int(_sms), ctypes.c_uint(min(heap.spin_limit, 2**31 - 1)), _stream()), "gemm_fused_reduce")
    count_launch()
    return heap.tensor(out, (T, N), torch.bfloat16)


def gemm_all_gather(x_local, w, heap, bias=None):
    """Column-parallel ``gather(x) @ w.T`` where the rows of ``x`` are sharded over the ranks of
    ``heap`` (equal shards, a multiple of 32 rows): the all-gather runs inside the GEMM kernel as
    NVLink pushes that overlap the tensor-core work.  Returns [world * T_loc, N] in local memory."""
    _require_bf16(x_local, w, bias)
    st = heap.fused_tp
    if x_local.stride(-1) != 1:
        x_local = x_local.contiguous()
    T_loc, K = x_local.shape
    N = w.shape[0]
    T = T_loc * heap.world
    if T * K > st.max_elems:
        raise RuntimeError(f"gather buffers hold {st.max_elems} elements, need {T * K}")
    flip = st.ag_flip
    st.ag_flip ^= 1
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x_local.device)
    ws = Workspace.get(x_local.device)
    _check(lib().b200_gemm_bf16_allgather(
        _p(x_local), _p(w), _p(y), _p(bias), c_int(T_loc), c_int(N), c_int(K), c_int(x_local.stride(0)),
        c_int(w.stride(0)), c_int(y.stride(0)), heap.peers_c, c_int(heap.rank), c_int(heap.world),
        c_ulonglong(st.xfull[flip].offset), c_ulonglong(st.xfull[flip].nbytes),
        c_ulonglong(st.tile_flags.offset), c_int(FusedTP.MAX_TILES), c_ulonglong(st.ag_done.offset), c_int(flip),
        _p(st.ctrl), _p(ws.status), c_int(_sms), ctypes.c_uint(min(heap.spin_limit, 2**31 - 1)), _stream()),
        "gemm_all_gather")
    count_launch()
    return y


class PendingReduce:
    """Output of a row-parallel GEMM whose partials have been pushed to every rank but not yet
    summed.  The consumer (``add_rms_norm`` or ``materialize``) sums them from this rank's receive
    region, so the all-reduce costs one NVLink store hop and rides in a kernel that runs anyway."""

    def __init__(self, heap, part, T: int, N: int, lead_shape):
        self.heap, self.part, self.T, self.N = heap, part, T, N
        self.shape = tuple(lead_shape) + (N,)
        self.dtype = torch.bfloat16
        self.device = heap.device
        self.is_cuda = True

    def _run(self, residual, weight, eps):
        st = self.heap.fused_tp
        y = torch.empty((self.T, self.N), dtype=torch.bfloat16, device=self.device)
        ws = Workspace.get(self.device)
        stride = (self.T * self.N * 2 + 255) // 256 * 256
        base = self.heap.local_ptr
        _check(lib().b200_reduce_pushed_rms_norm(
            c_void_p(base + self.part.offset), c_ulonglong(stride), c_void_p(base + st.tile_flags.offset),
            c_int(FusedTP.MAX_TILES), _p(st.ctrl), _p(residual), _p(weight), _p(y), c_int(self.T), c_int(self.N),
            c_int(self.heap.world), c_float(eps), _p(ws.status),
            ctypes.c_uint(min(self.heap.spin_limit, 2**31 - 1)), _stream()), "reduce_pushed_rms_norm")
        count_launch()
        return y.view(self.shape)

    def add_rms_norm(self, residual, weight, eps):
        """(RMSNorm(sum + residual) * weight, residual += sum) like ``fused_add_rms_norm``."""
        _require_bf16(residual, weight)
        assert residual.is_contiguous() and residual.numel() == self.T * self.N
        return self._run(residual, weight, eps), residual

    def materialize(self):
        return self._run(None, None, 0.0)


def gemm_push(x, w, heap):
    """Row-parallel ``x @ w.T`` whose partial is pushed to every rank of ``heap``; returns a
    :class:`PendingReduce`.  For shapes within ``FusedTP.can_push``."""
    _require_bf16(x, w)
    st = heap.fused_tp
    if x.stride(-1) != 1:
        x = x.contiguous()
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = w.shape[0]
    out, part = st.outs[st.flip], st.parts[st.flip]
    st.flip ^= 1
    ws = Workspace.get(x.device)
    _check(lib().b200_gemm_bf16_fused_reduce(
        _p(x2), _p(w), c_int(T), c_int(N), c_int(K), c_int(x2.stride(0)), c_int(w.stride(0)),
        heap.peers_c, c_int(heap.rank), c_int(heap.world), c_int(3),
        c_ulonglong(part.offset), c_ulonglong(st.part_bytes), c_ulonglong(st.one_shot_bytes),
        c_ulonglong(out.offset), c_ulonglong(st.tile_flags.offset),
        c_ulonglong(st.done_flags.offset), c_int(FusedTP.MAX_TILES), _p(st.ctrl), _p(ws.gemm_ws),
        c_size_t(ws.gemm_ws.numel()), _p(ws.gemm_counters), c_int(ws.gemm_counters.numel()), _p(ws.status),
        c_int(_sms), ctypes.c_uint(min(heap.spin_limit, 2**31 - 1)), _stream()), "gemm_push")
    count_launch()
    return PendingReduce(heap, part, T, N, x.shape[:-1])


def p2p_all_reduce(x, heap):
    """All-reduce of a bf16 tensor through a staging buffer in the symmetric heap."""
    _require_bf16(x)
    n = x.numel()
    pad = (-n) % 8
    buf = heap.alloc("ar_stage", heap.ar_stage_bytes)
    if (n + pad) * 2 > buf.nbytes:
        raise RuntimeError("all-reduce staging buffer too small")
    stage = heap.tensor(buf, (n + pad,), torch.bfloat16)
    stage[:n].copy_(x.reshape(-1))
    if pad:
        stage[n:].zero_()
    ws = Workspace.get(x.device)
    _check(lib().b200_p2p_all_reduce(
        heap.peers_c, c_int(heap.rank), c_int(heap.world), c_size_t(buf.offset), c_size_t(heap.flags.offset),
        _p(heap.ctrl), c_size_t(n + pad), _p(ws.status), ctypes.c_uint(min(heap.spin_limit, 2**31 - 1)),
        _stream()), "p2p_all_reduce")
    count_launch()
    x.copy_(stage[:n].view(x.shape))
    return x


# Kernels of the sub-modules under this module's name (``cuda.moe_experts`` ...), resolved on first use: the
# sub-modules import this module, so importing them here would make ``import ops.cuda_fp4`` depend on who came first.
_SUBMODULE_EXPORTS = {
    "cuda_moe": ("EpState", "gemm_swiglu", "group_bias_add", "grouped_gemm", "moe_experts", "moe_experts_ep",
                 "moe_route_post", "moe_permute", "moe_route", "moe_unpermute"),
    "cuda_fp8": ("fp8_block_gemm", "fp8_block_gemm_push", "fp8_block_gemm_push_quantised", "fp8_block_gemm_quantised",
                 "fp8_per_tensor_gemm", "fp8_rowwise_gemm", "grouped_fp8_gemm", "int8_gemm", "moe_experts_ep_fp8",
                 "moe_experts_fp8", "quant_act_1x128", "quant_act_int8", "quant_rows_1x128"),
    "cuda_fp4": ("grouped_w4a16_gemm", "moe_experts_w4a16", "w4a16_gemm", "w4a16_int4_gemm", "dequant_w4", "dequant_int4"),
    "cuda_gdn": ("gdn_forward", "kda_forward", "short_conv"),
    "cuda_mla": ("mla_absorb", "mla_paged_attention", "mla_unabsorb", "mla_write_cache", "permute_rows", "rope_rows"),
}
_EXPORT_HOME = {name: mod for mod, names in _SUBMODULE_EXPORTS.items() for name in names}


def __getattr__(name: str):
    mod = _EXPORT_HOME.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib
    value = getattr(importlib.import_module(f"{__package__}.{mod}"), name)
    globals()[name] = value
    return value
