"""Binding of the persistent decode kernel (``csrc/decode_mega.cu``): all decoder layers of a dense
model for one decode step in one cooperative launch.

``DecodeMega.build`` checks that a model qualifies (dense Llama-family layers, bf16 weights and KV
cache, head_dim 128, plain causal attention) and prepares the per-layer descriptors (TMA tensor maps
of the four weight matrices, norm weights, KV cache) and the scratch the kernel owns.  ``run`` takes
the embedding rows of a decode-only step of at most 64 requests and returns the residual stream after
the last layer; the caller applies the final norm.  Same role as the reference's decode-fused layers
and megakernel adapter (reference: src/vllm_torchtpu/layers/adapter/fused_moe_decode.py,
megakernel/adapter/plugin.py:52)."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p
from typing import Optional

import torch

from .. import envs
from . import count_launch
from .cuda import Workspace, _check, _p, _stream, lib

HEAD_DIM = 128


def max_tokens() -> int:
    return int(lib().b200_mega_max_tokens())


class DecodeMega:
    def __init__(self):
        self.ready = False

    # ------------------------------------------------------------------ eligibility
    @staticmethod
    def why_not(model, kv_caches, heap=None) -> Optional[str]:
        """None when the model can run on the persistent decode kernel, else the reason."""
        from ..models.llama import LlamaDecoderLayer, LlamaMLP
        from ..parallel.state import get_state
        from ..quantization.unquantized import UnquantizedLinearMethod
        cfg = model.cfg
        st = get_state()
        if not envs.B200_DECODE_MEGAKERNEL:
            return "disabled by B200_DECODE_MEGAKERNEL=0"
        if cfg.dtype != torch.bfloat16 or cfg.head_dim != HEAD_DIM:
            return "needs bf16 weights and head_dim 128"
        if st.pp.size > 1 or st.dcp.size > 1 or st.pcp.size > 1:
            return "pipeline / context parallel layouts use the per-layer kernels"
        if st.tp.size > 1 and (heap is None or st.tp.size > 8):
            return "tensor parallel without a peer heap"
        if cfg.sliding_window or cfg.logit_softcap:
            return "sliding window / soft-cap attention"
        if not model.layers or not kv_caches or len(kv_caches) != len(model.layers):
            return "no layers or KV caches"
        for layer, kv in zip(model.layers, kv_caches):
            if type(layer).forward is not LlamaDecoderLayer.forward or not isinstance(layer.mlp, LlamaMLP):
                return "a layer is not a dense attention + SwiGLU block"
            a = layer.self_attn
            for lin in (a.qkv, a.o, layer.mlp.gate_up, layer.mlp.down):
                if not isinstance(lin.method, UnquantizedLinearMethod) or lin.lora_targets:
                    return "quantised or LoRA-wired projections"
                if lin.weight is None or lin.weight.dtype != torch.bfloat16 or not lin.weight.is_contiguous():
                    return "weights are not contiguous bf16"
            if a.o.bias is not None or layer.mlp.gate_up.bias is not None or layer.mlp.down.bias is not None:
                return "biases outside the qkv projection"
            if a.attn.sinks is not None or a.attn.k_scale != 1.0 or a.attn.v_scale != 1.0:
                return "attention sinks / scaled KV"
            if not torch.is_tensor(kv) or kv.dtype != torch.bfloat16 or kv.dim() != 5:
                return "KV cache is not a bf16 paged cache"
            if a.attn.inv_freq.numel() * 2 != HEAD_DIM:
                return "partial rotary embedding"
        a0 = model.layers[0].self_attn.attn
        I = model.layers[0].mlp.gate_up.weight.shape[0] // 2
        if cfg.hidden_size % 128 or I % 128 or cfg.hidden_size > 8192:
            return "hidden / intermediate size not a multiple of 128 (or hidden > 8192)"
        if a0.num_q_heads % a0.num_kv_heads or a0.num_q_heads // a0.num_kv_heads > 16:
            return "GQA group larger than 16"
        return None

    # ------------------------------------------------------------------ set-up
    @classmethod
    def build(cls, model, kv_caches, device, heap=None) -> "DecodeMega":
        self = cls()
        L = lib()
        L.b200_mega_partial_bytes.restype = c_size_t
        cfg = model.cfg
        a0 = model.layers[0].self_attn.attn
        self.H = cfg.hidden_size
        self.Hq, self.Hkv = a0.num_q_heads, a0.num_kv_heads
        self.I = model.layers[0].mlp.gate_up.weight.shape[0] // 2
        self.num_layers = len(model.layers)
        self.eps = float(cfg.rms_norm_eps)
        self.scale = float(a0.scale)
        self.inv_freq = a0.inv_freq.to(device=device, dtype=torch.float32).contiguous()
        self.interleaved = 1 if a0.rope_interleaved else 0
        self.device = device
        self.heap = heap
        self.world = heap.world if heap is not None else 1
        self.rank = heap.rank if heap is not None else 0
        self.maxt = max_tokens()
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count
        nbytes = int(L.b200_mega_layer_desc_bytes())
        host = (ctypes.c_ubyte * (nbytes * self.num_layers))()
        self._keep = []
        for i, (layer, kv) in enumerate(zip(model.layers, kv_caches)):
            a = layer.self_attn
            wq, wo, wg, wd = a.qkv.weight, a.o.weight, layer.mlp.gate_up.weight, layer.mlp.down.weight
            self._keep += [wq, wo, wg, wd, kv, layer.input_ln, layer.post_ln]
            _check(L.b200_mega_fill_layer(
                ctypes.byref(host, i * nbytes), _p(wq), c_int(wq.shape[0]), c_int(wq.stride(0)),
                _p(wo), c_int(wo.shape[1]), c_int(wo.stride(0)), _p(wg), c_int(wg.shape[0]), c_int(wg.stride(0)),
                _p(wd), c_int(wd.shape[1]), c_int(wd.stride(0)), c_int(self.H), _p(layer.input_ln),
                _p(layer.post_ln), _p(a.qkv.bias), _p(a.q_norm_w), _p(a.k_norm_w), _p(kv)), "mega_fill_layer")
        self.layers_dev = torch.frombuffer(bytearray(host), dtype=torch.uint8).to(device)
        self.kv_shape = tuple(kv_caches[0].shape)
        T = self.maxt
        z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=device)
        self.h, self.o, self.act = z(T, self.H), z(T, self.Hq * HEAD_DIM), z(T, self.I)
        self.residual = z(T, self.H)
        self.zero_hidden = z(T, self.H)
        self.part_bytes = int(L.b200_mega_partial_bytes(c_int(self.H), c_int(self.Hq), c_int(self.Hkv), c_int(self.I),
                                                        c_int(self.sms)))
        self.part = torch.empty(self.part_bytes, dtype=torch.uint8, device=device)
        self.max_splits = 8
        units = T * self.Hkv * self.max_splits
        self.attn_part_o = torch.empty(units * 16 * HEAD_DIM, dtype=torch.float32, device=device)
        self.attn_part_ml = torch.empty(units * 16 * 2, dtype=torch.float32, device=device)
        self.attn_counters = torch.zeros(T * self.Hkv, dtype=torch.int32, device=device)
        self.ctrl = torch.zeros(64, dtype=torch.int32, device=device)
        self.dbg = None                  # int64 tensor [rows, CTAs]: phase end times (kernel header: Params::dbg)
        self.dbg_event = (-1, -1, 0)     # (layer, projection, first row) of the role events of one GEMM phase
        self.slab = [0, 0]
        self.flag = [0, 0]
        if heap is not None:
            for i in range(2):
                self.slab[i] = heap.alloc(f"mega_slab{i}", self.world * T * self.H * 2).offset
                fb = heap.alloc(f"mega_flags{i}", self.world * T * 4 * 4)
                fb.tensor.zero_()
                self.flag[i] = fb.offset
            torch.cuda.synchronize()
        self.ready = True
        return self

    def kv_splits(self, T: int, ctx_hint: int = 1024) -> int:
        """KV splits per (request, kv head).  A (request, kv head, split) unit is one warp's work and an
        SM runs four of them at a time: few long units leave warps idle, many short ones pay the fixed
        prologue and merge per unit."""
        if envs.B200_ATTN_SPLIT_KV > 0:
            return min(self.max_splits, envs.B200_ATTN_SPLIT_KV)
        pairs = max(1, T * self.Hkv)
        slots = 4 * self.sms
        chunks = max(1, ctx_hint // 16)
        best, best_cost = 1, None
        for s in (1, 2, 4, 8):
            rounds = -(-pairs * s // slots)
            cost = rounds * (chunks / s + 6.0)       # chunk times: streaming + prologue / merge per unit
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = s, cost
        return best

    # ------------------------------------------------------------------ launch
    def run(self, hidden0: torch.Tensor, meta, T: int):
        """hidden0 [T, H] bf16 -> (zeros [T, H], residual [T, H]) so that the caller's
        ``norm(hidden + residual)`` is the final norm of the residual stream."""
        assert self.ready and T <= self.maxt and hidden0.is_contiguous()
        for t in (meta.positions, meta.slot_mapping, meta.block_tables, meta.seq_lens):
            if t.dtype != torch.int32 or not t.is_contiguous():
                raise TypeError("decode step metadata must be contiguous int32 tensors")
        nb, _, _, bs, _ = self.kv_shape
        ws = Workspace.get(self.device)
        heap = self.heap
        peers = heap.peers_c if heap is not None else None
        spin = min(heap.spin_limit, 2**31 - 1) if heap is not None else 0
        _check(lib().b200_mega_decode(
            _p(self.layers_dev), c_int(self.num_layers), _p(hidden0), _p(self.residual), _p(self.h), _p(self.o),
            _p(self.act), _p(self.part), c_size_t(self.part_bytes), _p(meta.positions), _p(meta.slot_mapping),
            _p(meta.block_tables), _p(meta.seq_lens), c_int(meta.block_tables.shape[1]), c_int(bs), c_longlong(nb),
            c_int(T), c_int(self.H), c_int(self.Hq), c_int(self.Hkv), c_int(self.I), _p(self.inv_freq),
            c_int(self.inv_freq.numel()), c_int(self.interleaved), c_float(self.eps), c_float(self.scale),
            c_int(self.kv_splits(T)), _p(self.attn_part_o), _p(self.attn_part_ml), _p(self.attn_counters),
            _p(self.ctrl), _p(ws.status), c_int(self.world), c_int(self.rank), peers,
            c_ulonglong(self.slab[0]), c_ulonglong(self.slab[1]), c_ulonglong(self.flag[0]),
            c_ulonglong(self.flag[1]), ctypes.c_uint(spin), c_int(self.sms), _p(self.dbg),
            c_int(self.dbg_event[0]), c_int(self.dbg_event[1]), c_int(self.dbg_event[2]), _stream()), "mega_decode")
        count_launch()
        return self.zero_hidden[:T], self.residual[:T]

    def reset(self) -> None:
        """After a launch that reported a device status: re-arm the barrier words and counters."""
        self.ctrl[:2].zero_()
        self.ctrl[3:].zero_()          # keeps ctrl[2], the launch epoch the peers share
        self.attn_counters.zero_()
