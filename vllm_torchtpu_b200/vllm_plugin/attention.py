"""Attention backend for vLLM's V1 engine on this package's paged-attention kernels.

Registered under ``AttentionBackendEnum.CUSTOM``.  One ``forward`` writes the step's keys and values
into the request's pages and runs ragged paged attention over the mixed decode / prefill batch, which
is what the reference's backend does in one kernel call
(reference: src/vllm_torchtpu/layers/adapter/attention.py:598-758, 844-1698).  The KV cache layout is
this package's: ``[num_blocks, 2, kv_heads, block_size, head_size]``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional

import torch
from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl,
                                       AttentionMetadataBuilder, AttentionType, CommonAttentionMetadata)

from ..runner.attn_metadata import AttentionMetadata as NativeMeta


@dataclass
class B200AttentionMetadata:
    num_actual_tokens: int
    native: NativeMeta              # what ops.cuda.paged_attention takes


class B200MetadataBuilder(AttentionMetadataBuilder):
    # decode steps (one query per request) can be captured in a full CUDA graph: the launch shapes
    # only depend on the padded request count
    _cudagraph_support: ClassVar[AttentionCGSupport] = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
    reorder_batch_threshold: int = 1            # decodes first, as the kernels expect

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self.block_size = kv_cache_spec.block_size

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> B200AttentionMetadata:
        from vllm.v1.attention.backends.utils import split_decodes_and_prefills
        m = common_attn_metadata
        num_decodes, _, _, _ = split_decodes_and_prefills(m, decode_threshold=1)
        qsl_cpu = m.query_start_loc_cpu
        seq = m.seq_lens if m.seq_lens.dtype == torch.int32 else m.seq_lens.to(torch.int32)
        qsl = m.query_start_loc if m.query_start_loc.dtype == torch.int32 else m.query_start_loc.to(torch.int32)
        bt = m.block_table_tensor
        if bt.dtype != torch.int32 or not bt.is_contiguous():
            bt = bt.to(torch.int32).contiguous()
        native = NativeMeta(
            positions=None, slot_mapping=m.slot_mapping, block_tables=bt, seq_lens=seq, query_start_loc=qsl,
            num_reqs=m.num_reqs, num_tokens=m.num_actual_tokens, num_decode_reqs=int(num_decodes),
            max_query_len=int(m.max_query_len), max_seq_len=int(m.max_seq_len), padded_num_reqs=m.num_reqs,
            padded_num_tokens=m.num_actual_tokens, query_start_loc_cpu=qsl_cpu.long())
        return B200AttentionMetadata(num_actual_tokens=m.num_actual_tokens, native=native)


class B200AttentionImpl(AttentionImpl):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes=None, sliding_window: Optional[int] = None, kv_cache_dtype: str = "auto",
                 logits_soft_cap: Optional[float] = None, attn_type: str = AttentionType.DECODER,
                 kv_sharing_target_layer_name: Optional[str] = None, sinks=None, **kwargs) -> None:
        if alibi_slopes is not None:
            raise NotImplementedError("ALiBi is not supported by the b200 attention backend")
        if attn_type != AttentionType.DECODER:
            raise NotImplementedError("the b200 attention backend covers decoder self-attention")
        if kv_cache_dtype not in ("auto", "bfloat16"):
            raise NotImplementedError("the vLLM plugin path keeps a bf16 KV cache")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.sliding_window = sliding_window[0] if isinstance(sliding_window, (tuple, list)) else sliding_window
        self.logits_soft_cap = logits_soft_cap or None
        self.kv_cache_dtype = kv_cache_dtype
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
        self.sinks = sinks

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                output_block_scale=None):
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation")
        if attn_metadata is None:                       # memory-profiling run
            return output.fill_(0)
        from ..ops import cuda, cuda_misc
        n = attn_metadata.num_actual_tokens
        H, Hkv, D = self.num_heads, self.num_kv_heads, self.head_size
        meta = attn_metadata.native
        q = query[:n].reshape(n, H, D)
        if not q.is_contiguous():
            q = q.contiguous()
        if key is not None and self.kv_sharing_target_layer_name is None:
            k = key[:n].reshape(n, Hkv, D)
            v = value[:n].reshape(n, Hkv, D)
            if k.stride(2) != 1 or k.stride(1) != D:
                k = k.contiguous()
            if v.stride(2) != 1 or v.stride(1) != D:
                v = v.contiguous()
            cuda_misc.kv_write(k, v, kv_cache, meta.slot_mapping)
        out = cuda.paged_attention(q, kv_cache, meta, self.scale, sliding_window=self.sliding_window,
                                   softcap=self.logits_soft_cap, sinks=self.sinks)
        output[:n].view(n, H * D).copy_(out.view(n, H * D))
        return output


class B200AttentionBackend(AttentionBackend):
    accept_output_buffer: bool = True
    forward_includes_kv_cache_update: bool = True
    supported_dtypes: ClassVar[list] = [torch.bfloat16]
    supported_kv_cache_dtypes: ClassVar[list] = ["auto", "bfloat16"]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return B200AttentionImpl

    @staticmethod
    def get_builder_cls():
        return B200MetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes() -> list:
        return [16, 32, 64, 128]

    @classmethod
    def get_supported_head_sizes(cls) -> list:
        return [64, 128]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple:
        return (num_blocks, 2, num_kv_heads, block_size, head_size)

    @classmethod
    def supports_sink(cls) -> bool:
        return True

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return getattr(capability, "major", 10) == 10
