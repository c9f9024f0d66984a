"""Offline inference API: ``LLM(...).generate(prompts, sampling_params)``.

Mirrors the ``vllm.LLM`` surface the reference is used through
(reference: README.md:63-82): token-id or text prompts in, ``RequestOutput``
objects out, in input order.
"""
from __future__ import annotations

from typing import Optional, Sequence, Union

from ..config import (CacheConfig, EngineConfig, ModelConfig, ParallelConfig, SchedulerConfig,
                      model_preset)
from ..outputs import RequestOutput
from ..sampling_params import SamplingParams
from .llm_engine import LLMEngine


POOLING_MODES = ("last", "mean", "max", "cls", "all")     # "all": one vector per prompt token


class LLM:
    def __init__(self, model: Union[str, ModelConfig] = "tiny-llama", *, tokenizer=None,
                 tensor_parallel_size: int = 1, pipeline_parallel_size: int = 1,
                 data_parallel_size: int = 1, enable_expert_parallel: bool = False,
                 prefill_context_parallel_size: int = 1, decode_context_parallel_size: int = 1,
                 cp_kv_cache_interleave_size: int = 1, scheduler_block_size: int = 0,
                 max_model_len: Optional[int] = None, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, block_size: int = 16,
                 gpu_memory_utilization: float = 0.9, num_gpu_blocks_override: Optional[int] = None,
                 enable_prefix_caching: bool = False, enforce_eager: bool = False,
                 kv_cache_dtype: str = "auto", quantization: Optional[str] = None,
                 async_scheduling: bool = False, scheduler_cls: str = "default",
                 device: str = "cuda", dtype=None, seed: int = 0,
                 speculative_config: Optional[dict] = None, kv_transfer_config: Optional[dict] = None,
                 additional_config: Optional[dict] = None, load_format: str = "auto",
                 world_size: Optional[int] = None, init_dist: bool = True):
        import os
        model_path = tokenizer_path = None
        if isinstance(model, ModelConfig):
            mc = model
        elif os.path.isdir(str(model)) or "://" in str(model):
            # a URI: configuration and tokenizer are copied to this host once, weights are read from the source
            from ..models.model_source import resolve_model
            aux_dir, weights = resolve_model(str(model))
            if "://" in str(weights):
                raise ValueError(f"weights of {model} need a streaming reader for their scheme; none is built in")
            mc = ModelConfig.from_pretrained(aux_dir)
            model_path, tokenizer_path = weights, aux_dir
        else:
            mc = model_preset(model)
        if max_model_len:
            mc.max_model_len = max_model_len
        if dtype is not None:
            from ..config import parse_dtype
            mc.dtype = parse_dtype(dtype)
        if quantization:
            mc.quantization = quantization
        mc.seed = seed
        ws = world_size if world_size is not None else int(os.environ.get("WORLD_SIZE", 1))
        pc = ParallelConfig(tensor_parallel_size, data_parallel_size, pipeline_parallel_size,
                            enable_expert_parallel, prefill_context_parallel_size,
                            decode_context_parallel_size, world_size=ws,
                            rank=int(os.environ.get("RANK", 0)),
                            local_rank=int(os.environ.get("LOCAL_RANK", 0)),
                            backend="nccl" if device == "cuda" else "gloo")
        pc.cp_kv_cache_interleave_size = cp_kv_cache_interleave_size
        cfg = EngineConfig(
            model=mc, parallel=pc,
            cache=CacheConfig(block_size, gpu_memory_utilization, num_gpu_blocks_override, None,
                              enable_prefix_caching, kv_cache_dtype,
                              block_size * decode_context_parallel_size if decode_context_parallel_size > 1
                              else scheduler_block_size, scheduler_block_size),
            scheduler=SchedulerConfig(max_num_seqs, max_num_batched_tokens, True, scheduler_cls,
                                      async_scheduling),
            device=device, enforce_eager=enforce_eager,
            load_format="dummy" if (load_format == "auto" and model_path is None) else
            ("safetensors" if load_format == "auto" else load_format),
            model_path=model_path, speculative=speculative_config, kv_transfer=kv_transfer_config,
            additional=additional_config or {})
        self.engine = LLMEngine(cfg, init_dist=init_dist)
        self.tokenizer = tokenizer
        if tokenizer is None and model_path:
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_path or model_path)
            except Exception:
                self.tokenizer = None
        if self.tokenizer is not None and getattr(self.tokenizer, "eos_token_id", None) is not None:
            self.engine.eos_token_id = self.tokenizer.eos_token_id

    def _decode(self, ids) -> str:
        try:
            return self.tokenizer.decode(ids, skip_special_tokens=True)
        except TypeError:                                # tokenizers without the flag
            return self.tokenizer.decode(ids)

    def _encode(self, prompt) -> list:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer")
            return self.tokenizer.encode(prompt)
        if isinstance(prompt, dict):
            return list(prompt["prompt_token_ids"])
        return list(prompt)

    def chat(self, messages, sampling_params: Union[SamplingParams, Sequence, None] = None, *,
             add_generation_prompt: bool = True, continue_final_message: bool = False,
             chat_template_kwargs: Optional[dict] = None, tools: Optional[list] = None) -> list:
        """One conversation (a list of {role, content} messages) or a list of conversations -> ``RequestOutput``
        objects, through the tokenizer's chat template (``tools`` are handed to the template)."""
        from ..entrypoints.chat_template import build_chat_prompt
        convs = messages if messages and isinstance(messages[0], list) else [messages]
        kw = dict(chat_template_kwargs or {})
        if tools:
            kw.setdefault("tools", tools)
        prompts = [build_chat_prompt(self.tokenizer, self._encode, list(c), add_generation_prompt=add_generation_prompt,
                                     continue_final_message=continue_final_message, chat_template_kwargs=kw or None)
                   for c in convs]
        return self.generate(prompts, sampling_params)

    def embed(self, prompts: Sequence, pooling: str = "last", normalize: bool = True) -> list:
        """Pooled final hidden state per prompt (``last`` token or ``mean`` over the prompt), optionally
        L2-normalised: the embedding-model path (reference: src/vllm_torchtpu/runner/tpu_pooling.py)."""
        if pooling not in POOLING_MODES:
            raise ValueError(f"pooling must be one of {POOLING_MODES}")
        sp = SamplingParams(temperature=0.0, max_tokens=1, pooling=pooling)
        outs = self.generate(prompts, sp)
        vecs = []
        for o in outs:
            v = o.pooled
            if normalize and v is not None:
                n = sum(a * a for a in v) ** 0.5 or 1.0
                v = [a / n for a in v]
            vecs.append(v)
        return vecs

    def generate(self, prompts: Sequence, sampling_params: Union[SamplingParams, Sequence, None] = None,
                 priority: Optional[Sequence] = None) -> list:
        """One ``RequestOutput`` per prompt, in input order, with ``sampling_params.n`` completions each.
        Stop strings are matched on the detokenised text while the requests run; a request that produced one
        is ended there and its text is cut in front of the string."""
        from ..entrypoints.stop_strings import StopStringMatcher, truncate_at_stop
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else \
            [sampling_params or SamplingParams()] * len(prompts)
        groups, watch = [], {}
        prios = list(priority) if priority is not None else [0] * len(prompts)
        for k, (p, sp) in enumerate(zip(prompts, sps)):
            sp = sp or SamplingParams()
            sp.verify()
            if sp.stop and self.tokenizer is None:
                raise ValueError("stop strings need a tokenizer")
            ids = self._encode(p)
            group = [self.engine.add_request(ids, sp, priority=prios[k]) for _ in range(sp.n)]
            groups.append((group, sp))
            if sp.stop:
                for rid in group:
                    watch[rid] = [StopStringMatcher(sp.stop, sp.include_stop_str_in_output), 0]
        reqs = self.engine.scheduler.requests
        if watch:
            while self.engine.has_unfinished():
                self.engine.step()
                for rid in list(watch):
                    req = reqs.get(rid)
                    if req is None or req.status.finished:
                        del watch[rid]
                        continue
                    m, seen = watch[rid]
                    if len(req.output_token_ids) == seen:
                        continue
                    watch[rid][1] = len(req.output_token_ids)
                    if m.push(self._decode(req.output_token_ids))[1]:
                        self.engine.abort_request(rid)
                        del watch[rid]
        else:
            self.engine.run_until_done()
        detok = self._decode if self.tokenizer is not None else None
        outs = []
        for group, sp in groups:
            out = None
            for i, rid in enumerate(group):
                o = RequestOutput.from_request(reqs.pop(rid), detok)
                c = o.outputs[0]
                c.index = i
                if sp.stop and c.text is not None:
                    c.text, hit = truncate_at_stop(c.text, sp.stop, sp.include_stop_str_in_output)
                    if hit is not None:
                        c.finish_reason, c.stop_reason = "stop", hit
                if out is None:
                    out = o
                else:
                    out.outputs.append(c)
                    out.finished = out.finished and o.finished
            outs.append(out)
        return outs
