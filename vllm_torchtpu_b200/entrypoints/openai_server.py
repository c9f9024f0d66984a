"""OpenAI-compatible HTTP server.

Routes: ``/v1/completions`` (one or several prompts), ``/v1/chat/completions`` (function calling through
``tools`` / ``tool_choice``), both with SSE streaming, ``/v1/embeddings``, ``/v1/models``, ``/tokenize``,
``/detokenize``, ``/version``, ``/health``, ``/ping``, ``/metrics`` (Prometheus text), LoRA load / unload,
``/update_weights``, ``/reload_kernel``, ``/start_profile`` and ``/stop_profile``.  ``kv_transfer_params`` is accepted in requests and returned in
responses so the disaggregation proxy can chain a prefill and a decode instance
(reference surface: README.md:63-82, docs/user_guide/disaggregated_serving.md:98-108).

Prompts may be text (needs a tokenizer) or token-id lists; a model without a tokenizer
answers with token ids rendered as text.
"""
import json
import os
import time
import uuid
from typing import Optional

from ..sampling_params import SamplingParams
from .async_engine import AsyncEngine


def _structured_spec(body: dict):
    """``structured_outputs`` / ``guided`` pass through; ``guided_json`` / ``guided_regex`` / ``guided_choice`` and
    the OpenAI ``response_format`` (``json_schema`` / ``json_object``) are mapped onto the same spec."""
    spec = body.get("structured_outputs") or body.get("guided")
    if spec:
        return spec
    if body.get("guided_json") is not None:
        return {"json": body["guided_json"]}
    if body.get("guided_regex"):
        return {"regex": body["guided_regex"]}
    if body.get("guided_choice"):
        import re as _re
        return {"regex": "(" + "|".join(_re.escape(str(c)) for c in body["guided_choice"]) + ")"}
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return {"json": js.get("schema", js)}
    if rf.get("type") == "json_object":
        return {"json_object": True}
    return None


def _logprobs_from_body(body: dict):
    """Completions: ``logprobs`` = number of alternatives.  Chat: ``logprobs`` is a flag and
    ``top_logprobs`` the number."""
    lp = body.get("logprobs")
    if isinstance(lp, bool):
        return int(body.get("top_logprobs") or 0) if lp else None
    return lp


def _logprobs_payload(token_ids: list, entries: list, decode) -> dict:
    return {"tokens": [decode([t]) for t in token_ids], "token_ids": list(token_ids),
            "token_logprobs": [e["logprob"] for e in entries],
            "top_logprobs": [{str(i): v for i, v in e["top"]} for e in entries]}


def _sampling_from_body(body: dict) -> SamplingParams:
    return SamplingParams(
        temperature=float(body.get("temperature", 1.0) if body.get("temperature") is not None else 1.0),
        top_k=int(body.get("top_k", 0) or 0), top_p=float(body.get("top_p", 1.0) or 1.0),
        max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 16),
        min_tokens=int(body.get("min_tokens", 0) or 0), ignore_eos=bool(body.get("ignore_eos", False)),
        stop_token_ids=list(body.get("stop_token_ids") or []), logprobs=_logprobs_from_body(body),
        prompt_logprobs=body.get("prompt_logprobs"), lora_name=body.get("lora_name"),
        seed=body.get("seed"), structured=_structured_spec(body),
        n=int(body.get("n") or 1), stop=_stop_from_body(body),
        include_stop_str_in_output=bool(body.get("include_stop_str_in_output", False)),
        min_p=float(body.get("min_p") or 0.0), presence_penalty=float(body.get("presence_penalty") or 0.0),
        frequency_penalty=float(body.get("frequency_penalty") or 0.0),
        repetition_penalty=float(body.get("repetition_penalty") or 1.0),
        logit_bias=body.get("logit_bias") or None, allowed_token_ids=body.get("allowed_token_ids") or None)


def _template_kwargs(body: dict):
    """Extra keyword arguments of the chat template; ``tools`` reach the template this way."""
    kw = dict(body.get("chat_template_kwargs") or {})
    if body.get("tools") and body.get("tool_choice") != "none":
        kw.setdefault("tools", body["tools"])
    return kw or None


def _stop_from_body(body: dict) -> list:
    stop = body.get("stop")
    if stop is None:
        return []
    return [stop] if isinstance(stop, str) else list(stop)


def build_app(engine, model_name: str, tokenizer=None):
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI(title="b200 serving")
    aeng = AsyncEngine(engine)
    app.state.async_engine = aeng
    profiler = {"active": None}

    def encode(prompt) -> list:
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return prompt
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], list):
            return prompt[0]
        if tokenizer is None:
            raise HTTPException(400, "this model has no tokenizer: send token ids")
        return tokenizer.encode(prompt if isinstance(prompt, str) else prompt[0])

    def decode(ids: list) -> str:
        if tokenizer is None:
            return " ".join(str(i) for i in ids)
        try:
            return tokenizer.decode(ids, skip_special_tokens=True)
        except TypeError:
            return tokenizer.decode(ids)

    def visible(ids: list, finish, sp) -> list:
        """The token ids whose text is shown: the end-of-sequence or stop token that ended a completion is
        reported in ``token_ids`` but is not part of the text."""
        if finish == "stop" and ids and not sp.include_stop_str_in_output and \
                (ids[-1] in sp.stop_token_ids or ids[-1] == engine.eos_token_id):
            return ids[:-1]
        return ids

    def chat_prompt(body: dict) -> list:
        from .chat_template import build_chat_prompt
        try:
            return build_chat_prompt(tokenizer, encode, body.get("messages", []),
                                     add_generation_prompt=body.get("add_generation_prompt", True),
                                     continue_final_message=bool(body.get("continue_final_message", False)),
                                     chat_template_kwargs=_template_kwargs(body))
        except ValueError as e:
            raise HTTPException(400, str(e))

    async def run(body: dict, prompt_ids: list, chat: bool):
        tools, tool_choice = [], None
        try:
            if chat:
                from .tool_calls import structured_spec_for, validate_tools
                tools, tool_choice = validate_tools(body)
                forced = structured_spec_for(tools, tool_choice)
                if forced is not None:
                    body = dict(body, structured_outputs=forced)
            sp = _sampling_from_body(body)
            sp.verify()
            from ..platform import B200Platform
            B200Platform.validate_request(sp)
        except ValueError as e:
            raise HTTPException(400, str(e))
        if sp.structured and tokenizer is not None and getattr(engine, "vocab_strings", None) is None:
            # the grammar matcher needs the text of every token; built on the first structured request
            from ..structured import vocab_strings_of
            engine.vocab_strings = vocab_strings_of(tokenizer, engine.cfg.model.vocab_size)
        rid = f"{'chatcmpl' if chat else 'cmpl'}-{uuid.uuid4().hex}"
        created = int(time.time())
        kvp = body.get("kv_transfer_params")
        mm = None
        if body.get("mm_items"):
            # [{"patches": [[...], ...], "offset": first placeholder token}, ...]; the engine needs a
            # vision encoder (LLMEngine.enable_vision) for these
            import torch
            try:
                mm = [(torch.tensor(it["patches"], dtype=torch.float32), int(it["offset"])) for it in body["mm_items"]]
            except (KeyError, TypeError, ValueError) as e:
                raise HTTPException(400, f"bad mm_items: {e}")
        obj = "chat.completion" if chat else "text_completion"

        def chunk_payload(text, finish, final_item=None, index=0):
            choice = {"index": index, "finish_reason": finish}
            if chat:
                choice["delta" if body.get("stream") else "message"] = {"role": "assistant", "content": text}
            else:
                choice["text"] = text
            out = {"id": rid, "object": obj + (".chunk" if chat and body.get("stream") else ""),
                   "created": created, "model": model_name, "choices": [choice]}
            if final_item is not None:
                out["usage"] = {"prompt_tokens": final_item.num_prompt_tokens,
                                "completion_tokens": final_item_tokens[0],
                                "total_tokens": final_item.num_prompt_tokens + final_item_tokens[0],
                                "prompt_tokens_details": {"cached_tokens": final_item.num_cached_tokens}}
                if final_item.kv_transfer_params:
                    out["kv_transfer_params"] = final_item.kv_transfer_params
            return out

        final_item_tokens = [0]
        n = sp.n
        if sp.stop and tokenizer is None:
            raise HTTPException(400, "stop strings need a tokenizer: send stop_token_ids")

        async def events(i):
            """Completion i as (index, text that may be shown, new token ids, logprobs, finish reason, item,
            ended).  With stop strings the text lags the tokens by what could still become a stop string."""
            from .stop_strings import StopStringMatcher
            m = StopStringMatcher(sp.stop, sp.include_stop_str_in_output) if sp.stop else None
            gen = aeng.generate(rid if n == 1 else f"{rid}-{i}", prompt_ids, sp, kvp, mm,
                                priority=int(body.get("priority") or 0))
            toks = []
            try:
                async for item in gen:
                    toks += item.new_token_ids
                    if item.error or m is None:
                        yield i, decode(visible(item.new_token_ids, item.finish_reason, sp)), item.new_token_ids, \
                            item.logprobs, item.finish_reason, item, item.finished
                        continue
                    text, hit = m.push(decode(visible(toks, item.finish_reason, sp)), final=item.finished)
                    yield i, text, item.new_token_ids, item.logprobs, \
                        ("stop" if hit else item.finish_reason), item, (hit or item.finished)
                    if hit:
                        return          # closing the generator aborts the request
            finally:
                await gen.aclose()

        async def merged():
            if n == 1:
                async for ev in events(0):
                    yield ev
                return
            import asyncio
            q: asyncio.Queue = asyncio.Queue()

            async def pump(i):
                try:
                    async for ev in events(i):
                        await q.put(ev)
                finally:
                    await q.put(None)
            tasks = [asyncio.create_task(pump(i)) for i in range(n)]
            left = n
            try:
                while left:
                    ev = await q.get()
                    if ev is None:
                        left -= 1
                    else:
                        yield ev
            finally:
                for t in tasks:
                    t.cancel()

        if body.get("stream"):
            seen_text: dict = {}

            async def sse():
                left = n
                async for i, text, new_ids, lps_i, finish, item, ended in merged():
                    final_item_tokens[0] += len(new_ids)
                    if item.error:
                        yield f"data: {json.dumps({'error': item.error})}\n\n"
                        break
                    left -= bool(ended)
                    payload = chunk_payload(text, finish, item if ended and not left else None, index=i)
                    if lps_i:
                        payload["choices"][0]["logprobs"] = _logprobs_payload(new_ids, lps_i, decode)
                    if tools:
                        # the text streams as it comes; calls found in a finished completion follow as one delta
                        seen_text[i] = seen_text.get(i, "") + text
                        if ended:
                            from .tool_calls import extract_tool_calls
                            _, calls = extract_tool_calls(seen_text[i], tools, tool_choice)
                            if calls:
                                ch = payload["choices"][0]
                                ch["delta"]["tool_calls"] = [dict(c, index=j) for j, c in enumerate(calls)]
                                ch["finish_reason"] = "tool_calls"
                    yield f"data: {json.dumps(payload)}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        acc = [{"text": [], "toks": [], "lps": [], "finish": None, "last": None} for _ in range(n)]
        async for i, text, new_ids, lps_i, finish, item, ended in merged():
            c = acc[i]
            c["text"].append(text)
            c["toks"] += new_ids
            c["lps"] += lps_i or []
            c["finish"], c["last"] = finish, item
            if item.error:
                raise HTTPException(500, item.error)
        final_item_tokens[0] = sum(len(c["toks"]) for c in acc)
        payload = None
        for i, c in enumerate(acc):
            toks, last = c["toks"], c["last"]
            text = "".join(c["text"]) if sp.stop else decode(visible(toks, c["finish"], sp))
            one = chunk_payload(text, c["finish"], last if i == n - 1 else None, index=i)
            ch = one["choices"][0]
            if tools:
                from .tool_calls import extract_tool_calls
                content, calls = extract_tool_calls(text, tools, tool_choice)
                if calls:
                    ch["message"]["content"], ch["message"]["tool_calls"] = content, calls
                    ch["finish_reason"] = "tool_calls"
            ch["token_ids"] = toks
            if c["lps"]:
                ch["logprobs"] = _logprobs_payload(toks, c["lps"], decode)
            if last is not None and last.prompt_logprobs:
                ch["prompt_logprobs"] = [
                    None if e is None else {"token_id": e["token_id"], "logprob": e["logprob"], "rank": e["rank"]}
                    for e in last.prompt_logprobs]
            if payload is None:
                payload = one
            else:
                payload["choices"].append(ch)
                for k in ("usage", "kv_transfer_params"):
                    if k in one:
                        payload[k] = one[k]
        return JSONResponse(payload)

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt", "")
        batch = isinstance(prompt, list) and len(prompt) > 1 and not isinstance(prompt[0], int)
        if not batch:
            return await run(body, encode(prompt), chat=False)
        # several prompts in one request: they run concurrently and come back as choices in prompt order
        if body.get("stream"):
            raise HTTPException(400, "streaming takes one prompt per request")
        import asyncio
        parts = await asyncio.gather(*[run(body, encode(p), chat=False) for p in prompt])
        merged = None
        for k, resp in enumerate(parts):
            one = json.loads(resp.body)
            for ch in one["choices"]:
                ch["index"] += k * int(body.get("n") or 1)
            if merged is None:
                merged = one
            else:
                merged["choices"] += one["choices"]
                for key in ("prompt_tokens", "completion_tokens", "total_tokens"):
                    merged["usage"][key] += one["usage"][key]
        return JSONResponse(merged)

    @app.post("/tokenize")
    async def tokenize(request: Request):
        body = await request.json()
        ids = chat_prompt(body) if body.get("messages") is not None else encode(body.get("prompt", ""))
        return {"tokens": ids, "count": len(ids), "max_model_len": engine.cfg.model.max_model_len}

    @app.post("/detokenize")
    async def detokenize(request: Request):
        body = await request.json()
        toks = body.get("tokens")
        if not isinstance(toks, list) or any(not isinstance(t, int) for t in toks):
            raise HTTPException(400, "tokens must be a list of token ids")
        return {"prompt": decode(toks)}

    @app.get("/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    @app.get("/ping")
    @app.post("/ping")
    async def ping():
        return {"status": "ok"}

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await request.json()
        return await run(body, chat_prompt(body), chat=True)

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        """``input``: one prompt or a list (token-id lists, or text with a tokenizer); ``pooling``: last | mean."""
        body = await request.json()
        inp = body.get("input")
        if inp is None:
            raise HTTPException(400, "missing input")
        many = isinstance(inp, list) and inp and not isinstance(inp[0], int)
        prompts = inp if many else [inp]
        pooling = body.get("pooling", "last")
        if pooling not in ("last", "mean", "max", "cls"):
            raise HTTPException(400, "pooling must be 'last', 'mean', 'max' or 'cls'")
        data, used = [], 0
        for i, pr in enumerate(prompts):
            ids = encode(pr)
            sp = SamplingParams(temperature=0.0, max_tokens=1, pooling=pooling)
            rid = f"embd-{uuid.uuid4().hex}"
            last = None
            async for item in aeng.generate(rid, ids, sp, None):
                last = item
            if last is None or last.error or last.pooled is None:
                raise HTTPException(500, (last.error if last else None) or "no embedding produced")
            vec = last.pooled
            if body.get("normalize", True):
                n = sum(a * a for a in vec) ** 0.5 or 1.0
                vec = [a / n for a in vec]
            data.append({"object": "embedding", "index": i, "embedding": vec})
            used += len(ids)
        return JSONResponse({"object": "list", "model": model_name, "data": data,
                             "usage": {"prompt_tokens": used, "total_tokens": used}})

    @app.post("/v1/load_lora_adapter")
    async def load_lora(request: Request):
        """``lora_name`` + ``lora_path`` (a safetensors file of ``<layer>.lora_A.weight`` / ``lora_B.weight``
        pairs), with ``rank`` and ``alpha``."""
        body = await request.json()
        try:
            from safetensors.torch import load_file
            tensors = load_file(body["lora_path"])
            weights = {}
            for k, a in tensors.items():
                if k.endswith(".lora_A.weight"):
                    base = k[: -len(".lora_A.weight")]
                    weights[base] = (a, tensors[base + ".lora_B.weight"])
            rank = int(body.get("rank") or next(iter(weights.values()))[0].shape[0])
            ok = await aeng.call(lambda eng: eng.add_lora(body["lora_name"], rank, float(body.get("alpha", rank)),
                                                        weights))
        except (KeyError, OSError, StopIteration, ValueError) as e:
            raise HTTPException(400, f"cannot load adapter: {e}")
        return JSONResponse({"loaded": bool(ok), "lora_name": body["lora_name"]})

    @app.post("/v1/unload_lora_adapter")
    async def unload_lora(request: Request):
        body = await request.json()
        ok = await aeng.call(lambda eng: eng.remove_lora(body.get("lora_name", "")))
        return JSONResponse({"unloaded": bool(ok)})

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "b200",
                                            "max_model_len": engine.cfg.model.max_model_len}]}

    @app.get("/health")
    @app.get("/healthcheck")
    async def health():
        return {"status": "ok"}

    @app.get("/metrics")
    async def metrics():
        m = aeng.metrics
        aeng.serving_metrics.model_name = model_name
        text = aeng.serving_metrics.render(m, engine)
        if m["ttft_n"]:
            text += f"b200_time_to_first_token_seconds_mean {m['ttft_sum'] / m['ttft_n']:.6f}\n"
        return PlainTextResponse(text)

    @app.post("/reload_kernel")
    async def reload_kernel(request: Request):
        """Development aid: load the kernel library again (after a rebuild, or from ``path``) and re-capture the
        decode graphs without restarting the server; the engine must be idle
        (reference: src/vllm_torchtpu/platforms/tpu_platform.py:269 /reload_kernel)."""
        body = await request.json() if await request.body() else {}
        try:
            loaded = await aeng.call(lambda eng: eng.reload_kernels(body.get("path")))
        except RuntimeError as e:
            raise HTTPException(409, str(e))
        return {"status": "reloaded", "library": loaded}

    @app.post("/update_weights")
    async def update_weights(request: Request):
        """Load checkpoint-named tensors from safetensors files on the server's disk into the running model
        (``{"path": file-or-directory}``); cached prefixes are dropped; the engine must be idle."""
        body = await request.json()
        path = body.get("path")
        if not path or not os.path.exists(path):
            raise HTTPException(400, "path to a safetensors file or directory is required")

        def load(eng):
            from ..models.loader import iter_safetensors
            return eng.update_weights(list(iter_safetensors(path)))
        try:
            n = await aeng.call(load)
        except RuntimeError as e:
            raise HTTPException(409, str(e))
        except (ValueError, OSError) as e:
            raise HTTPException(400, str(e))
        return {"status": "updated", "tensors": int(n)}

    @app.post("/start_profile")
    async def start_profile(request: Request):
        from ..tracing.profiler import start_profile as sp
        body = await request.json() if await request.body() else {}
        profiler["active"] = sp(body.get("prefix", ""))
        return {"status": "started", "dir": profiler["active"].out_dir}

    @app.post("/stop_profile")
    async def stop_profile():
        if profiler["active"] is None:
            raise HTTPException(400, "no profile is running")
        path = profiler["active"].stop()
        profiler["active"] = None
        return {"status": "stopped", "trace": path}

    return app


def serve(engine, model_name: str, tokenizer=None, host: str = "0.0.0.0", port: int = 8000):
    import uvicorn
    uvicorn.run(build_app(engine, model_name, tokenizer), host=host, port=port, log_level="warning")
