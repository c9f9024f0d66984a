"""Prefill/decode disaggregation proxy.

For every ``/v1/completions`` or ``/v1/chat/completions`` request: send it to a prefill instance
with ``max_tokens=1`` (stream off), take ``kv_transfer_params`` from the answer, send the original
request plus those params to a decode instance and relay its answer (streaming or not).
Instances are picked round-robin; a failed prefill is retried on the next instance.
Also serves ``/v1/models`` and ``/healthcheck``
(reference: examples/disagg/toy_proxy_server.py:445-719)."""
import itertools
import json


def build_proxy_app(prefill_urls: list, decode_urls: list, retries: int = 2, client_factory=None):
    import aiohttp
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    app = FastAPI(title="b200 P/D proxy")
    rr_p, rr_d = itertools.cycle(prefill_urls), itertools.cycle(decode_urls)
    app.state.counts = {"prefill": 0, "decode": 0, "retries": 0}
    make_client = client_factory or (lambda: aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=600)))

    async def _prefill(path: str, body: dict) -> dict:
        pb = dict(body)
        pb.update({"max_tokens": 1, "max_completion_tokens": 1, "stream": False})
        pb.setdefault("kv_transfer_params", {})["do_remote_decode"] = True
        last = None
        for attempt in range(retries + 1):
            url = next(rr_p) + path
            try:
                async with make_client() as s:
                    async with s.post(url, json=pb) as r:
                        if r.status != 200:
                            raise RuntimeError(f"prefill {url} answered {r.status}: {await r.text()}")
                        data = await r.json()
                app.state.counts["prefill"] += 1
                if not data.get("kv_transfer_params"):
                    raise RuntimeError("prefill instance returned no kv_transfer_params")
                return data
            except Exception as e:                     # noqa: BLE001 - try the next instance
                last = e
                app.state.counts["retries"] += 1
        raise HTTPException(502, f"all prefill attempts failed: {last!r}")

    async def _handle(path: str, request: Request):
        body = await request.json()
        pre = await _prefill(path, body)
        db = dict(body)
        db["kv_transfer_params"] = pre["kv_transfer_params"]
        url = next(rr_d) + path
        app.state.counts["decode"] += 1
        if body.get("stream"):
            async def relay():
                async with make_client() as s:
                    async with s.post(url, json=db) as r:
                        async for chunk in r.content.iter_any():
                            yield chunk
            return StreamingResponse(relay(), media_type="text/event-stream")
        async with make_client() as s:
            async with s.post(url, json=db) as r:
                if r.status != 200:
                    raise HTTPException(r.status, await r.text())
                return JSONResponse(await r.json())

    @app.post("/v1/completions")
    async def completions(request: Request):
        return await _handle("/v1/completions", request)

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        return await _handle("/v1/chat/completions", request)

    @app.get("/v1/models")
    async def models():
        async with make_client() as s:
            async with s.get(decode_urls[0] + "/v1/models") as r:
                return JSONResponse(await r.json())

    @app.get("/healthcheck")
    async def health():
        return {"status": "ok", **app.state.counts}

    return app


def run_proxy(prefill_hosts, prefill_ports, decode_hosts, decode_ports, host="0.0.0.0", port=8000):
    import uvicorn
    p = [f"http://{h}:{pt}" for h, pt in zip(prefill_hosts, prefill_ports)]
    d = [f"http://{h}:{pt}" for h, pt in zip(decode_hosts, decode_ports)]
    uvicorn.run(build_proxy_app(p, d), host=host, port=port, log_level="warning")
