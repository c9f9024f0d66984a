"""Prefill/decode disaggregation proxy.

For every ``/v1/completions`` or ``/v1/chat/completions`` request: send it to a prefill instance
with ``max_tokens=1`` (stream off), take ``kv_transfer_params`` from the answer, send the original
request plus those params to a decode instance and relay its answer (streaming or not).
Instances are picked round-robin from the given lists, or, with a controller address, from the controller's
registry (least loaded live instance of the role; an instance that failed is reported unreachable and left
out of the retry); a failed prefill is retried on the next instance.
Also serves ``/v1/models`` and ``/healthcheck``
(reference: examples/disagg/toy_proxy_server.py:445-719)."""
import itertools
import json


def build_proxy_app(prefill_urls: list, decode_urls: list, retries: int = 2, client_factory=None,
                    controller=None):
    import aiohttp
    from fastapi import FastAPI, HTTPException, Request
    from fastapi.responses import JSONResponse, StreamingResponse

    app = FastAPI(title="b200 P/D proxy")
    rr_p, rr_d = itertools.cycle(prefill_urls or [""]), itertools.cycle(decode_urls or [""])
    app.state.counts = {"prefill": 0, "decode": 0, "retries": 0, "reported_unreachable": 0}
    ctl = None
    if controller is not None:
        from .controller import ControllerClient
        ctl = controller if isinstance(controller, ControllerClient) else ControllerClient(controller)

    def pick(role: str, fallback, exclude=()):
        """(base url, engine id or None) of an instance of ``role``."""
        if ctl is not None:
            e = ctl.pick(role, exclude=exclude)
            if e is None:
                raise RuntimeError(f"the controller knows no live {role} instance")
            return e["http_url"], e["engine_id"]
        return next(fallback), None

    def report(engine_id) -> None:
        if ctl is not None and engine_id:
            try:
                ctl.report_unreachable(engine_id, reporter="proxy")
                app.state.counts["reported_unreachable"] += 1
            except (OSError, TimeoutError, ConnectionError):
                pass
    make_client = client_factory or (lambda: aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=600)))

    async def _prefill(path: str, body: dict) -> dict:
        pb = dict(body)
        pb.update({"max_tokens": 1, "max_completion_tokens": 1, "stream": False})
        pb.setdefault("kv_transfer_params", {})["do_remote_decode"] = True
        last = None
        tried = []
        for attempt in range(retries + 1):
            eid = None
            try:
                base, eid = pick("prefill", rr_p, tried)
                url = base + path
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
                if eid:
                    tried.append(eid)
                    if isinstance(e, (OSError, ConnectionError, TimeoutError)) or "Cannot connect" in repr(e):
                        report(eid)
        raise HTTPException(502, f"all prefill attempts failed: {last!r}")

    async def _handle(path: str, request: Request):
        body = await request.json()
        pre = await _prefill(path, body)
        db = dict(body)
        db["kv_transfer_params"] = pre["kv_transfer_params"]
        try:
            base, _ = pick("decode", rr_d)
        except RuntimeError as e:
            raise HTTPException(503, str(e))
        url = base + path
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
        base = decode_urls[0] if decode_urls else pick("decode", rr_d)[0]
        async with make_client() as s:
            async with s.get(base + "/v1/models") as r:
                return JSONResponse(await r.json())

    @app.get("/healthcheck")
    async def health():
        return {"status": "ok", **app.state.counts}

    return app


def run_proxy(prefill_hosts, prefill_ports, decode_hosts, decode_ports, host="0.0.0.0", port=8000,
              controller: str = ""):
    import uvicorn
    p = [f"http://{h}:{pt}" for h, pt in zip(prefill_hosts or [], prefill_ports or [])]
    d = [f"http://{h}:{pt}" for h, pt in zip(decode_hosts or [], decode_ports or [])]
    ctl = None
    if controller:
        h, pt = controller.rsplit(":", 1)
        ctl = (h, int(pt))
    uvicorn.run(build_proxy_app(p, d, controller=ctl), host=host, port=port, log_level="warning")
