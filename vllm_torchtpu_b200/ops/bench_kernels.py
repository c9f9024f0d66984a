"""Kernel micro-benchmarks with roofline fractions.

    python -m vllm_torchtpu_b200.ops.bench_kernels gemm --T 64 --N 4096 --K 4096
    python -m vllm_torchtpu_b200.ops.bench_kernels gemm-sweep
    python -m vllm_torchtpu_b200.ops.bench_kernels attn-decode --reqs 64 --ctx 1100
    python -m vllm_torchtpu_b200.ops.bench_kernels attn-prefill --reqs 8 --q 1024
    python -m vllm_torchtpu_b200.ops.bench_kernels decode-layer --reqs 64 --ctx 1100
    python -m vllm_torchtpu_b200.ops.bench_kernels decode-model --reqs 64 --ctx 1100 --tp 8

Timing: CUDA events on the launching stream, >= 3 warm-up launches, L2 flushed
(a 256 MB buffer is rewritten) before every timed launch, median of the timed
launches.  Fractions are against the measured peaks in ``MEASURED_PEAKS.json`` at
the repository root when that file exists, else the fallback figures below.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"]}, "of measured"
    return dict(FALLBACK), "of fallback"


def time_fn(fn, iters: int = 20, warmup: int = 3, flush: bool = True, use_graph: bool = True) -> float:
    from . import cuda
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # the op is captured into a CUDA graph so that host launch latency (ctypes, Python) between the
    # events does not count: small kernels would otherwise be timed as launch-bound
    replay = fn
    if use_graph:
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        replay = g.replay
    ts = []
    for _ in range(iters):
        if flush:
            cuda.flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def _select_gemm_impl(impl: str) -> None:
    """'2sm' routes every dense GEMM of this process to the two-SM kernel, 'tcgen05' to the one-SM one."""
    import os
    from .. import envs
    os.environ["B200_GEMM_2SM_MIN_T"] = "1" if impl == "2sm" else "0"
    envs.reset()


def bench_gemm(T, N, K, iters=20, impl="tcgen05", check=True) -> dict:
    from . import cuda
    pk, tag = peaks()
    _select_gemm_impl(impl)
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    if impl in ("tcgen05", "2sm"):
        fn = lambda: cuda.gemm(x, w, out=y)
    else:
        fn = lambda: torch.matmul(x, w.t(), out=y)
    ms = time_fn(fn, iters)
    err = None
    if check and impl in ("tcgen05", "2sm"):
        want = x.float() @ w.float().t()
        err = float((y.float() - want).abs().max() / want.abs().max())
    flops = 2.0 * T * N * K
    byts = 2.0 * (T * K + N * K + T * N)
    tf = flops / ms / 1e9
    gbs = byts / ms / 1e6
    t_roof = max(flops / (pk["bf16_tflops"] * 1e12), byts / (pk["hbm_gbs"] * 1e9)) * 1e3
    bn, splits, _, _ = cuda.gemm_plan(T, N, K)
    return {"op": "gemm", "impl": impl, "T": T, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
            "gbs": round(gbs, 1), "roofline_ms": round(t_roof, 4), "frac_of_roofline": round(t_roof / ms, 3),
            "peaks": tag, "bn": bn, "splits": splits, "rel_err": err, "status": cuda.check_status()}


def bench_attn_decode(reqs, ctx, Hq=32, Hkv=8, D=128, iters=20, kv_fp8=False) -> dict:
    from ..runner.attn_metadata import AttentionMetadata
    from . import cuda
    pk, tag = peaks()
    bs = 16
    nblk_per = -(-ctx // bs)
    nb = reqs * nblk_per + 1
    cache = (torch.randn(nb, 2, Hkv, bs, D, device="cuda") * 0.5).bfloat16()
    if kv_fp8:
        cache = cache.to(torch.float8_e4m3fn)
    bt = (torch.randperm(nb - 1, device="cuda") + 1).to(torch.int32).view(reqs, nblk_per).contiguous()
    q = torch.randn(reqs, Hq, D, device="cuda").bfloat16()
    qsl = torch.arange(reqs + 1, device="cuda", dtype=torch.int32)
    sl = torch.full((reqs,), ctx, device="cuda", dtype=torch.int32)
    meta = AttentionMetadata(None, None, bt, sl, qsl, reqs, reqs, num_decode_reqs=reqs, max_seq_len=ctx,
                             padded_num_reqs=reqs, padded_num_tokens=reqs)
    fn = lambda: cuda.paged_attention(q, cache, meta, D ** -0.5)
    ms = time_fn(fn, iters)
    byts = reqs * ctx * 2 * Hkv * D * float(cache.element_size())
    gbs = byts / ms / 1e6
    return {"op": "attn_decode", "kv": "e4m3" if kv_fp8 else "bf16", "reqs": reqs, "ctx": ctx, "Hq": Hq, "Hkv": Hkv, "ms": round(ms, 4),
            "kv_gbs": round(gbs, 1), "frac_of_hbm": round(gbs / pk["hbm_gbs"], 3), "peaks": tag,
            "splits": cuda.decode_splits(reqs, Hkv)}


def bench_attn_prefill(reqs, qlen, Hq=32, Hkv=8, D=128, iters=10) -> dict:
    from ..runner.attn_metadata import AttentionMetadata
    from . import cuda
    pk, tag = peaks()
    bs = 16
    nblk_per = -(-qlen // bs)
    nb = reqs * nblk_per + 1
    cache = (torch.randn(nb, 2, Hkv, bs, D, device="cuda") * 0.5).bfloat16()
    bt = (torch.randperm(nb - 1, device="cuda") + 1).to(torch.int32).view(reqs, nblk_per).contiguous()
    T = reqs * qlen
    q = torch.randn(T, Hq, D, device="cuda").bfloat16()
    qsl = (torch.arange(reqs + 1, device="cuda", dtype=torch.int32) * qlen)
    sl = torch.full((reqs,), qlen, device="cuda", dtype=torch.int32)
    meta = AttentionMetadata(None, None, bt, sl, qsl, reqs, T, num_decode_reqs=0, max_query_len=qlen,
                             max_seq_len=qlen, padded_num_reqs=reqs, padded_num_tokens=T,
                             query_start_loc_cpu=qsl.cpu().long())
    fn = lambda: cuda.paged_attention(q, cache, meta, D ** -0.5)
    ms = time_fn(fn, iters)
    flops = reqs * Hq * 4.0 * D * qlen * qlen / 2
    return {"op": "attn_prefill", "reqs": reqs, "q": qlen, "ms": round(ms, 4),
            "tflops_causal": round(flops / ms / 1e9, 1),
            "frac_of_bf16_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3), "peaks": tag}


def bench_decode_layer(reqs, ctx, layers=8, parts="all", iters=10, H=4096, I=14336, Hq=32, Hkv=8, D=128,
                       tp=1) -> dict:
    """One CUDA graph of ``layers`` Llama-8B-shaped decoder layers (distinct weights and KV, so every
    layer streams from HBM) on a batch of ``reqs`` decode tokens at context ``ctx``; reports device
    time per layer.  ``parts`` keeps a subset: gemm | attn | elem | all."""
    from ..runner.attn_metadata import AttentionMetadata
    from . import cuda
    from . import reference as ref
    pk, tag = peaks()
    # the per-rank shapes of a tensor-parallel layout, run on one GPU without the collectives
    I, Hq, Hkv = I // tp, Hq // tp, max(1, Hkv // tp)
    bs = 16
    nblk_per = -(-(ctx + 1) // bs)
    nb = reqs * nblk_per + 1
    T = reqs
    dev = "cuda"
    Ws = [dict(qkv=(torch.randn((Hq + 2 * Hkv) * D, H, device=dev) * 0.02).bfloat16(),
               o=(torch.randn(H, Hq * D, device=dev) * 0.02).bfloat16(),
               gu=(torch.randn(2 * I, H, device=dev) * 0.02).bfloat16(),
               down=(torch.randn(H, I, device=dev) * 0.02).bfloat16(),
               ln1=torch.ones(H, device=dev, dtype=torch.bfloat16), ln2=torch.ones(H, device=dev, dtype=torch.bfloat16),
               kv=(torch.randn(nb, 2, Hkv, bs, D, device=dev) * 0.5).bfloat16()) for _ in range(layers)]
    bt = (torch.randperm(nb - 1, device=dev) + 1).to(torch.int32).view(reqs, nblk_per).contiguous()
    qsl = torch.arange(reqs + 1, device=dev, dtype=torch.int32)
    sl = torch.full((reqs,), ctx + 1, device=dev, dtype=torch.int32)
    pos = torch.full((T,), ctx, device=dev, dtype=torch.int32)
    slots = (bt[:, ctx // bs].long() * bs + ctx % bs).to(torch.int32)
    inv = ref.rope_inv_freq(D, 500000.0).to(dev)
    meta = AttentionMetadata(pos, slots, bt, sl, qsl, reqs, T, num_decode_reqs=reqs, max_query_len=1,
                             max_seq_len=ctx + 1, padded_num_reqs=reqs, padded_num_tokens=T)
    x0 = torch.randn(T, H, device=dev).bfloat16()
    res0 = torch.randn(T, H, device=dev).bfloat16()
    qkv_fix = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
    q_fix = torch.randn(T, Hq, D, device=dev).bfloat16()
    act_fix = torch.randn(T, I, device=dev).bfloat16()
    g, a, e = parts in ("all", "gemm"), parts in ("all", "attn"), parts in ("all", "elem")

    def fn():
        h, res = x0, res0.clone()
        for w in Ws:
            if e:
                h, res = cuda.fused_add_rms_norm(h, res, w["ln1"], 1e-5)
            qkv = cuda.gemm(h, w["qkv"]) if g else qkv_fix
            q = cuda.rope_and_cache(qkv, pos, inv, w["kv"], slots, Hq, Hkv, D) if e else q_fix
            o = cuda.paged_attention(q, w["kv"], meta, D ** -0.5) if a else q
            h = cuda.gemm(o.view(T, Hq * D), w["o"]) if g else x0
            if e:
                h, res = cuda.fused_add_rms_norm(h, res, w["ln2"], 1e-5)
            if g:
                h = cuda.gemm(cuda.gemm_swiglu(h, w["gu"]), w["down"])
        return h

    ms = time_fn(fn, iters, flush=False)
    w_bytes = 2.0 * ((Hq + 2 * Hkv) * D * H + H * Hq * D + 2 * I * H + H * I)
    kv_bytes = reqs * (ctx + 1) * 2 * Hkv * D * 2.0
    byts = (w_bytes if g else 0) + (kv_bytes if a else 0)
    us = ms * 1e3 / layers
    roof_us = byts / (pk["hbm_gbs"] * 1e9) * 1e6
    return {"op": "decode_layer", "parts": parts, "reqs": reqs, "ctx": ctx, "layers": layers, "tp_shapes": tp,
            "us_per_layer": round(us, 2), "hbm_roofline_us": round(roof_us, 2),
            "frac_of_hbm": round(roof_us / us, 3) if us > 0 else None, "peaks": tag,
            "status": cuda.check_status()}


def bench_decode_model(reqs, ctx, layers=8, iters=10, H=4096, I=14336, Hq=32, Hkv=8, tp=1) -> list:
    """A dense Llama-8B-shaped model of ``layers`` decoder layers (per-rank shapes of TP degree ``tp``,
    run on one GPU without collectives) on a decode batch: the persistent decode kernel against the
    per-layer kernel chain, both replayed from a CUDA graph; device time per layer."""
    from ..config import ModelConfig
    from ..models.llama import LlamaForCausalLM
    from ..runner.attn_metadata import AttentionMetadata
    from . import cuda
    pk, tag = peaks()
    I, Hq, Hkv = I // tp, Hq // tp, max(1, Hkv // tp)
    cfg = ModelConfig(name="bench", num_layers=layers, hidden_size=H, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=128,
                      intermediate_size=I, vocab_size=1024, max_model_len=ctx + 64, dtype=torch.bfloat16)
    m = LlamaForCausalLM(cfg, "cuda")
    m.init_dummy()
    bs, dev = 16, "cuda"
    nblk_per = -(-(ctx + 1) // bs)
    nb = reqs * nblk_per + 1
    kvs = [(torch.randn(nb, 2, Hkv, bs, 128, device=dev) * 0.5).bfloat16() for _ in range(layers)]
    bt = (torch.randperm(nb - 1, device=dev) + 1).to(torch.int32).view(reqs, nblk_per).contiguous()
    qsl = torch.arange(reqs + 1, device=dev, dtype=torch.int32)
    sl = torch.full((reqs,), ctx + 1, device=dev, dtype=torch.int32)
    pos = torch.full((reqs,), ctx, device=dev, dtype=torch.int32)
    slots = (bt[:, ctx // bs].long() * bs + ctx % bs).to(torch.int32)
    meta = AttentionMetadata(pos, slots, bt, sl, qsl, reqs, reqs, num_decode_reqs=reqs, max_query_len=1,
                             max_seq_len=ctx + 1, padded_num_reqs=reqs, padded_num_tokens=reqs)
    x0 = torch.randn(reqs, H, device=dev).bfloat16()
    w_bytes = 2.0 * ((Hq + 2 * Hkv) * 128 * H + H * Hq * 128 + 2 * I * H + H * I)
    kv_bytes = reqs * (ctx + 1) * 2 * Hkv * 128 * 2.0
    roof_us = (w_bytes + kv_bytes) / (pk["hbm_gbs"] * 1e9) * 1e6
    out = []
    import os
    from .. import envs
    os.environ["B200_DECODE_MEGAKERNEL"] = "1"
    envs.reset()
    for mode in ("persistent", "per-layer"):
        if mode == "persistent":
            m.setup_decode_fusion(kvs)
            if m.decode_mega is None:
                out.append({"op": "decode_model", "mode": mode, "skipped": m.decode_mega_reason})
                continue
        else:
            m.decode_mega = None
        ms = time_fn(lambda: m.forward(None, meta, kvs, hidden=x0), iters, flush=False)
        us = ms * 1e3 / layers
        out.append({"op": "decode_model", "mode": mode, "reqs": reqs, "ctx": ctx, "layers": layers, "tp_shapes": tp,
                    "us_per_layer": round(us, 2), "hbm_roofline_us": round(roof_us, 2),
                    "frac_of_hbm": round(roof_us / us, 3), "peaks": tag, "status": cuda.check_status()})
    return out


def bench_fp8_gemm(T, N, K, iters=20) -> list:
    """Block-scaled e4m3 GEMM (128x128 weight scales, 1x128 activation scales) of this package, with and
    without the activation quantisation kernel, next to ``torch._scaled_mm`` on the same e4m3 operands
    (library kernel; per-tensor scales, and row-wise scales where the library accepts them) and to the
    bf16 tcgen05 GEMM of the same shape.  Roofline: fp8 weight + activation bytes and bf16 output bytes
    over the measured copy bandwidth, FLOPs over twice the measured bf16 GEMM rate."""
    from . import cuda
    from ..quantization.fp8 import fp8_block_gemm_reference, quantize_weight_block
    pk, tag = peaks()
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    wq, wsi = quantize_weight_block(w)
    xq, xs = cuda.quant_act_1x128(x)
    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    from . import cuda_fp8

    def gemm_only():
        cuda_fp8.fp8_block_gemm_quantised(xq, xs, wq, wsi, y)
    flops = 2.0 * T * N * K
    byts = float(T * K + N * K + 2 * T * N)
    t_roof = max(flops / (2 * pk["bf16_tflops"] * 1e12), byts / (pk["hbm_gbs"] * 1e9)) * 1e3
    rows = []

    def row(impl, ms, err=None, note=None):
        r = {"op": "fp8-gemm", "impl": impl, "T": T, "N": N, "K": K, "ms": round(ms, 4),
             "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
             "roofline_ms": round(t_roof, 4), "frac_of_roofline": round(t_roof / ms, 3), "peaks": tag,
             "rel_err": err, "status": cuda.check_status()}
        if note:
            r["note"] = note
        rows.append(r)
    want = fp8_block_gemm_reference(x, wq, wsi).float() if T * N <= (1 << 24) else None
    ms = time_fn(gemm_only, iters)
    err = float((y.float() - want).abs().max() / want.abs().max()) if want is not None else None
    row("tcgen05 block-scaled (operands quantised)", ms, err)
    ms = time_fn(lambda: cuda.fp8_block_gemm(x, wq, wsi, out=y), iters)
    row("tcgen05 block-scaled + activation quant kernel", ms)
    one = torch.ones((), device="cuda", dtype=torch.float32)
    wt = wq.t()                                   # column-major second operand, as the library wants
    try:
        ms = time_fn(lambda: torch._scaled_mm(xq, wt, scale_a=one, scale_b=one, out_dtype=torch.bfloat16), iters)
        row("torch._scaled_mm per-tensor scales", ms, note="library kernel; coarser scaling than the block kernel")
    except Exception as e:                        # noqa: BLE001 - recorded in the output
        rows.append({"op": "fp8-gemm", "impl": "torch._scaled_mm per-tensor scales", "unavailable": str(e)[:200]})
    try:
        sa = torch.ones(T, 1, device="cuda", dtype=torch.float32)
        sb = torch.ones(1, N, device="cuda", dtype=torch.float32)
        ms = time_fn(lambda: torch._scaled_mm(xq, wt, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16), iters)
        row("torch._scaled_mm row-wise scales", ms, note="library kernel")
    except Exception as e:                        # noqa: BLE001
        rows.append({"op": "fp8-gemm", "impl": "torch._scaled_mm row-wise scales", "unavailable": str(e)[:200]})
    ms = time_fn(lambda: cuda.gemm(x, w, out=y), iters)
    row("tcgen05 bf16 (same shape)", ms, note="bf16 operands: twice the weight bytes")
    return rows


def bench_w4a16(T, N, K, iters=20) -> list:
    """mxfp4 / nvfp4 weights expanded in shared memory in front of tcgen05 (W4A16) next to the bf16 GEMM of
    the same shape.  Roofline: packed weight + scale + activation + output bytes over the measured copy
    bandwidth, FLOPs over the measured bf16 GEMM rate."""
    from . import cuda
    from ..quantization import fp4 as q
    pk, tag = peaks()
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05)
    rows = []
    flops = 2.0 * T * N * K
    for fmt in ("mxfp4", "nvfp4"):
        if fmt == "mxfp4":
            wp, sc = q.quantize_mxfp4(w)
            gs = None
            wd = q.dequantize_mxfp4(wp, sc)
        else:
            wp, sc, gs = q.quantize_nvfp4(w)
            wd = q.dequantize_nvfp4(wp, sc, gs)
        wp, sc = wp.contiguous(), sc.contiguous()
        ms = time_fn(lambda: cuda.w4a16_gemm(x, wp, sc, fmt, gs), iters)
        err = None
        if T * N <= (1 << 24):
            y = cuda.w4a16_gemm(x, wp, sc, fmt, gs)
            want = x.float() @ wd.bfloat16().float().t()
            err = float((y.float() - want).abs().max() / want.abs().max())
        byts = float(N * K // 2 + sc.numel() + 2 * T * K + 2 * T * N)
        t_roof = max(flops / (pk["bf16_tflops"] * 1e12), byts / (pk["hbm_gbs"] * 1e9)) * 1e3
        rows.append({"op": "w4a16-gemm", "fmt": fmt, "T": T, "N": N, "K": K, "ms": round(ms, 4),
                     "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                     "roofline_ms": round(t_roof, 4), "frac_of_roofline": round(t_roof / ms, 3), "peaks": tag,
                     "rel_err": err, "status": cuda.check_status()})
    # AWQ / GPTQ style int4 (fp16 group scales and zero points, group 128) on the same kernel
    from ..quantization.int4 import dequantize_int4_group, quantize_int4_group
    from . import cuda_fp4
    wp, sc, zp = quantize_int4_group(w, 128)
    wp, sh, zp = wp.contiguous(), sc.half().contiguous(), zp.contiguous()
    ms = time_fn(lambda: cuda_fp4.w4a16_int4_gemm(x, wp, sh, zp, 128), iters)
    err = None
    if T * N <= (1 << 24):
        want = x.float() @ dequantize_int4_group(wp, sc, zp, 128).bfloat16().float().t()
        err = float((cuda_fp4.w4a16_int4_gemm(x, wp, sh, zp, 128).float() - want).abs().max() / want.abs().max())
    byts = float(N * K // 2 + 3 * sh.numel() + 2 * T * K + 2 * T * N)
    t_roof = max(flops / (pk["bf16_tflops"] * 1e12), byts / (pk["hbm_gbs"] * 1e9)) * 1e3
    rows.append({"op": "w4a16-gemm", "fmt": "int4 g128", "T": T, "N": N, "K": K, "ms": round(ms, 4),
                 "tflops": round(flops / ms / 1e9, 1), "gbs": round(byts / ms / 1e6, 1),
                 "roofline_ms": round(t_roof, 4), "frac_of_roofline": round(t_roof / ms, 3), "peaks": tag,
                 "rel_err": err, "status": cuda.check_status()})
    wb = w.bfloat16()
    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    ms = time_fn(lambda: cuda.gemm(x, wb, out=y), iters)
    rows.append({"op": "w4a16-gemm", "fmt": "bf16 weights (same shape)", "T": T, "N": N, "K": K, "ms": round(ms, 4),
                 "tflops": round(flops / ms / 1e9, 1)})
    return rows


def bench_misc(iters=20, only: str = "") -> list:
    """Element-wise, routing, sampling and MLA kernels at serving shapes: device time (graph replay, L2
    flushed), algorithmic bytes over the measured copy bandwidth."""
    from ..runner.attn_metadata import AttentionMetadata
    from . import cuda
    from . import reference as ref
    pk, tag = peaks()
    rows = []

    def row(op, shape, fn, byts, note=None):
        if only and only not in op:
            return                                  # --only <substring>: time one kernel family (profiler captures)
        ms = time_fn(fn, iters)
        r = {"op": op, "shape": shape, "us": round(ms * 1e3, 2), "gbs": round(byts / ms / 1e6, 1),
             "frac_of_hbm": round(byts / ms / 1e6 / pk["hbm_gbs"], 3), "peaks": tag, "status": cuda.check_status()}
        if note:
            r["note"] = note
        rows.append(r)
    dev = "cuda"
    for T in (64, 8192):
        H, I = 4096, 14336
        x = torch.randn(T, H, device=dev).bfloat16()
        res = torch.randn(T, H, device=dev).bfloat16()
        w = torch.ones(H, device=dev).bfloat16()
        row("rms_norm", [T, H], lambda: cuda.rms_norm(x, w, 1e-5), 2.0 * T * H * 2)
        row("fused_add_rms_norm", [T, H], lambda: cuda.fused_add_rms_norm(x, res, w, 1e-5),
            4.0 * T * H * 2)
        gu = torch.randn(T, 2 * I, device=dev).bfloat16()
        row("silu_and_mul", [T, 2 * I], lambda: cuda.silu_and_mul(gu), 3.0 * T * I * 2)
        row("quant_act_1x128", [T, I], lambda: cuda.quant_act_1x128(gu[:, :I].contiguous()),
            T * I * 3.0 + T * I * 2.0, note="includes the contiguous copy of the slice")
        row("quant_rows_1x128 swiglu", [T, 2 * I], lambda: cuda.quant_rows_1x128(gu, I, swiglu=True),
            T * I * 5.0)
        # RoPE + q/k norm-free KV write, Llama-8B heads
        Hq, Hkv, D, bs = 32, 8, 128, 16
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).bfloat16()
        nb = T // bs + 2
        cache = torch.zeros(nb, 2, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
        pos = torch.arange(T, device=dev, dtype=torch.int32)
        slots = torch.arange(T, device=dev, dtype=torch.int32)
        inv_freq = ref.rope_inv_freq(D, 500000.0, None).to(dev)
        row("rope_and_cache", [T, Hq, Hkv, D],
            lambda: cuda.rope_and_cache(qkv, pos, inv_freq, cache, slots, Hq, Hkv, D),
            T * (Hq + 2 * Hkv) * D * 2.0 + T * (Hq + 2 * Hkv) * D * 2.0)
        # MoE routing / permutation, Qwen3-30B-A3B shape
        E, k, Hm = 128, 8, 2048
        logits = torch.randn(T, E, device=dev)
        row("moe_route", [T, E, k], lambda: cuda.moe_route(logits, k), T * E * 4.0 + T * k * 8.0)
        ids, wts = cuda.moe_route(logits, k)
        xm = torch.randn(T, Hm, device=dev).bfloat16()
        row("moe_permute", [T, k, Hm], lambda: cuda.moe_permute(xm, ids, 0, E),
            T * Hm * 2.0 + T * k * Hm * 2.0)
        xp, goff, _, inv = cuda.moe_permute(xm, ids, 0, E)
        row("moe_unpermute", [T, k, Hm], lambda: cuda.moe_unpermute(xp, inv, wts, T),
            T * k * Hm * 2.0 + T * Hm * 2.0)
    # sampling over the Llama-3 vocabulary
    R, V = 64, 128256
    lg = torch.randn(R, V, device=dev).bfloat16()
    row("argmax", [R, V], lambda: cuda.argmax(lg), R * V * 2.0)
    temp = torch.full((R,), 0.8, device=dev)
    tk = torch.full((R,), 50, device=dev, dtype=torch.int32)
    tp = torch.full((R,), 0.9, device=dev)
    row("sample top-k 50 top-p 0.9", [R, V], lambda: cuda.sample(lg, temp, tk, tp, None, False, 1),
        R * V * 2.0, note="several passes over the row by design (bisection); bytes = one pass")
    # MLA decode, DeepSeek-V3 per-rank shape at TP8: 16 heads, latent 512 + 64
    for reqs, ctx in ((64, 2048),):
        Hh, L, Rr, bs = 16, 512, 64, 16
        nblk = -(-ctx // bs)
        cache = (torch.randn(reqs * nblk + 1, bs, L + Rr, device=dev) * 0.3).bfloat16()
        bt = (torch.randperm(reqs * nblk, device=dev) + 1).to(torch.int32).view(reqs, nblk).contiguous()
        q = torch.randn(reqs, Hh, L + Rr, device=dev).bfloat16()
        qsl = torch.arange(reqs + 1, device=dev, dtype=torch.int32)
        sl = torch.full((reqs,), ctx, device=dev, dtype=torch.int32)
        meta = AttentionMetadata(None, None, bt, sl, qsl, reqs, reqs, num_decode_reqs=reqs, max_seq_len=ctx,
                                 padded_num_reqs=reqs, padded_num_tokens=reqs)
        row("mla_decode", [reqs, ctx, Hh, L + Rr],
            lambda: cuda.mla_paged_attention(q, cache, meta, (128 + 64) ** -0.5, L),
            reqs * ctx * (L + Rr) * 2.0, note="bytes = one read of every latent row")
        w_uk_t = (torch.randn(Hh, L, 128, device=dev) * 0.05).bfloat16()
        qq = torch.randn(reqs, Hh, 192, device=dev).bfloat16()
        kvx = torch.randn(reqs, L + Rr, device=dev).bfloat16()
        pos = torch.full((reqs,), ctx - 1, device=dev, dtype=torch.int32)
        inv_freq = ref.rope_inv_freq(64, 10000.0, None).to(dev)
        row("mla_absorb (permute, grouped GEMM, permute, 2 x rope)", [reqs, Hh, 128, L],
            lambda: cuda.mla_absorb(qq, kvx, pos, inv_freq, w_uk_t, 128, 64, L, False),
            Hh * L * 128 * 2.0 + reqs * Hh * (192 + L + 64) * 2.0, note="five launches")
    return rows


def bench_gemm_swiglu(T, I, K, iters=20, impl="tcgen05") -> dict:
    """silu(x Wg^T) * (x Wu^T) with W = [2I, K]; 'cublas' is torch.matmul followed by an eager activation."""
    from . import cuda
    pk, tag = peaks()
    _select_gemm_impl(impl)
    x = torch.randn(T, K, device="cuda").bfloat16()
    w = (torch.randn(2 * I, K, device="cuda") * 0.05).bfloat16()
    y = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    if impl in ("tcgen05", "2sm"):
        fn = lambda: cuda.gemm_swiglu(x, w, out=y)
    else:
        def fn():
            gu = torch.matmul(x, w.t())
            torch.mul(torch.nn.functional.silu(gu[:, :I]), gu[:, I:], out=y)
    ms = time_fn(fn, iters)
    gu = x.float() @ w.float().t()
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    err = float((y.float() - want).abs().max() / want.abs().max())
    tf = 4.0 * T * I * K / ms / 1e9
    return {"op": "gemm_swiglu", "impl": impl, "T": T, "I": I, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
            "frac_of_bf16_peak": round(tf / pk["bf16_tflops"], 3), "peaks": tag, "rel_err": err,
            "status": cuda.check_status()}


def bench_gemm_sustained(T, N, K, seconds=3.0, impl="tcgen05") -> dict:
    """The same GEMM launched back to back for ``seconds`` (under the board power cap the clocks
    settle below the burst value): average TFLOP/s over the whole run, with distinct weights cycled
    so that operands stream from HBM."""
    import subprocess
    import time
    from . import cuda
    pk, tag = peaks()
    x = torch.randn(T, K, device="cuda").bfloat16()
    ws = [(torch.randn(N, K, device="cuda") * 0.05).bfloat16() for _ in range(4)]
    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    _select_gemm_impl(impl)
    fn = ((lambda w: cuda.gemm(x, w, out=y)) if impl in ("tcgen05", "2sm")
          else (lambda w: torch.matmul(x, w.t(), out=y)))
    g = torch.cuda.CUDAGraph()
    for w in ws:
        fn(w)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        for _ in range(8):
            for w in ws:
                fn(w)
    per_replay = 32
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_end = time.time() + seconds
    n = 0
    a.record()
    while time.time() < t_end:
        g.replay()
        n += per_replay
        if n % (per_replay * 16) == 0:
            torch.cuda.synchronize()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    clk = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-i",
                          str(torch.cuda.current_device())], capture_output=True, text=True).stdout.strip()
    tf = 2.0 * T * N * K * n / ms / 1e9
    return {"op": "gemm_sustained", "impl": impl, "T": T, "N": N, "K": K, "seconds": round(ms / 1e3, 2),
            "tflops": round(tf, 1), "launches": n, "clock_power_after": clk, "peaks": tag}


LLAMA8B_SHAPES = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096)]


def bench_omni(S=8192, H=16, D=128, iters=10) -> list:
    """Diffusion-transformer kernels at one sequence of S tokens: the tcgen05 attention kernel without the causal
    mask (timed on a pre-packed paged layout, as the kernel sees it) and the fused q/k norm + RoPE over
    H * D channels."""
    from ctypes import c_float, c_int, c_longlong, c_void_p

    from ..omni.ops import qk_norm_rope
    from ..omni.rope import rope_table_1d
    from . import cuda
    pk, tag = peaks()
    bs = 16
    nblk = -(-S // bs)
    cache = (torch.randn(nblk, 2, H, bs, D, device="cuda") * 0.5).bfloat16()
    bt = torch.arange(nblk, device="cuda", dtype=torch.int32).view(1, nblk).contiguous()
    q = torch.randn(S, H, D, device="cuda").bfloat16()
    out = torch.empty_like(q)
    qsl = torch.tensor([0, S], device="cuda", dtype=torch.int32)
    sl = torch.tensor([S], device="cuda", dtype=torch.int32)
    ws = cuda.Workspace.get(q.device)
    tiles = -(-S // 64)

    def attn():
        cuda._check(cuda.lib().b200_attn_encoder_tc(
            cuda._p(q), cuda._p(cache), cuda._p(out), c_void_p(0), cuda._p(bt), cuda._p(sl), cuda._p(qsl), c_int(0),
            c_int(1), c_int(tiles), c_int(S), c_int(nblk), c_int(bs), c_longlong(nblk), c_int(H), c_int(H), c_int(D),
            c_float(D ** -0.5), cuda._p(ws.status), cuda._stream()), "attn_encoder_tc")
    ms = time_fn(attn, iters)
    flops = 4.0 * D * S * S * H
    rows = [{"op": "attn_non_causal_tc", "S": S, "heads": H, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
             "frac_of_bf16_peak": round(flops / ms / 1e9 / pk["bf16_tflops"], 3), "peaks": tag}]
    C = H * D
    qkv = torch.randn(S, 3 * C, device="cuda").bfloat16()
    wq, wk = torch.ones(C, device="cuda").bfloat16(), torch.ones(C, device="cuda").bfloat16()
    cos, sin = rope_table_1d(S, D, device="cuda")
    ms = time_fn(lambda: qk_norm_rope(qkv, wq, wk, cos, sin, H, H, D), iters)
    nbytes = 4.0 * S * C * 2 + 4.0 * S * D       # q, k read and written; two fp32 tables of D / 2 per token
    rows.append({"op": "qk_norm_rope", "T": S, "channels": C, "ms": round(ms, 4),
                 "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3),
                 "peaks": tag})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "fp8-gemm", "w4a16-gemm", "misc", "gemm-swiglu", "gemm-sweep", "gemm-sustained", "attn-decode", "attn-prefill",
                                     "decode-layer", "decode-model", "omni", "all"])
    ap.add_argument("--T", type=int, default=64)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--reqs", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1100)
    ap.add_argument("--q", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="", help="misc: time only the rows whose name contains this")
    ap.add_argument("--impl", default="tcgen05", choices=["tcgen05", "2sm", "cublas"])
    ap.add_argument("--impls", default="tcgen05,cublas", help="gemm-sustained: implementations to run")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tp", type=int, default=1, help="decode-layer: use the per-rank shapes of this TP degree")
    ap.add_argument("--parts", default="all,gemm,attn,elem")
    ap.add_argument("--kv-fp8", action="store_true", help="attn-decode: e4m3 KV cache")
    a = ap.parse_args()
    if a.what == "gemm":
        print(json.dumps(bench_gemm(a.T, a.N, a.K, a.iters, a.impl)))
    elif a.what in ("gemm-sweep", "all"):
        for T in (64, 256, 1024, 8192):
            for N, K in LLAMA8B_SHAPES:
                if T == 8192 and N > 100000:
                    continue
                for impl in ("tcgen05", "cublas"):
                    print(json.dumps(bench_gemm(T, N, K, max(5, a.iters // 2), impl, check=(T <= 1024))))
    if a.what == "omni":
        for r in bench_omni(a.q, a.T, 128, a.iters):
            print(json.dumps(r))
    if a.what == "w4a16-gemm":
        for r in bench_w4a16(a.T, a.N, a.K, a.iters):
            print(json.dumps(r))
    if a.what == "misc":
        for r in bench_misc(a.iters, a.only):
            print(json.dumps(r))
    if a.what == "fp8-gemm":
        for r in bench_fp8_gemm(a.T, a.N, a.K, a.iters):
            print(json.dumps(r))
    if a.what == "gemm-swiglu":
        print(json.dumps(bench_gemm_swiglu(a.T, a.N, a.K, a.iters, a.impl)))
    if a.what == "gemm-sustained":
        for impl in a.impls.split(","):
            print(json.dumps(bench_gemm_sustained(a.T, a.N, a.K, 3.0, impl)))
    if a.what == "decode-model":
        for row in bench_decode_model(a.reqs, a.ctx, a.layers, a.iters, tp=a.tp):
            print(json.dumps(row))
    if a.what == "decode-layer":
        for parts in a.parts.split(","):
            print(json.dumps(bench_decode_layer(a.reqs, a.ctx, a.layers, parts, a.iters, tp=a.tp)))
    if a.what in ("attn-decode", "all"):
        for reqs, ctx in ((a.reqs, a.ctx),) if a.what == "attn-decode" else ((64, 1100), (256, 2048), (8, 8000)):
            print(json.dumps(bench_attn_decode(reqs, ctx, iters=a.iters, kv_fp8=a.kv_fp8)))
    if a.what in ("attn-prefill", "all"):
        for reqs, q in ((a.reqs, a.q),) if a.what == "attn-prefill" else ((8, 1024), (2, 4096)):
            print(json.dumps(bench_attn_prefill(reqs, q, iters=max(5, a.iters // 2))))


if __name__ == "__main__":
    main()
