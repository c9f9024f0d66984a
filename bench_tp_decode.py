"""Decode-layer chain under tensor parallelism, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        bench_tp_decode.py --reqs 64 --ctx 1100

One CUDA graph of ``--layers`` Llama-3.1-8B-shaped decoder layers (per-rank shapes, distinct weights)
is replayed; the two row-parallel projections of a layer are reduced across ranks by
  push   partial pushed to every rank inside the GEMM, summed in the add + RMSNorm kernel
  fused  GEMM + one-shot all-reduce in one kernel, then add + RMSNorm
  nccl   GEMM, NCCL all-reduce, add + RMSNorm
  none   no reduction (what the layer costs without any cross-rank traffic)
Device time per layer, max over ranks."""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reqs", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1100)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--planes", default="push,fused,nccl,none")
    a = ap.parse_args()
    from vllm_torchtpu_b200.config import ParallelConfig
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    from vllm_torchtpu_b200.parallel import communicator
    from vllm_torchtpu_b200.parallel.state import init_distributed, leave_process
    from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata
    world, rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"])
    st = init_distributed(ParallelConfig(tensor_parallel_size=world, world_size=world, rank=rank,
                                         local_rank=int(os.environ["LOCAL_RANK"])), backend="nccl", timeout_s=120)
    dev = torch.device("cuda", st.local_rank)
    H, I, Hq, Hkv, D = 4096, 14336 // world, 32 // world, max(1, 8 // world), 128
    T, bs = a.reqs, 16
    heap = communicator.ensure_tp_heap(max(T, 256), H)
    nblk_per = -(-(a.ctx + 1) // bs)
    nb = T * nblk_per + 1
    Ws = [dict(qkv=(torch.randn((Hq + 2 * Hkv) * D, H, device=dev) * 0.02).bfloat16(),
               o=(torch.randn(H, Hq * D, device=dev) * 0.02).bfloat16(),
               gu=(torch.randn(2 * I, H, device=dev) * 0.02).bfloat16(),
               down=(torch.randn(H, I, device=dev) * 0.02).bfloat16(),
               ln=torch.ones(H, device=dev, dtype=torch.bfloat16),
               kv=(torch.randn(nb, 2, Hkv, bs, D, device=dev) * 0.5).bfloat16()) for _ in range(a.layers)]
    bt = (torch.randperm(nb - 1, device=dev) + 1).to(torch.int32).view(T, nblk_per).contiguous()
    qsl = torch.arange(T + 1, device=dev, dtype=torch.int32)
    sl = torch.full((T,), a.ctx + 1, device=dev, dtype=torch.int32)
    pos = torch.full((T,), a.ctx, device=dev, dtype=torch.int32)
    slots = (bt[:, a.ctx // bs].long() * bs + a.ctx % bs).to(torch.int32)
    inv = ref.rope_inv_freq(D, 500000.0).to(dev)
    meta = AttentionMetadata(pos, slots, bt, sl, qsl, T, T, num_decode_reqs=T, max_query_len=1,
                             max_seq_len=a.ctx + 1, padded_num_reqs=T, padded_num_tokens=T)
    x0 = torch.randn(T, H, device=dev).bfloat16()
    res0 = torch.randn(T, H, device=dev).bfloat16()

    def reduce_norm(plane, inp, w, res, ln):
        if plane == "push":
            return cuda.gemm_push(inp, w, heap).add_rms_norm(res, ln, 1e-5)
        if plane == "fused":
            return cuda.fused_add_rms_norm(cuda.gemm_all_reduce(inp, w, heap), res, ln, 1e-5)
        y = cuda.gemm(inp, w)
        if plane == "nccl":
            dist.all_reduce(y)
        return cuda.fused_add_rms_norm(y, res, ln, 1e-5)

    def chain(plane):
        h, res = x0, res0.clone()
        for w in Ws:
            qkv = cuda.gemm(h, w["qkv"])
            q = cuda.rope_and_cache(qkv, pos, inv, w["kv"], slots, Hq, Hkv, D)
            o = cuda.paged_attention(q, w["kv"], meta, D ** -0.5)
            h, res = reduce_norm(plane, o.view(T, Hq * D), w["o"], res, w["ln"])
            act = cuda.gemm_swiglu(h, w["gu"])
            h, res = reduce_norm(plane, act, w["down"], res, w["ln"])
        return h

    for plane in a.planes.split(","):
        for _ in range(3):
            chain(plane)
        torch.cuda.synchronize()
        dist.barrier()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            chain(plane)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            chain(plane)
        ts = []
        for _ in range(a.iters):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"op": "tp_decode_layer", "plane": plane, "world": world, "reqs": T, "ctx": a.ctx,
                              "layers": a.layers, "us_per_layer": round(float(t) * 1e3 / a.layers, 2),
                              "status": cuda.check_status()}), flush=True)
        del g
    dist.barrier()
    leave_process(0)


if __name__ == "__main__":
    main()
