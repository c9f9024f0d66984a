"""Child process of the multi-GPU tests: the fused expert-parallel plane (NVLink dispatch, grouped
tcgen05 GEMMs, combine in the GEMM epilogue) against a dense fp32 MoE of the same tokens.  Every rank
holds E / world experts and brings its own tokens (a different count on every rank).

``--timing`` runs the bf16 plane at Qwen3-30B-A3B expert shapes (128 experts, top-8, hidden 2048, intermediate
768) instead and prints CUDA-event times (max over ranks) of the fused plane next to the NCCL plane
(all-gather of rows and routing, local grouped GEMMs, reduce-scatter)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    from vllm_torchtpu_b200.config import ParallelConfig
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    from vllm_torchtpu_b200.parallel import communicator
    from vllm_torchtpu_b200.parallel.state import init_distributed

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    pc = ParallelConfig(tensor_parallel_size=world, world_size=world, rank=rank,
                        local_rank=int(os.environ["LOCAL_RANK"]), enable_expert_parallel=True)
    st = init_distributed(pc, backend="nccl", timeout_s=120)
    dev = torch.device("cuda", st.local_rank)
    timing = "--timing" in sys.argv
    E, k, H, I, T_max = (128, 8, 2048, 768, 2048) if timing else (16, 4, 512, 256, 256)
    heap = communicator.ensure_ep_heap(T_max, k, H, I, E)
    assert heap is not None and heap.ep_state is not None
    e_local = E // world
    g = torch.Generator(device=dev).manual_seed(7)          # same weights on every rank
    w13 = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, I, device=dev, generator=g) * 0.05).bfloat16()
    lo = rank * e_local
    w13_l, w2_l = w13[lo:lo + e_local].contiguous(), w2[lo:lo + e_local].contiguous()
    ok = True
    if timing:
        ok = _timing(cuda, dist, heap, dev, rank, world, E, k, H, I, w13, w2, w13_l, w2_l, lo, ref)
        t = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if rank == 0:
            print("EP_TIMING_OK" if int(t.item()) == 1 else "EP_TIMING_FAIL", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if int(t.item()) == 1 else 1)
    for it, T in enumerate([37 + 11 * rank, 1, 200 - 50 * rank, 0 if rank == 0 else 5, 256]):
        gr = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(T, H, device=dev, generator=gr).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gr)
        topk_w, topk_ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        topk_ids = topk_ids.to(torch.int32).contiguous()
        topk_w = topk_w.float().contiguous()
        for rep in range(2):
            # the bounded flag waits of the plane are short in tests: start every call together, so that
            # one rank's lazy set-up (tensor maps, kernel attributes) does not run into the peers' limit
            torch.cuda.synchronize()
            dist.barrier()
            y = cuda.moe_experts_ep(x, w13_l, w2_l, topk_ids, topk_w, heap, E)
        torch.cuda.synchronize()
        status = cuda.check_status()
        want = ref.moe_experts(x, w13, w2, topk_ids, topk_w, 0) if T else y
        err = (y.float() - want.float()).abs().max().item() if T else 0.0
        tol = 3e-2 * (want.float().abs().max().item() if T else 1.0) + 2e-2
        if err > tol or status != 0:
            ok = False
            print(f"[rank {rank}] moe_experts_ep T={T}: err {err} tol {tol} status {status}", flush=True)
    # fp8 experts on the same plane (quantised rows, grouped fp8 GEMMs, routed epilogue) against the
    # single-rank fp8 pipeline over all experts
    from vllm_torchtpu_b200.ops.cuda_fp8 import moe_experts_fp8
    from vllm_torchtpu_b200.quantization.fp8 import quantize_weight_block
    q13, s13, q2, s2 = [], [], [], []
    for e in range(E):
        a, b = quantize_weight_block(w13[e])
        c, d = quantize_weight_block(w2[e])
        q13.append(a); s13.append(b); q2.append(c); s2.append(d)
    q13, s13, q2, s2 = torch.stack(q13), torch.stack(s13), torch.stack(q2), torch.stack(s2)
    lq13, ls13 = q13[lo:lo + e_local].contiguous(), s13[lo:lo + e_local].contiguous()
    lq2, ls2 = q2[lo:lo + e_local].contiguous(), s2[lo:lo + e_local].contiguous()
    for it, T in enumerate([1, 7 + rank, 64, 200 - 13 * rank, T_max]):
        gr = torch.Generator(device=dev).manual_seed(500 * it + rank)
        x = torch.randn(T, H, device=dev, generator=gr).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gr)
        topk_w, topk_ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        topk_ids = topk_ids.to(torch.int32).contiguous()
        topk_w = topk_w.float().contiguous()
        want = moe_experts_fp8(x, q13, s13, q2, s2, topk_ids, topk_w, 0)
        for rep in range(2):
            torch.cuda.synchronize()
            dist.barrier()
            got = cuda.moe_experts_ep_fp8(x, lq13, ls13, lq2, ls2, topk_ids, topk_w, heap, E)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        tol = 3e-2 * want.float().abs().max().item() + 2e-2
        status = cuda.check_status()
        if err > tol or status != 0:
            ok = False
            print(f"[rank {rank}] moe_experts_ep_fp8 T={T}: err {err} tol {tol} status {status}", flush=True)
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EP_FUSED_OK" if int(t.item()) == 1 else "EP_FUSED_FAIL", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 1 else 1)


def _timing(cuda, dist, heap, dev, rank, world, E, k, H, I, w13, w2, w13_l, w2_l, lo, ref) -> bool:
    from vllm_torchtpu_b200.ops.cuda_moe import moe_experts
    ok = True
    for T in (64, 512, 2048):
        gr = torch.Generator(device=dev).manual_seed(900 + rank)
        x = torch.randn(T, H, device=dev, generator=gr).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=gr)
        topk_w, topk_ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        topk_ids, topk_w = topk_ids.to(torch.int32).contiguous(), topk_w.float().contiguous()

        def fused():
            return cuda.moe_experts_ep(x, w13_l, w2_l, topk_ids, topk_w, heap, E)

        def nccl_plane():
            gx = torch.empty(world * T, H, dtype=x.dtype, device=dev)
            gi = torch.empty(world * T, k, dtype=topk_ids.dtype, device=dev)
            gw = torch.empty(world * T, k, dtype=topk_w.dtype, device=dev)
            dist.all_gather_into_tensor(gx, x)
            dist.all_gather_into_tensor(gi, topk_ids)
            dist.all_gather_into_tensor(gw, topk_w)
            y = moe_experts(gx, w13_l, w2_l, gi, gw, lo)
            out = torch.empty(T, H, dtype=y.dtype, device=dev)
            dist.reduce_scatter_tensor(out, y)
            return out

        def timed(fn, iters=20):
            for _ in range(3):
                torch.cuda.synchronize()
                dist.barrier()
                fn()
            ts = []
            for _ in range(iters):
                torch.cuda.synchronize()
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b) * 1e3)
            t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        y = fused()
        torch.cuda.synchronize()
        want = ref.moe_experts(x, w13, w2, topk_ids, topk_w, 0)
        err = (y.float() - want.float()).abs().max().item()
        tol = 3e-2 * want.float().abs().max().item() + 2e-2
        y2 = nccl_plane()
        err2 = (y2.float() - want.float()).abs().max().item()
        t_f, t_n = timed(fused), timed(nccl_plane)
        # phases of one fused call and of the local expert pipeline of the NCCL plane
        torch.cuda.synchronize()
        dist.barrier()
        ev = []
        cuda.moe_experts_ep(x, w13_l, w2_l, topk_ids, topk_w, heap, E, phase_events=ev)
        torch.cuda.synchronize()
        ph = [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(len(ev) - 1)]
        gx = torch.cat([x] * world)
        gi, gw = torch.cat([topk_ids] * world), torch.cat([topk_w] * world)
        t_local = timed(lambda: moe_experts(gx, w13_l, w2_l, gi, gw, lo))
        if rank == 0:
            print(f"PHASES EP T={T}: dispatch {ph[0]:.1f} us, first GEMM {ph[1]:.1f} us, routed GEMM {ph[2]:.1f} us, "
                  f"combine {ph[3]:.1f} us; local experts of the NCCL plane (permute, 2 GEMMs, un-permute) "
                  f"{t_local:.1f} us", flush=True)
        status = cuda.check_status()
        ok = ok and err <= tol and err2 <= tol and status == 0
        if rank == 0:
            # bytes a rank sends: T*k rows of H bf16 out (minus the share it owns) and as many back
            nv = 2 * T * k * H * 2 * (world - 1) / world
            print(f"TIMING EP world={world} T={T}/rank E={E} k={k} H={H} I={I}: fused plane {t_f:.1f} us, "
                  f"all-gather + local experts + reduce-scatter {t_n:.1f} us; NVLink bytes per rank "
                  f"{nv / 1e6:.2f} MB; err {err:.4f} / {err2:.4f} tol {tol:.4f} status {status}", flush=True)
    return ok


if __name__ == "__main__":
    import faulthandler
    faulthandler.dump_traceback_later(100, exit=True)
    main()
