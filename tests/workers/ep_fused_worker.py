"""Child process of the multi-GPU tests: the fused expert-parallel plane (NVLink dispatch, grouped
tcgen05 GEMMs, combine in the GEMM epilogue) against a dense fp32 MoE of the same tokens.  Every rank
holds E / world experts and brings its own tokens (a different count on every rank)."""
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
    E, k, H, I, T_max = 16, 4, 512, 256, 256
    heap = communicator.ensure_ep_heap(T_max, k, H, I, E)
    assert heap is not None and heap.ep_state is not None
    e_local = E // world
    g = torch.Generator(device=dev).manual_seed(7)          # same weights on every rank
    w13 = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, I, device=dev, generator=g) * 0.05).bfloat16()
    lo = rank * e_local
    w13_l, w2_l = w13[lo:lo + e_local].contiguous(), w2[lo:lo + e_local].contiguous()
    ok = True
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


if __name__ == "__main__":
    import faulthandler
    faulthandler.dump_traceback_later(100, exit=True)
    main()
