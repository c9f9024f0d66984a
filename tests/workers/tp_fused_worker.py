"""Child process of the multi-GPU tests (launched by torch.distributed.run, one rank per GPU):
fused row-parallel GEMM + reduction over peer memory vs NCCL, peer all-reduce vs NCCL, and a
TP engine run with the fused plane vs the NCCL plane."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    from vllm_torchtpu_b200.config import ParallelConfig
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.parallel import communicator
    from vllm_torchtpu_b200.parallel.state import init_distributed

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    pc = ParallelConfig(tensor_parallel_size=world, world_size=world, rank=rank,
                        local_rank=int(os.environ["LOCAL_RANK"]))
    st = init_distributed(pc, backend="nccl", timeout_s=120)
    dev = torch.device("cuda", st.local_rank)
    heap = communicator.ensure_tp_heap(1024, 4096)
    assert heap is not None and heap.fused_tp is not None
    ok = True
    for (T, N, K) in [(16, 512, 256), (64, 4096, 512), (64, 4096, 1792), (300, 1024, 512), (1000, 2048, 1024)]:
        g = torch.Generator(device=dev).manual_seed(1000 * rank + T)
        x = torch.randn(T, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
        for rep in range(3):                      # repeated launches reuse flags with growing epochs
            y = cuda.gemm_all_reduce(x, w, heap).clone()
        torch.cuda.synchronize()
        want = x.float() @ w.float().t()
        dist.all_reduce(want)
        err = (y.float() - want).abs().max().item()
        tol = 3e-2 * want.abs().max().item() + 2e-2
        status = cuda.check_status()
        if err > tol or status != 0:
            ok = False
            print(f"[rank {rank}] gemm_all_reduce {(T, N, K)}: err {err} tol {tol} status {status}", flush=True)
    # stand-alone peer all-reduce
    for n in (8, 4096, 1 << 20):
        g = torch.Generator(device=dev).manual_seed(rank + n)
        x = torch.randn(n, device=dev, generator=g).bfloat16()
        want = x.float().clone()
        dist.all_reduce(want)
        got = cuda.p2p_all_reduce(x.clone(), heap)
        torch.cuda.synchronize()
        err = (got.float() - want).abs().max().item()
        if err > 2e-2 * want.abs().max().item() + 2e-2 or cuda.check_status() != 0:
            ok = False
            print(f"[rank {rank}] p2p_all_reduce n={n}: err {err}", flush=True)
    t = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_FUSED_OK" if int(t.item()) == 1 else "TP_FUSED_FAIL", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(t.item()) == 1 else 1)


if __name__ == "__main__":
    main()
