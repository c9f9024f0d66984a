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
    heap = communicator.ensure_tp_heap(8192, 4096)
    assert heap is not None and heap.fused_tp is not None
    ok = True
    ft = heap.fused_tp
    one_shot_default = ft.one_shot_bytes

    def owner_mask(T, N):
        """[T, N] bool: elements of the output tiles this rank owns (tile % world == rank)."""
        bn = 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
        n_tiles, t_tiles = -(-N // 128), -(-T // bn)
        m = torch.zeros(T, N, dtype=torch.bool, device=dev)
        per_group = 16 * t_tiles
        for tile in range(n_tiles * t_tiles):
            g = tile // per_group
            first_n = g * 16
            gsize = min(16, n_tiles - first_n)
            r = tile - g * per_group
            n_tile, t_tile = first_n + r % gsize, r // gsize
            if tile % world == rank:
                m[t_tile * bn:(t_tile + 1) * bn, n_tile * 128:(n_tile + 1) * 128] = True
        return m

    shapes = [(16, 512, 256), (64, 4096, 512), (64, 4096, 1792), (300, 1024, 512), (1000, 2048, 1024),
              (2048, 4096, 512)]
    # plane: one-shot where the default threshold allows it, then everything through tile owners
    for one_shot in (one_shot_default, 0):
        ft.one_shot_bytes = one_shot
        for (T, N, K) in shapes:
            g = torch.Generator(device=dev).manual_seed(1000 * rank + T)
            x = torch.randn(T, K, device=dev, generator=g).bfloat16()
            w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
            want = x.float() @ w.float().t()
            dist.all_reduce(want)
            tol = 3e-2 * want.abs().max().item() + 2e-2
            for mode in (0, 1):
                for rep in range(3):                  # repeated launches reuse flags with growing epochs
                    y = cuda.gemm_all_reduce(x, w, heap, mode=mode).clone()
                torch.cuda.synchronize()
                diff = (y.float() - want).abs()
                if mode == 1:
                    diff = diff[owner_mask(T, N)]
                err = diff.max().item() if diff.numel() else 0.0
                status = cuda.check_status()
                if err > tol or status != 0:
                    ok = False
                    print(f"[rank {rank}] gemm_all_reduce {(T, N, K)} mode {mode} one_shot {one_shot}: "
                          f"err {err} tol {tol} status {status}", flush=True)
    ft.one_shot_bytes = one_shot_default

    # push plane: partials pushed to every rank, summed inside the add + RMSNorm consumer
    for (T, N, K) in [(1, 512, 256), (16, 512, 256), (64, 4096, 512), (64, 4096, 1792), (200, 1024, 512)]:
        assert ft.can_push(T, N)
        g = torch.Generator(device=dev).manual_seed(77 * rank + T)
        x = torch.randn(T, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
        g2 = torch.Generator(device=dev).manual_seed(5)
        res0 = torch.randn(T, N, device=dev, generator=g2).bfloat16()
        nw = (1 + 0.1 * torch.randn(N, device=dev, generator=g2)).bfloat16()
        part = (x.float() @ w.float().t()).bfloat16().float()
        dist.all_reduce(part)
        want_sum = part.bfloat16()
        want_res = (want_sum.float() + res0.float()).bfloat16()
        want_y = cuda.rms_norm(want_res, nw, 1e-5)
        for rep in range(3):
            res = res0.clone()
            y, res_out = cuda.gemm_push(x, w, heap).add_rms_norm(res, nw, 1e-5)
            s_only = cuda.gemm_push(x, w, heap).materialize()
        torch.cuda.synchronize()
        e1 = (y.float() - want_y.float()).abs().max().item()
        e2 = (res_out.float() - want_res.float()).abs().max().item()
        e3 = (s_only.float() - want_sum.float()).abs().max().item()
        tol = 3e-2 * max(1.0, want_res.float().abs().max().item())
        if max(e1, e2, e3) > tol or cuda.check_status() != 0:
            ok = False
            print(f"[rank {rank}] gemm_push {(T, N, K)}: y {e1} residual {e2} sum {e3} tol {tol} "
                  f"status {cuda.check_status()}", flush=True)

    # fp8 push plane: block-scaled e4m3 weights, partial pushed from the epilogue (token tiles 32 / 64 /
    # 128, cluster split-K and plain), alternating with bf16 push launches on the same control block
    from vllm_torchtpu_b200.quantization.fp8 import fp8_block_gemm_reference, quantize_weight_block
    for (T, N, K) in [(1, 512, 256), (16, 1024, 512), (48, 4096, 1792), (64, 4096, 512), (128, 2048, 1024)]:
        assert ft.can_push(T, N)
        g = torch.Generator(device=dev).manual_seed(91 * rank + T)
        x = torch.randn(T, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
        wq, wsi = quantize_weight_block(w)
        part = fp8_block_gemm_reference(x, wq, wsi).float()
        dist.all_reduce(part)
        for rep in range(3):
            got = cuda.fp8_block_gemm_push(x, wq, wsi, heap).materialize()
            cuda.gemm_push(x, w, heap).materialize()
        torch.cuda.synchronize()
        err = (got.float() - part).abs().max().item()
        tol = 3e-2 * part.abs().max().item() + 2e-2
        if err > tol or cuda.check_status() != 0:
            ok = False
            print(f"[rank {rank}] fp8_block_gemm_push {(T, N, K)}: err {err} tol {tol} "
                  f"status {cuda.check_status()}", flush=True)

    # all-gather -> GEMM: row-sharded activations, gathered inside the column-parallel GEMM
    for (T_loc, N, K) in [(32, 512, 256), (64, 1536, 4096), (256, 1024, 512), (1024, 3584, 4096)]:
        g = torch.Generator(device=dev).manual_seed(31 * rank + T_loc)
        x_loc = torch.randn(T_loc, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
        gathered = [torch.empty_like(x_loc) for _ in range(world)]
        dist.all_gather(gathered, x_loc)
        want = torch.cat(gathered, 0).float() @ w.float().t()
        for rep in range(3):
            y = cuda.gemm_all_gather(x_loc, w, heap)
        torch.cuda.synchronize()
        err = (y.float() - want).abs().max().item()
        tol = 3e-2 * want.abs().max().item() + 2e-2
        status = cuda.check_status()
        if err > tol or status != 0:
            ok = False
            print(f"[rank {rank}] gemm_all_gather {(T_loc, N, K)}: err {err} tol {tol} status {status}", flush=True)
    for (T_loc, N, K) in [(8192 // world, 6144 // world, 4096), (8192 // world, 28672 // world, 4096)]:
        x_loc = torch.randn(T_loc, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
        gathered = torch.empty(T_loc * world, K, device=dev, dtype=torch.bfloat16)

        def plain_ag(x_loc=x_loc, w=w, gathered=gathered):
            dist.all_gather_into_tensor(gathered, x_loc)
            return cuda.gemm(gathered, w)
        # timed further down, once the timing helper exists
        globals().setdefault("_AG_CASES", []).append((x_loc, w, gathered, plain_ag, T_loc, N, K))

    # device time of the fused kernel next to GEMM + NCCL all-reduce (information only)
    def timed(fn, iters=20):
        for _ in range(5):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for (T, N, K) in [(64, 4096, 4096 // world), (64, 4096, 14336 // world), (8192, 4096, 4096 // world),
                      (8192, 4096, 14336 // world)]:
        x = torch.randn(T, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()

        def plain():
            y = cuda.gemm(x, w)
            dist.all_reduce(y)
            return y
        t_push = -1.0
        if ft.can_push(T, N):
            res = torch.zeros(T, N, device=dev, dtype=torch.bfloat16)
            nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
            t_push = timed(lambda: cuda.gemm_push(x, w, heap).add_rms_norm(res, nw, 1e-5))
            t_norm = timed(lambda: cuda.fused_add_rms_norm(res, res, nw, 1e-5))
            if rank == 0:
                print(f"TIMING T={T} N={N} K={K}: push gemm + reduce/add/norm {t_push:.1f} us "
                      f"(plain add+norm alone {t_norm:.1f} us)", flush=True)
            if T <= 128:
                wq, wsi = quantize_weight_block(w)

                def plain_fp8():
                    y = cuda.fp8_block_gemm(x, wq, wsi)
                    dist.all_reduce(y)
                    return cuda.fused_add_rms_norm(y, res, nw, 1e-5)
                t_f8 = timed(lambda: cuda.fp8_block_gemm_push(x, wq, wsi, heap).add_rms_norm(res, nw, 1e-5))
                t_f8_plain = timed(plain_fp8)
                if rank == 0:
                    print(f"TIMING fp8 T={T} N={N} K={K}: push gemm + reduce/add/norm {t_f8:.1f} us, "
                          f"fp8 gemm + nccl + add/norm {t_f8_plain:.1f} us", flush=True)
        t_fused = timed(lambda: cuda.gemm_all_reduce(x, w, heap))
        t_nccl = timed(plain)
        t_gemm = timed(lambda: cuda.gemm(x, w))
        if rank == 0:
            print(f"TIMING T={T} N={N} K={K} world={world}: fused {t_fused:.1f} us, gemm+nccl {t_nccl:.1f} us, "
                  f"gemm alone {t_gemm:.1f} us, status {cuda.check_status()}", flush=True)
    for (x_loc, w, gathered, plain_ag, T_loc, N, K) in globals().get("_AG_CASES", []):
        t_fused = timed(lambda: cuda.gemm_all_gather(x_loc, w, heap))
        t_plain = timed(plain_ag)
        t_gemm = timed(lambda: cuda.gemm(gathered, w))
        if rank == 0:
            print(f"TIMING all-gather->GEMM T_loc={T_loc} N={N} K={K} world={world}: fused {t_fused:.1f} us, "
                  f"nccl all-gather + gemm {t_plain:.1f} us, gemm alone {t_gemm:.1f} us, "
                  f"status {cuda.check_status()}", flush=True)
    if cuda.check_status() != 0:
        ok = False
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
