"""Child process of the two-GPU KV-transfer test: rank 0 owns a paged pool on GPU 0 and exports it through
CUDA IPC; rank 1 maps it and pulls blocks into its own pool on GPU 1 with one kernel (NVLink peer loads),
screens them for NaN and checks the bytes.  The ranks meet on a gloo group; nobody leaves mid-transfer."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler
    faulthandler.dump_traceback_later(100, exit=True)
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=2)
    torch.cuda.set_device(rank)
    from vllm_torchtpu_b200.kv_transfer.transport import IpcTransport, nan_blocks
    from vllm_torchtpu_b200.ops import cuda
    dev = torch.device("cuda", rank)
    shape = (2, 2, 16, 128)
    layers, nb = 4, 24
    g = torch.Generator(device=dev).manual_seed(123)
    # small tensors share one allocator segment: the exported offsets matter
    pool = [torch.randn((nb,) + shape, device=dev, generator=g).bfloat16() if rank == 0 else
            torch.zeros((nb,) + shape, dtype=torch.bfloat16, device=dev) for _ in range(layers)]
    tr = IpcTransport(f"engine{rank}")
    tr.register_pool(pool)
    infos = [None, None]
    dist.all_gather_object(infos, tr.export())
    ok = True
    if rank == 1:
        tr.open_remote(infos[0])
        src_ids, dst_ids = [0, 5, 23, 7, 11], [3, 4, 0, 22, 9]
        tr.pull("engine0", src_ids, dst_ids)
        torch.cuda.synchronize()
        g0 = torch.Generator(device=dev).manual_seed(123)
        want = [torch.randn((nb,) + shape, device=dev, generator=g0).bfloat16() for _ in range(layers)]
        for got, w in zip(pool, want):
            ok &= bool(torch.equal(got[dst_ids], w[src_ids]))
        ok &= nan_blocks(tr.local, dst_ids) == []
        ok &= cuda.check_status(dev) == 0
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    if rank == 0:
        print("IPC_PULL_OK" if int(flag) == 1 else "IPC_PULL_FAILED", flush=True)
    dist.barrier()
    from vllm_torchtpu_b200.parallel.state import leave_process
    leave_process(0)


if __name__ == "__main__":
    main()
