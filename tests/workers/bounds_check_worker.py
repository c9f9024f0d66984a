"""Child process: tiny attention cases on the bounds-checked library.  A healthy block table leaves the
violation counter at zero; a table with an id outside the pool is clamped (no fault) and counted."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ["B200_BOUNDS_CHECK"] = "1"


def main():
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata
    dev = "cuda"
    Hq, Hkv, D, bs, nb = 8, 2, 128, 16, 64
    g = torch.Generator(device=dev).manual_seed(0)
    kv = (torch.randn(nb, 2, Hkv, bs, D, device=dev, generator=g) * 0.5).bfloat16()
    seq = [37, 150, 16]
    R = len(seq)
    max_blocks = 16
    bt = torch.zeros(R, max_blocks, dtype=torch.int32, device=dev)
    nxt = 1
    for r, n in enumerate(seq):
        for i in range(-(-n // bs)):
            bt[r, i] = nxt
            nxt += 1
    qsl = torch.arange(R + 1, dtype=torch.int32, device=dev)
    sl = torch.tensor(seq, dtype=torch.int32, device=dev)
    meta = AttentionMetadata(positions=torch.tensor([n - 1 for n in seq], dtype=torch.int32, device=dev),
                             slot_mapping=torch.zeros(R, dtype=torch.int32, device=dev), block_tables=bt,
                             seq_lens=sl, query_start_loc=qsl, num_reqs=R, num_tokens=R, num_decode_reqs=R,
                             max_query_len=1, max_seq_len=max(seq), seq_lens_cpu=sl.cpu(),
                             query_start_loc_cpu=qsl.cpu())
    q = torch.randn(R, Hq, D, device=dev, generator=g).bfloat16()
    cuda.bad_index_count()
    out = cuda.paged_attention(q, kv, meta, D ** -0.5)
    torch.cuda.synchronize()
    want = ref.paged_attention(q, kv, bt, meta.seq_lens, qsl, D ** -0.5, num_reqs=R)
    err = (out.float() - want.float()).abs().max().item()
    clean = cuda.bad_index_count()
    bt[1, 3] = nb + 5                          # an id outside the pool
    cuda.paged_attention(q, kv, meta, D ** -0.5)
    torch.cuda.synchronize()
    dirty = cuda.bad_index_count()
    again = cuda.bad_index_count()
    print(f"RESULT err={err:.4f} clean={clean} dirty={dirty} again={again} status={cuda.check_status()}")
    ok = err < 0.03 and clean == 0 and dirty > 0 and again == 0
    print("BOUNDS_OK" if ok else "BOUNDS_FAIL")


if __name__ == "__main__":
    main()
