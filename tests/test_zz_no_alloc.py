"""The allocation-free decode-attention entry point, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the
library in the same process; it must pass alone as well.  The test itself allocates its
inputs with torch; the entry point under test allocates nothing."""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from vllm_torchtpu_b200.ops import cuda
    L = cuda.lib()
    L.b200_attn_decode_static.restype = c_int
    L.b200_attn_decode_static_setup.restype = c_int
    L.b200_attn_decode_static_reset.restype = c_int
    return L


def _p(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _case(ctx_lens, Hq, Hkv, D, bs=16, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    R = len(ctx_lens)
    seq = [c + 1 for c in ctx_lens]
    maxb = max(-(-s // bs) for s in seq) + 1
    nb = sum(-(-s // bs) for s in seq) + 2
    cache = (torch.randn(nb, 2, Hkv, bs, D, device=DEV, generator=g) * 0.5).bfloat16()
    perm = (torch.randperm(nb - 1, device=DEV, generator=g) + 1).to(torch.int32)
    bt = torch.zeros(R, maxb, dtype=torch.int32, device=DEV)
    off = 0
    for r, s in enumerate(seq):
        n = -(-s // bs)
        bt[r, :n] = perm[off:off + n]
        off += n
    q = torch.randn(R, Hq, D, device=DEV, generator=g).bfloat16()
    qsl = torch.arange(R + 1, dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    return q, cache, bt, sl, qsl, maxb, nb


def _existing(L, q, cache, bt, sl, qsl, maxb, nb, Hq, Hkv, D, splits):
    """The ordinary entry point, with caller-provided scratch and counters."""
    R = q.shape[0]
    L.b200_attn_decode_scratch_bytes.restype = ctypes.c_size_t
    need = L.b200_attn_decode_scratch_bytes(c_int(R), c_int(Hkv), c_int(splits), c_int(D))
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
    counters = torch.zeros(R * Hkv, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    lse = torch.full((R, Hq), float("-inf"), dtype=torch.float32, device=DEV)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.b200_attn_decode(_p(q), _p(cache), _p(out), _p(lse), _p(bt), _p(sl), _p(qsl), c_int(0), c_int(R),
                            c_int(maxb), c_int(cache.shape[3]), c_longlong(nb), c_int(Hq), c_int(Hkv), c_int(D),
                            c_float(D ** -0.5), c_int(0), c_float(0.0), c_void_p(0), c_int(splits), _p(scratch),
                            _p(counters), stream)
    assert rc == 0, L.b200_get_last_error().decode()
    torch.cuda.synchronize()
    return out, lse


def _static(L, q, cache, bt, sl, qsl, maxb, nb, Hq, Hkv, D, splits):
    R = q.shape[0]
    out = torch.zeros_like(q)
    lse = torch.full((R, Hq), float("-inf"), dtype=torch.float32, device=DEV)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.b200_attn_decode_static(_p(q), _p(cache), _p(out), _p(lse), _p(bt), _p(sl), _p(qsl), c_int(R),
                                   c_int(maxb), c_int(cache.shape[3]), c_longlong(nb), c_int(Hq), c_int(Hkv),
                                   c_int(D), c_float(D ** -0.5), c_int(0), c_float(0.0), c_void_p(0),
                                   c_int(splits), stream)
    return rc, out, lse


@pytest.mark.parametrize("Hq,Hkv,D,splits", [(32, 8, 128, 4), (8, 2, 64, 3)])
def test_static_scratch_decode_matches_existing_entry_point(Hq, Hkv, D, splits):
    from vllm_torchtpu_b200.ops import reference as ref
    L = _lib()
    assert L.b200_attn_decode_static_setup() == 0, L.b200_get_last_error().decode()
    # two calls in a row on different inputs: the second one finds the counters re-armed by the first
    for seed, ctx in ((0, [0, 15, 16, 100, 1023, 2500, 7]), (1, [700, 3, 64, 1999, 31])):
        args = _case(ctx, Hq, Hkv, D, seed=seed)
        want, want_lse = _existing(L, *args, Hq, Hkv, D, splits)
        rc, got, got_lse = _static(L, *args, Hq, Hkv, D, splits)
        assert rc == 0, L.b200_get_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got_lse, want_lse, rtol=1e-2, atol=1e-2)
        q, cache, bt, sl, qsl, _, _ = args
        oracle = ref.paged_attention(q, cache, bt, sl, qsl, D ** -0.5, num_reqs=q.shape[0])
        torch.testing.assert_close(got.float(), oracle.float(), rtol=2e-2, atol=2e-2)


def test_static_scratch_refuses_oversized_calls():
    L = _lib()
    Hq, Hkv, D = 32, 8, 128
    args = _case([40] * 40, Hq, Hkv, D)
    # 40 requests x 8 kv heads x 4 splits = 1280 partial tiles > the 1006 that fit at D = 128
    rc, _, _ = _static(L, *args, Hq, Hkv, D, 4)
    assert rc == -1
    assert "built-in scratch" in L.b200_get_last_error().decode()
    # the same batch without splitting needs no scratch and runs
    rc, got, _ = _static(L, *args, Hq, Hkv, D, 1)
    assert rc == 0, L.b200_get_last_error().decode()
    want, _ = _existing(L, *args, Hq, Hkv, D, 1)
    torch.cuda.synchronize()
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    assert L.b200_attn_decode_static_reset(c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
