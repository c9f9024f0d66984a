"""MoE kernels and the SwiGLU / grouped tcgen05 GEMM variants vs PyTorch fp32."""
import pytest
import torch

from vllm_torchtpu_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cu():
    from vllm_torchtpu_b200.ops import cuda
    return cuda


@pytest.mark.parametrize("T,I,K", [(16, 256, 512), (64, 1536, 2048), (200, 768, 1024), (1000, 512, 512),
                                   (64, 1792, 4096), (64, 7168, 4096), (33, 3584, 4096), (5, 640, 4096),
                                   (64, 14336, 4096), (48, 11008, 2048), (128, 12000, 1024)])
def test_gemm_swiglu(T, I, K):
    g = torch.Generator(device=DEV).manual_seed(T)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV, generator=g) * 0.05).bfloat16()
    y = cu().gemm_swiglu(x, w)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    h = x.float() @ w.float().t()
    want = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("scoring,E,k,ng,tg,bias", [("softmax", 128, 8, 1, 1, False),
                                                   ("sigmoid", 256, 8, 8, 4, True),
                                                   ("softmax", 8, 2, 1, 1, False),
                                                   ("sigmoid", 64, 6, 4, 2, False)])
def test_moe_route(scoring, E, k, ng, tg, bias):
    T = 77
    g = torch.Generator(device=DEV).manual_seed(0)
    logits = torch.randn(T, E, device=DEV, generator=g)
    b = (torch.randn(E, device=DEV, generator=g) * 0.1) if bias else None
    kw = dict(scoring=scoring, renormalize=True, routed_scaling=2.5, score_bias=b, n_group=ng, topk_group=tg)
    ids, w = cu().moe_route(logits, k, **kw)
    rid, rw = ref.moe_route(logits, k, **kw)
    # compare as sets per token (order of equal-rank picks may differ)
    got = torch.zeros(T, E, device=DEV).scatter_(1, ids.long(), w)
    want = torch.zeros(T, E, device=DEV).scatter_(1, rid.long(), rw)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("T,E,k,H,I,lo,El", [(64, 8, 2, 256, 128, 0, 8), (300, 16, 4, 512, 256, 0, 16),
                                             (33, 128, 8, 2048, 768, 0, 128), (50, 16, 4, 256, 128, 4, 8),
                                             (1, 8, 2, 256, 128, 0, 8)])
def test_moe_experts_matches_reference(T, E, k, H, I, lo, El):
    g = torch.Generator(device=DEV).manual_seed(T + E)
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w13 = (torch.randn(El, 2 * I, H, device=DEV, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(El, H, I, device=DEV, generator=g) * 0.05).bfloat16()
    logits = torch.randn(T, E, device=DEV, generator=g)
    ids, w = ref.moe_route(logits, k)
    got = cu().moe_experts(x, w13, w2, ids, w, lo)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    want = ref.moe_experts(x, w13, w2, ids, w, lo)
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 3e-2 * want.float().abs().max().item() + 1e-2, err


def test_tiny_moe_engine_on_gpu():
    import numpy as np
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.engine.llm import LLM
    cfg = ModelConfig(name="moe", architecture="qwen3_moe", qk_norm=True, num_layers=2, hidden_size=512,
                      num_q_heads=8, num_kv_heads=2, head_dim=128, vocab_size=2048, max_model_len=256,
                      num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, dtype=torch.bfloat16)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, 2048, size=n).tolist() for n in (9, 40, 70)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    kw = dict(device="cuda", max_num_seqs=8, max_num_batched_tokens=128, num_gpu_blocks_override=256,
              init_dist=False)
    eager = [o.outputs[0].token_ids for o in LLM(cfg, enforce_eager=True, **kw).generate(prompts, sp)]
    graph = [o.outputs[0].token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    assert eager == graph
    assert cu().check_status() == 0


@pytest.mark.parametrize("sim", ["", "uniform", "hash"])
def test_route_post_kernel_matches_reference(sim):
    from vllm_torchtpu_b200.ops import reference as ref
    g = torch.Generator(device=DEV).manual_seed(0)
    T, k, E = 77, 8, 128
    ids = torch.randint(0, E, (T, k), device=DEV, generator=g, dtype=torch.int32)
    w = torch.rand(T, k, device=DEV, generator=g)
    nv = torch.tensor([50], dtype=torch.int32, device=DEV)
    want_ids, want_w = ref.moe_route_post(ids.cpu().clone(), w.cpu().clone(), E, nv.cpu(), sim)
    got_ids, got_w = cu().moe_route_post(ids, w, E, nv, sim)
    assert torch.equal(got_ids.cpu(), want_ids)
    torch.testing.assert_close(got_w.cpu(), want_w)
    # masked pairs drop out of the expert pipeline
    x = torch.randn(T, 256, device=DEV, generator=g).bfloat16()
    w13 = (torch.randn(E, 256, 256, device=DEV, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, 256, 128, device=DEV, generator=g) * 0.05).bfloat16()
    y = cu().moe_experts(x, w13, w2, got_ids, got_w, 0)
    torch.cuda.synchronize()
    assert not y[50:].float().abs().sum().item() and cu().check_status() == 0
    want = ref.moe_experts(x, w13, w2, got_ids, got_w, 0)
    assert (y.float() - want.float()).abs().max().item() <= 3e-2 * want.float().abs().max().item() + 2e-2


@pytest.mark.parametrize("packed", [False, True])
def test_experts_with_biases_oai_swiglu_and_padded_hidden(packed):
    """GPT-OSS style experts on the device: expert biases through the grouped bias kernel, the OAI SwiGLU kernel,
    a hidden size (192) below the down projection's padded 256 rows; bf16 experts and packed mxfp4 experts."""
    cu()                                             # the kernel module first: it pulls in its sub-modules itself
    from vllm_torchtpu_b200.ops import cuda_fp4
    from vllm_torchtpu_b200.ops import reference as ref
    from vllm_torchtpu_b200.quantization.fp4 import dequantize_mxfp4, quantize_mxfp4
    g = torch.Generator(device=DEV).manual_seed(2)
    T, H, Hp, I, E, k = 45, 192, 256, 128, 8, 2
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.08).bfloat16()
    w2 = torch.zeros(E, Hp, I, device=DEV, dtype=torch.bfloat16)
    w2[:, :H] = (torch.randn(E, H, I, device=DEV, generator=g) * 0.08).bfloat16()
    b13 = (torch.randn(E, 2 * I, device=DEV, generator=g) * 0.1).bfloat16()
    b2 = torch.zeros(E, Hp, device=DEV, dtype=torch.bfloat16)
    b2[:, :H] = (torch.randn(E, H, device=DEV, generator=g) * 0.1).bfloat16()
    logits = torch.randn(T, E, device=DEV, generator=g)
    wt, ids = torch.topk(torch.softmax(logits, -1), k, -1)
    ids, wt = ids.int().contiguous(), wt.float().contiguous()
    act = "swigluoai:1.702:7.0"
    if packed:
        q13 = [quantize_mxfp4(w13[e].float()) for e in range(E)]
        q2 = [quantize_mxfp4(w2[e].float()) for e in range(E)]
        w13q, s13 = torch.stack([a for a, _ in q13]), torch.stack([b for _, b in q13])
        w2q, s2 = torch.stack([a for a, _ in q2]), torch.stack([b for _, b in q2])
        got = cuda_fp4.moe_experts_w4a16(x, w13q, s13, w2q, s2, ids, wt, 0, "mxfp4", act=act, b13=b13, b2=b2)
        w13 = torch.stack([dequantize_mxfp4(w13q[e], s13[e]) for e in range(E)]).bfloat16()
        w2 = torch.stack([dequantize_mxfp4(w2q[e], s2[e]) for e in range(E)]).bfloat16()
    else:
        got = cu().moe_experts(x, w13, w2, ids, wt, 0, act=act, b13=b13, b2=b2)
    torch.cuda.synchronize()
    assert got.shape == (T, H) and cu().check_status() == 0
    want = ref.moe_experts(x, w13, w2, ids, wt, 0, act=act, b13=b13, b2=b2)
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 3e-2 * want.float().abs().max().item() + 2e-2, err
