"""Child process: a tiny Llama checkpoint served by ``vllm.LLM`` through the b200 platform plugin
(attention backend, custom-op providers) and by this package's native engine; prints both token lists."""
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    import faulthandler
    faulthandler.dump_traceback_later(280, exit=True)
    tmp = tempfile.mkdtemp(prefix="b200_vllm_")
    # what an installed copy of the package looks like to importlib.metadata
    di = os.path.join(tmp, "site", "vllm_torchtpu_b200-0.1.0.dist-info")
    os.makedirs(di)
    with open(os.path.join(di, "METADATA"), "w") as f:
        f.write("Metadata-Version: 2.1\nName: vllm-torchtpu-b200\nVersion: 0.1.0\n")
    with open(os.path.join(di, "entry_points.txt"), "w") as f:
        f.write("[vllm.platform_plugins]\nb200 = vllm_torchtpu_b200.vllm_plugin:register_platform\n\n"
                "[vllm.general_plugins]\nb200 = vllm_torchtpu_b200.vllm_plugin:register_general\n")
    sys.path.insert(0, os.path.join(tmp, "site"))
    os.environ["PYTHONPATH"] = os.pathsep.join([ROOT, os.path.join(tmp, "site"), os.environ.get("PYTHONPATH", "")])
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_PLUGINS", "b200")

    import numpy as np
    import torch
    from vllm_torchtpu_b200 import SamplingParams as NativeSP
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.engine.llm import LLM as NativeLLM
    from vllm_torchtpu_b200.models.loader import save_hf_checkpoint
    from vllm_torchtpu_b200.ops import launch_count

    cfg = ModelConfig(name="plugin-llama", num_layers=2, hidden_size=1024, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=2048, vocab_size=4096, max_model_len=512, dtype=torch.bfloat16,
                      rope_theta=10000.0, init_std=0.05)
    native = NativeLLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=128,
                       init_dist=False)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, 4096, size=n).tolist() for n in (8, 33, 70)]
    want = [o.outputs[0].token_ids for o in native.generate(prompts, NativeSP(temperature=0.0, max_tokens=8,
                                                                               ignore_eos=True))]
    ckpt = os.path.join(tmp, "ckpt")
    hf = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 1024,
          "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 2048,
          "vocab_size": 4096, "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": 10000.0, "max_position_embeddings": 512,
          "torch_dtype": "bfloat16", "hidden_act": "silu", "tie_word_embeddings": False, "bos_token_id": 1,
          "eos_token_id": 2}
    save_hf_checkpoint(native.engine.runner.model, ckpt, hf)
    del native
    torch.cuda.empty_cache()

    import vllm
    from vllm.platforms import current_platform
    platform_name = type(current_platform).__name__
    c0 = launch_count()
    llm = vllm.LLM(model=ckpt, skip_tokenizer_init=True, dtype="bfloat16", enforce_eager=True, max_model_len=512,
                   gpu_memory_utilization=0.25, block_size=16, max_num_seqs=8, enable_prefix_caching=False)
    sp = vllm.SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, detokenize=False)
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp)
    got = [list(o.outputs[0].token_ids) for o in outs]
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    print("RESULT " + json.dumps({"platform": platform_name, "want": want, "got": got,
                                  "backend": AttentionBackendEnum.CUSTOM.get_path(),
                                  "b200_launches": launch_count() - c0}), flush=True)


if __name__ == "__main__":
    main()
