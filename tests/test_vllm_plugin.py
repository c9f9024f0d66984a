"""vLLM platform plugin: the entry points resolve to a class vLLM can use as its platform, the
attention backend is registered under CUSTOM, and the configuration hooks run on a build host."""
import importlib
import os
import sys

import pytest

vllm = pytest.importorskip("vllm")


def test_entry_points_are_declared():
    import tomllib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "pyproject.toml"), "rb") as f:
        eps = tomllib.load(f)["project"]["entry-points"]
    assert eps["vllm.platform_plugins"]["b200"] == "vllm_torchtpu_b200.vllm_plugin:register_platform"
    assert eps["vllm.general_plugins"]["b200"] == "vllm_torchtpu_b200.vllm_plugin:register_general"
    for target in list(eps["vllm.platform_plugins"].values()) + list(eps["vllm.general_plugins"].values()):
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn))


def test_platform_is_a_vllm_platform_and_resolves_through_the_plugin_group(tmp_path, monkeypatch):
    """A dist-info directory with this package's entry points on sys.path is what an installed copy
    looks like to importlib.metadata; vLLM's resolver must then pick the plugin's class."""
    from vllm.platforms.interface import Platform
    from vllm_torchtpu_b200.vllm_plugin import PLATFORM_CLASS, register_platform
    from vllm_torchtpu_b200.vllm_plugin.platform import B200VllmPlatform
    assert issubclass(B200VllmPlatform, Platform)
    for hook in ("get_attn_backend_cls", "get_device_communicator_cls", "check_and_update_config",
                 "validate_request"):
        assert hook in B200VllmPlatform.__dict__, hook
    monkeypatch.delenv("B200_VLLM_PLUGIN_FORCE", raising=False)
    import torch
    if not torch.cuda.is_available():
        assert register_platform() is None              # no Blackwell GPU here: vLLM keeps looking
    monkeypatch.setenv("B200_VLLM_PLUGIN_FORCE", "1")
    assert register_platform() == PLATFORM_CLASS
    di = tmp_path / "vllm_torchtpu_b200-0.1.0.dist-info"
    di.mkdir()
    (di / "METADATA").write_text("Metadata-Version: 2.1\nName: vllm-torchtpu-b200\nVersion: 0.1.0\n")
    (di / "entry_points.txt").write_text(
        "[vllm.platform_plugins]\nb200 = vllm_torchtpu_b200.vllm_plugin:register_platform\n\n"
        "[vllm.general_plugins]\nb200 = vllm_torchtpu_b200.vllm_plugin:register_general\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    importlib.invalidate_caches()
    import vllm.platforms as P
    assert P.resolve_current_platform_cls_qualname() == PLATFORM_CLASS
    from vllm.utils.import_utils import resolve_obj_by_qualname
    assert resolve_obj_by_qualname(PLATFORM_CLASS) is B200VllmPlatform


def test_general_plugin_registers_backend_and_ops():
    from vllm.model_executor.custom_op import op_registry_oot
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    from vllm_torchtpu_b200.vllm_plugin import ATTENTION_BACKEND, register_general
    register_general()
    register_general()                                  # idempotent
    assert AttentionBackendEnum.CUSTOM.get_path() == ATTENTION_BACKEND
    cls = AttentionBackendEnum.CUSTOM.get_class()
    assert cls.get_name() == "CUSTOM"
    assert cls.get_kv_cache_shape(7, 16, 2, 128) == (7, 2, 2, 16, 128)
    assert cls.get_impl_cls().__name__ == "B200AttentionImpl" and cls.get_builder_cls().__name__ == "B200MetadataBuilder"
    assert "RMSNorm" in op_registry_oot and "SiluAndMul" in op_registry_oot


def test_platform_hooks_on_a_build_host():
    import torch
    from types import SimpleNamespace
    from vllm_torchtpu_b200.vllm_plugin.platform import ATTENTION_BACKEND, COMMUNICATOR, B200VllmPlatform as P
    sel = SimpleNamespace(head_size=128, dtype=torch.bfloat16, use_mla=False, use_sparse=False)
    assert P.get_attn_backend_cls(None, sel) == ATTENTION_BACKEND
    assert P.get_device_communicator_cls() == COMMUNICATOR
    with pytest.raises(ValueError):
        P.validate_request(params=SimpleNamespace(seed=3, temperature=1.0))
    P.validate_request(params=SimpleNamespace(seed=None, temperature=0.0))
    assert P.is_kv_cache_dtype_supported("fp8") and not P.is_kv_cache_dtype_supported("int4")
