"""Quantisation method dispatch.

``get_linear_method`` / ``get_moe_method`` map a model's quantisation name to
the method object of each layer, the way the reference dispatches on the
checkpoint's quantisation config
(reference: src/vllm_torchtpu/layers/adapter/quantization/__init__.py:51-101).
"""
from __future__ import annotations

from typing import Optional


class QuantConfig:
    def __init__(self, name: Optional[str], weight_block_size=(128, 128), ignored_layers=(),
                 activation_scheme: str = "dynamic"):
        self.name = name
        self.weight_block_size = tuple(weight_block_size)
        self.ignored_layers = tuple(ignored_layers)
        self.activation_scheme = activation_scheme

    def is_ignored(self, layer_name: str) -> bool:
        return any(p in layer_name for p in self.ignored_layers)


def get_linear_method(quant_config: Optional[QuantConfig], layer_name: str = ""):
    from .unquantized import UnquantizedLinearMethod
    if quant_config is None or quant_config.name is None or quant_config.is_ignored(layer_name):
        return UnquantizedLinearMethod()
    n = quant_config.name
    if n == "fp8_block":
        from .fp8 import Fp8BlockLinearMethod
        return Fp8BlockLinearMethod(quant_config.weight_block_size)
    if n == "fp8":
        from .fp8 import Fp8PerTensorLinearMethod
        return Fp8PerTensorLinearMethod()
    if n == "online_fp8":
        from .fp8 import OnlineFp8LinearMethod
        return OnlineFp8LinearMethod(quant_config.weight_block_size)
    if n in ("int8", "compressed-tensors"):
        from .int8 import Int8LinearMethod
        return Int8LinearMethod()
    if n == "mxfp4":
        from .fp4 import Mxfp4LinearMethod
        return Mxfp4LinearMethod()
    if n == "nvfp4":
        from .fp4 import Nvfp4LinearMethod
        return Nvfp4LinearMethod()
    if n in ("awq", "gptq"):
        from .int4 import Int4GroupLinearMethod
        return Int4GroupLinearMethod(fmt=n)
    raise ValueError(f"unknown quantization {n!r}")


def get_moe_method(quant_config: Optional[QuantConfig], layer_name: str = ""):
    from .unquantized import UnquantizedMoEMethod
    if quant_config is None or quant_config.name is None or quant_config.is_ignored(layer_name):
        return UnquantizedMoEMethod()
    n = quant_config.name
    if n in ("fp8_block", "online_fp8"):
        from .fp8 import Fp8BlockMoEMethod
        return Fp8BlockMoEMethod(quant_config.weight_block_size, online=(n == "online_fp8"))
    if n == "mxfp4":
        from .fp4 import Mxfp4MoEMethod
        return Mxfp4MoEMethod()
    # other schemes keep experts in the activation dtype
    return UnquantizedMoEMethod()
