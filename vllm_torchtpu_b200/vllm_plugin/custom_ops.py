"""Out-of-tree providers of vLLM custom ops on this package's kernels: RMSNorm (+ fused residual add)
and SiLU*mul (reference: src/vllm_torchtpu/layers/adapter/ir_ops.py:50-88 registers CUDA-numerics
norm providers the same way).  The kernels are wrapped as ``torch.library`` custom ops so that a
traced model sees one opaque call."""
from __future__ import annotations

import torch

_LIB_READY = False


def _define_ops() -> None:
    global _LIB_READY
    if _LIB_READY:
        return
    _LIB_READY = True

    @torch.library.custom_op("b200::rms_norm", mutates_args=())
    def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        from ..ops import cuda
        return cuda.rms_norm(x, weight, eps)

    @rms_norm.register_fake
    def _(x, weight, eps):
        return torch.empty_like(x)

    @torch.library.custom_op("b200::fused_add_rms_norm", mutates_args=("residual",))
    def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        from ..ops import cuda
        y, _ = cuda.fused_add_rms_norm(x, residual, weight, eps)
        return y

    @fused_add_rms_norm.register_fake
    def _(x, residual, weight, eps):
        return torch.empty_like(x)

    @torch.library.custom_op("b200::silu_and_mul", mutates_args=())
    def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
        from ..ops import cuda
        return cuda.silu_and_mul(x)

    @silu_and_mul.register_fake
    def _(x):
        return x.new_empty(x.shape[:-1] + (x.shape[-1] // 2,))


def register() -> None:
    from vllm.model_executor.custom_op import CustomOp, op_registry_oot
    from vllm.model_executor.layers.activation import SiluAndMul
    from vllm.model_executor.layers.layernorm import RMSNorm
    _define_ops()

    def _ours(x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0

    if "RMSNorm" not in op_registry_oot:
        @CustomOp.register_oot(name="RMSNorm")
        class B200RMSNorm(RMSNorm):
            """RMSNorm / fused add + RMSNorm on the one-pass bf16 kernel; other dtypes and the
            variance-size override keep vLLM's path."""

            def _b200(self, x, residual=None):
                if (not _ours(x) or self.variance_size_override is not None
                        or not getattr(self, "has_weight", True) or self.weight.dtype != torch.bfloat16):
                    return None
                x2 = x.reshape(-1, x.shape[-1])
                if not x2.is_contiguous():
                    x2 = x2.contiguous()
                if residual is None:
                    return torch.ops.b200.rms_norm(x2, self.weight.data, float(self.variance_epsilon)).view(x.shape)
                r2 = residual.reshape(-1, residual.shape[-1])
                if not r2.is_contiguous():
                    return None
                y = torch.ops.b200.fused_add_rms_norm(x2, r2, self.weight.data, float(self.variance_epsilon))
                return y.view(x.shape), residual

            def forward_cuda(self, x, residual=None):
                out = self._b200(x, residual)
                return out if out is not None else super().forward_cuda(x, residual)

            def forward_oot(self, x, residual=None):
                out = self._b200(x, residual)
                return out if out is not None else self.forward_native(x, residual)

    if "SiluAndMul" not in op_registry_oot:
        @CustomOp.register_oot(name="SiluAndMul")
        class B200SiluAndMul(SiluAndMul):
            def _b200(self, x):
                if not _ours(x) or x.shape[-1] % 16:
                    return None
                x2 = x.reshape(-1, x.shape[-1])
                if not x2.is_contiguous():
                    x2 = x2.contiguous()
                return torch.ops.b200.silu_and_mul(x2).view(x.shape[:-1] + (x.shape[-1] // 2,))

            def forward_cuda(self, x):
                out = self._b200(x)
                return out if out is not None else super().forward_cuda(x)

            def forward_oot(self, x):
                out = self._b200(x)
                return out if out is not None else self.forward_native(x)
