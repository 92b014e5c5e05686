"""RMSNorm as a part: y = (x * rsqrt(mean(x^2) + eps)) * (w + offset), statistics
in 32-bit (src/metal/kernels/tensor_ops.metal:76-105).

"layernorm": y = (x - mean) * rsqrt(var + eps) * (w + offset) + b with the variance
as the mean of the squared deviations; its kernel can also add the result to a
32-bit residual (``add_to``), which is how a block with norms on its sublayers'
outputs uses it."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Norm, Runtime, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec, weight_name: str, runtime: Runtime):
        self.spec = spec
        self.weight_name = weight_name
        self.runtime = runtime
        self.weight: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.spec.size,))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """x, out: [rows, k * size]; every run of ``size`` features is one group."""
        n = self.spec.size
        if x.shape[-1] == n:
            self.runtime.kernels.rmsnorm(x, self.weight, self.spec.eps, self.spec.weight_offset, out)
        else:
            if not x.is_contiguous() or not out.is_contiguous():
                raise ValueError("grouped norm needs contiguous rows")
            self.runtime.kernels.rmsnorm(x.view(-1, n), self.weight, self.spec.eps,
                                         self.spec.weight_offset, out.view(-1, n))


    def forward_fused(self, residual: torch.Tensor, pending, out: torch.Tensor, scaled_ok: bool = False):
        k = self.runtime.kernels
        if pending is not None and residual.shape[-1] == self.spec.size:
            if hasattr(pending, "finish_with_norm"):
                # a product of many rows that has not run yet: it writes the norm's output itself
                return pending.finish_with_norm(residual, self.weight, self.spec.eps, self.spec.weight_offset,
                                                out, scaled_ok)
            fused = getattr(k, "reduce_residual_rmsnorm", None)
            if fused is not None and hasattr(pending, "partial"):
                fused(pending, residual, self.weight, self.spec.eps, self.spec.weight_offset, out)
                return out
        return super().forward_fused(residual, pending, out, scaled_ok)

    def add_to(self, y: torch.Tensor, residual: torch.Tensor, copy_out: torch.Tensor = None) -> None:
        """residual += norm(y); ``copy_out`` takes the new residual in its own type."""
        self.runtime.kernels.norm_rows(y, self.weight, None, self.spec.eps, self.spec.weight_offset, False,
                                       residual=residual, out=copy_out)


class LayerNorm(Norm):
    def __init__(self, spec, weight_name: str, runtime: Runtime):
        self.spec = spec
        self.weight_name = weight_name
        self.bias_name = weight_name + spec.bias_suffix
        self.runtime = runtime
        self.weight: torch.Tensor = None
        self.bias: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.spec.size,)),
                TensorSpec(self.bias_name, (self.spec.size,), init=("normal", 0.0, 0.1))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].to(self.weight.dtype).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        self.runtime.kernels.norm_rows(x, self.weight, self.bias, self.spec.eps, self.spec.weight_offset, True,
                                       out=out)

    def add_to(self, y: torch.Tensor, residual: torch.Tensor, copy_out: torch.Tensor = None) -> None:
        """residual += norm(y); ``copy_out`` takes the new residual in its own type."""
        self.runtime.kernels.norm_rows(y, self.weight, self.bias, self.spec.eps, self.spec.weight_offset, True,
                                       residual=residual, out=copy_out)


register_norm("rmsnorm", RMSNorm, replace=True)
register_norm("layernorm", LayerNorm, replace=True)
