"""Norms.

``layer_norm``: mean and biased variance of the row in float32, eps inside the
root, weight and bias (include/ai/LocalModel.hpp:1355-1367).

``dynamic_tanh``: tanh(alpha x) * weight + bias with a learned scalar alpha; no
mean, no variance, no eps.  Tensors ``weight``, ``bias``, ``alpha`` (a scalar).

``rms_norm``: x / sqrt(mean(x^2) + eps) * weight, statistics in float32."""
from __future__ import annotations

from ..config.base import PartSpec
from .base import Norm, TensorSpec, register_part


class LayerNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.size,), role="vector", init="norm_weight"),
                TensorSpec(self.tensor_name("bias"), (self.size,), role="vector", init="norm_bias"))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]
        self.bias = tensors[self.tensor_name("bias")]

    def forward(self, x, rows=None):
        return self.runtime.ops.layernorm(x, self.weight, self.bias, self.eps, self.runtime.dtype, rows=rows)

    def lazy(self, x, rows=None):
        """Not computed yet: the product kernels know this norm and make it while they load their rows."""
        return self.runtime.ops.NormedInput(x, self.weight, self.bias, self.eps, self.runtime.dtype, rows=rows)


class DynamicTanh(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(self.param("size"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.size,), role="vector", init="norm_weight"),
                TensorSpec(self.tensor_name("bias"), (self.size,), role="vector", init="norm_bias"),
                TensorSpec(self.tensor_name("alpha"), (), role="vector", init="norm_alpha"))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]
        self.bias = tensors[self.tensor_name("bias")]
        self.alpha = tensors[self.tensor_name("alpha")].reshape(1)

    def forward(self, x, rows=None):
        return self.runtime.ops.dynamic_tanh(x, self.weight, self.bias, self.alpha, self.runtime.dtype, rows=rows)

    def forward_float(self, x, out=None):
        return self.runtime.ops.dynamic_tanh(x, self.weight, self.bias, self.alpha, out=out)

    def add_into(self, y, residual) -> None:
        self.runtime.ops.dynamic_tanh(y, self.weight, self.bias, self.alpha, out=residual, add=True)


class RmsNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.size,), role="vector", init="norm_weight"),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def forward(self, x, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long())
        return self.runtime.ops.rms_norm(x, self.weight, self.eps, self.runtime.dtype)


register_part("norm", "layer_norm", LayerNorm, replace=True)
register_part("norm", "dynamic_tanh", DynamicTanh, replace=True)
class IdentityNorm(Norm):
    """Stands where a layer has no norm: the rows in the compute dtype."""

    def forward(self, x, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long())
        return x.to(self.runtime.dtype)


register_part("norm", "rms_norm", RmsNorm, replace=True)
register_part("norm", "identity", IdentityNorm, replace=True)
