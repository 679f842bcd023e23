"""Norms.

``layer_norm``: mean and biased variance of the row in float32, eps inside the
root, weight and bias (include/ai/LocalModel.hpp:1355-1367).

``dynamic_tanh``: tanh(alpha x) * weight + bias with a learned scalar alpha; no
mean, no variance, no eps.  Tensors ``weight``, ``bias``, ``alpha`` (a scalar).

``rms_norm``: scale * x / sqrt(mean(x^2) + eps) * (weight_offset + weight), statistics in float32.
``weight_offset`` (0 unless given; 1 for a weight stored around zero) and ``scale`` (1 unless given:
the multiplier with which a normed sublayer output joins the residual stream) are parameters."""
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
        self.offset = float(self.param("weight_offset", 0.0))
        self.scale = float(self.param("scale", 1.0))

    def tensor_specs(self):
        return (TensorSpec(self.tensor_name("weight"), (self.size,), role="vector",
                           init=self.param("init", "norm_weight")),)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tensor_name("weight")]

    def forward(self, x, rows=None):
        return self.runtime.ops.rms_norm_out(x, self.weight, self.eps, self.offset, self.scale,
                                             out_dtype=self.runtime.dtype, rows=rows)

    def forward_float(self, x, out=None):
        return self.runtime.ops.rms_norm_out(x, self.weight, self.eps, self.offset, self.scale, out=out)

    def add_into(self, y, residual, copy=None, second=None) -> None:
        """residual += norm(y); ``copy`` (bfloat16, shaped like the stream) receives the stream as it then is;
        ``second`` = (a, y2, b): the norm's input is a * y + b * y2."""
        self.runtime.ops.rms_norm_out(y, self.weight, self.eps, self.offset, self.scale, out=residual, add=True,
                                      copy=copy, second=second)


register_part("norm", "layer_norm", LayerNorm, replace=True)
register_part("norm", "dynamic_tanh", DynamicTanh, replace=True)
class IdentityNorm(Norm):
    """Stands where a layer has no norm: the rows in the compute dtype."""

    def forward(self, x, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long())
        if x.dtype == self.runtime.dtype:
            return x
        import torch
        if x.dtype == torch.float32 and self.runtime.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1:
            return self.runtime.ops.cast_rows(x)
        return x.to(self.runtime.dtype)


register_part("norm", "rms_norm", RmsNorm, replace=True)
register_part("norm", "identity", IdentityNorm, replace=True)
