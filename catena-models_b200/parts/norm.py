"""RMSNorm: y = (x / sqrt(mean(x^2) + eps)) * w, the product with w taken in float before
the one rounding to the activation dtype (src/catena/qwen35.hex:912-946,
src/catena/fused_normalization.hex:23-39).  The weight is float32 as in the reference's
tensor list (src/spec.rs:722-735).  Fused kernels (residual sum + norms) read `weight` and
`eps` directly.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True
    fused_kind = "rms"          # what the fused residual kernel can absorb

    def __init__(self, name, width, eps, weight_offset=0.0):
        """weight_offset: what is added to the stored weight (1 for a checkpoint that stores the distance
        of the weight from one); the sum is formed once, in float, when the tensor is bound."""
        self.name, self.width, self.eps = name, width, float(eps)
        self.weight_offset = float(weight_offset)
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), "norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.name].to(torch.float32).contiguous()
        if self.weight_offset:
            self.weight = self.weight + self.weight_offset
        self._bound = [self.weight]

    def apply(self, rt, x):
        if x.dtype == torch.float32 and (rt.dtype != torch.float32 or self.width % 8):
            # rows of a float residual stream: normed in float, written as activations
            y = torch.empty(x.shape, dtype=rt.dtype, device=x.device)
            kernels.norm_f32in(y, x, self.weight, self.eps)
            return y
        y = torch.empty_like(x)
        kernels.rmsnorm(y, x, self.weight, self.eps)
        return y


class ScalarRMSNorm(RMSNorm):
    """An RMS norm whose weight is one number for all channels: y = x / sqrt(mean(x^2) + eps) * g.  The number is
    repeated over the width when it is bound, so every kernel that takes an RMS norm takes this one."""

    def tensor_specs(self):
        return [TensorSpec(self.name, (), "norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.name].to(torch.float32).reshape(1).expand(self.width).contiguous()
        self._bound = [self.weight]


class DynamicTanh(Norm):
    """y = tanh(alpha x) * w + b in place of a norm: no mean, no variance, nothing that looks along the row.
    `alpha` is a learned scalar stored as `<name>.alpha`, the shift as `<name>.b`.  Takes float32 rows (a
    float32 residual stream) and writes activations; the residual kernel of such a stream applies it in the
    same launch (`fused_kind`)."""
    prompt_capturable = True
    supports_append = True
    fused_kind = "dyt"

    def __init__(self, name, width):
        self.name, self.width, self.eps = name, width, 0.0
        self.weight = self.alpha = self.shift = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), "norm"), TensorSpec(self.name + ".alpha", (), "vector"),
                TensorSpec(self.name + ".b", (self.width,), "vector")]

    def bind(self, tensors, rt):
        f32 = lambda n: tensors[n].to(torch.float32).contiguous()
        self.weight, self.shift = f32(self.name), f32(self.name + ".b")
        self.alpha = f32(self.name + ".alpha").reshape(1)
        self._bound = [self.weight, self.shift, self.alpha]

    def apply(self, rt, x):
        if x.dtype != torch.float32:
            raise NotImplementedError("the dynamic tanh reads float32 rows (ModelDefinition.residual_float32)")
        y = torch.empty(x.shape, dtype=rt.dtype, device=x.device)
        kernels.norm_f32in(y, x.contiguous(), self.weight, 0.0, dyt=(self.alpha, self.shift))
        return y


register_part("norm", "rms", RMSNorm)
register_part("norm", "scalar_rms", ScalarRMSNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
