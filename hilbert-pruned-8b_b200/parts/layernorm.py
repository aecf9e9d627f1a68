"""Layer norm with weight and bias: ``y = (x - mean) / sqrt(var + eps) * w + b`` over a row, ``var`` the
mean squared deviation from the mean; sums, deviations and scaling in 32-bit on the device, the result
in the dtype the next matrix product reads.

As a norm on a sublayer's OUTPUT (``add_normed``) it adds the normed output to the 32-bit residual
stream and, when asked, leaves a copy of the stream's new rows in the products' dtype: in a block whose
sublayers read the stream itself, that copy is what a bfloat16 product reads next.  ``add_normed_sum``
norms the weighted sum of two outputs without that sum ever being stored.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import NORMS, Norm, ParamSpec


@NORMS.register("layernorm")
class LayerNorm(Norm):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        # below the part's prefix ("": the prefix itself); the bias is the weight's name with a suffix
        self.tensor_name = spec.get("tensor_name", "weight")
        self.bias_name = self.tensor_name + spec.get("bias_suffix", ".b")
        self.weight = self.bias = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor_name, (self.size,), kind="vector", init="ones"),
                ParamSpec(self.bias_name, (self.size,), kind="vector", init="zeros")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name].reshape(self.size).to(torch.float32).contiguous()
        self.bias = tensors[self.bias_name].reshape(self.size).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.size * 8

    def forward(self, x, out, rows=None) -> None:
        """``out[i] = norm(x[rows[i]])`` (``rows`` None: every row of ``x``)."""
        self.ctx.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)

    def add_normed(self, y, x, then=None, then_out=None, copy=None) -> bool:
        """``x += norm(y)``; ``copy`` also receives the stream's new rows in its own dtype.  No second norm is made here:
        returns False when one was asked for (the caller then runs it)."""
        self.ctx.ops.layernorm_add(y, self.weight, self.bias, self.eps, x, copy=copy)
        return False

    def add_normed_sum(self, a, sa: float, b, sb: float, x, copy=None) -> None:
        """``x += norm(sa * a + sb * b)``; ``copy`` as in ``add_normed``."""
        self.ctx.ops.layernorm_add(a, self.weight, self.bias, self.eps, x, copy=copy, y2=b, sa=sa, sb=sb)
