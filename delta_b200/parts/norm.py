"""RMSNorm: x * rsqrt(mean(x^2) + eps) * weight, the statistics in 32 bit
(reference: DELTA/Engine/DELTA/model.py:521-532), and the layer norm,
(x - mean) / sqrt(var + eps) * weight (+ bias) with var the mean of the squared deviations."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import NORMS, Norm, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """``width`` and ``eps`` are parameters.  ``cast_before_weight`` keeps the order of
    the reference in reduced precision: the normalised value is rounded to the
    activation type before it is multiplied by the weight (model.py:531-532)."""

    kind = "rms"       # what a kernel that normalises a 32-bit stream is told

    def __init__(self, name: str, width: int, eps: float, cast_before_weight: bool = True):
        self.name = name
        self.width = int(width)
        self.eps = float(eps)
        self.cast_before_weight = bool(cast_before_weight)
        self.weight = None
        self._weight32 = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.width,), kind="vector", init="norm")]

    def bind(self, tensors):
        self.weight = tensors[self.name]
        self._weight32 = None

    def weight32(self):
        """The weight in 32 bit, for kernels that normalise a 32-bit stream."""
        if self._weight32 is None:
            self._weight32 = self.weight.float().contiguous()
        return self._weight32

    def forward(self, ctx, x, add=None, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=x.dtype, device=x.device)
        cast_first = self.cast_before_weight and x.dtype != torch.float32
        return ops.rms_norm(x, self.weight, self.eps, out, add=add, rows=rows, cast_first=cast_first)


@NORMS.register("layer_norm")
class LayerNorm(Norm):
    """Layer norm with a weight and, with ``bias``, a bias (the tensor ``<name>.b``); ``scale`` names a vector that the result is
    multiplied by, column by column (folded into weight and bias when they are bound).  It reads a 32-bit residual stream (``parts/residual.py``), whose kernel
    takes the mean and the squared deviations in two passes over the row; it has no kernel for a stream in the compute
    type, so a model with the ``single`` stream cannot name it."""
    kind = "layer"

    def __init__(self, name: str, width: int, eps: float, bias: bool = False, scale: str = None):
        self.name, self.width, self.eps, self.has_bias = name, int(width), float(eps), bool(bias)
        self.scale_name = scale
        self.weight = self.bias = self.scale = None
        self._weight32 = self._bias32 = None

    def tensor_specs(self):
        specs = [TensorSpec(self.name, (self.width,), kind="vector", init="norm")]
        if self.has_bias:
            specs.append(TensorSpec(self.name + ".b", (self.width,), kind="vector", init="uniform:-0.1:0.1"))
        if self.scale_name:
            specs.append(TensorSpec(self.scale_name, (self.width,), kind="vector", init="uniform:0.5:1.5"))
        return specs

    def bind(self, tensors):
        self.weight = tensors[self.name]
        self.bias = tensors[self.name + ".b"] if self.has_bias else None
        self.scale = tensors[self.scale_name] if self.scale_name else None
        self._weight32 = self._bias32 = None

    def weight32(self):
        """The weight in 32 bit, times the scale: (n w + b) s = n (w s) + (b s)."""
        if self._weight32 is None:
            w = self.weight.float()
            self._weight32 = (w * self.scale.float() if self.scale is not None else w).contiguous()
        return self._weight32

    def bias32(self):
        """The bias in 32 bit, times the scale (None: the norm has no bias)."""
        if self._bias32 is None and self.bias is not None:
            b = self.bias.float()
            self._bias32 = (b * self.scale.float() if self.scale is not None else b).contiguous()
        return self._bias32

    def forward(self, ctx, x, add=None, rows=None):
        if x.dtype != torch.float32:
            raise TypeError("layer_norm reads a 32-bit residual stream (stream 'residual_f32')")
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=ctx.dtype, device=x.device)
        return ops.residual_norm(x, out, updates=() if add is None else (add,), weight=self.weight32(), bias=self.bias32(), eps=self.eps,
                                 kind="layer", rows=rows, write_back=rows is None)
