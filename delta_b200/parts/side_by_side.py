"""Two mixers side by side: both read the same input; each output goes through an RMS norm over the model width with a weight
of its own, and the result is ``factor`` times their sum (1/2: the mean),

    out = factor * ( rms_norm(left(h)) * w_left + rms_norm(right(h)) * w_right ).

Either mixer may keep a paged cache (at most one of them) and either may keep a per-run state; the pair hands both on.  The
branches' outputs are taken in 32 bit (``wide_output``) and the norms and the sum are one kernel; a branch whose output
projection has a bias lets this kernel add it.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, Mixer, PartSpec, TensorSpec


@MIXERS.register("side_by_side")
class SideBySide(Mixer):
    """``left`` / ``right``: ``PartSpec`` of the two mixers (built with ``wide_output=True``).  Tensor names: ``<prefix>left.out``,
    ``<prefix>right.out`` [width]."""

    def __init__(self, prefix: str, width: int, left: PartSpec, right: PartSpec, eps: float, factor: float = 0.5):
        self.prefix, self.width, self.eps, self.factor = prefix, int(width), float(eps), float(factor)
        self.left = left.build(MIXERS, wide_output=True)
        self.right = right.build(MIXERS, wide_output=True)
        if self.left.cache_spec() is not None and self.right.cache_spec() is not None:
            raise ValueError("only one of two mixers side by side may keep a paged cache")
        for m in (self.left, self.right):
            if hasattr(m, "fold_out_bias"):
                m.fold_out_bias = True
        self.w_left = self.w_right = None

    def children(self):
        return (self.left, self.right)

    def tensor_specs(self):
        own = [TensorSpec(self.prefix + "left.out", (self.width,), kind="vector", init="norm"),
               TensorSpec(self.prefix + "right.out", (self.width,), kind="vector", init="norm")]
        return self.left.tensor_specs() + self.right.tensor_specs() + own

    def bind(self, tensors):
        self.left.bind(tensors)
        self.right.bind(tensors)
        self.w_left = tensors[self.prefix + "left.out"].float().contiguous()
        self.w_right = tensors[self.prefix + "right.out"].float().contiguous()

    def cache_spec(self):
        return self.left.cache_spec() or self.right.cache_spec()

    def state_specs(self):
        return {**self.left.state_specs(), **self.right.state_specs()}

    def run_state_specs(self):
        out = {}
        for m in self.children():
            if hasattr(m, "run_state_specs"):
                for k, v in m.run_state_specs().items():
                    if k in out:
                        raise ValueError(f"both mixers side by side keep a state named '{k}'")
                    out[k] = v
        return out

    def begin_step(self, ctx):
        self.left.begin_step(ctx)
        self.right.begin_step(ctx)

    def decode_rows_differ(self):
        return self.left.decode_rows_differ() or self.right.decode_rows_differ()

    def forward(self, ctx, x, cache):
        a = self.left.forward(ctx, x, cache)
        b = self.right.forward(ctx, x, cache)
        if a.dtype != torch.float32 or b.dtype != torch.float32:
            raise TypeError("mixers side by side hand their outputs on in 32 bit (wide_output)")
        out = torch.empty_like(a)
        bias = lambda m: getattr(m, "out_bias", None) if getattr(m, "fold_out_bias", False) else None     # noqa: E731
        return ops.normed_sum([(a, bias(self.left), self.w_left), (b, bias(self.right), self.w_right)], out, self.eps, self.factor)
