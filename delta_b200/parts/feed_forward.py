"""SwiGLU feed-forward:  down( silu(gate x) * (up x) )
(reference: DELTA/Engine/DELTA/model.py:495-518, ``w2(silu(w1 x) * w3 x)``), a dense feed-forward with one of several
activations, and a gated one with clamped branches."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from . import linear
from .base import FEED_FORWARDS, FeedForward, TensorSpec


# g sigmoid(alpha (g + cubic g^3)) (u + shift): the constants of two common gates
SILU_GATE = dict(alpha=1.0, shift=0.0, cubic=0.0)                                        # silu(g) u
GELU_TANH_GATE = dict(alpha=2.0 * math.sqrt(2.0 / math.pi), shift=0.0, cubic=0.044715)   # 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``width`` d and ``intermediate`` I are parameters.  gate_proj and up_proj
    are stacked into one [2I, d] matrix so that one product feeds the gate kernel."""

    def __init__(self, prefix: str, width: int, intermediate: int):
        self.prefix = prefix
        self.width = int(width)
        self.intermediate = int(intermediate)
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p, d, i = self.prefix, self.width, self.intermediate
        return [TensorSpec(p + "gate_proj.weight", (i, d)), TensorSpec(p + "up_proj.weight", (i, d)),
                TensorSpec(p + "down_proj.weight", (d, i))]

    def bind(self, tensors):
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, ctx, x):
        act = linear.swiglu_linear(ctx, x, self.w_gate_up)
        if act is None:
            gu = linear.linear(ctx, x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act)
        return linear.linear(ctx, act, self.w_down)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    """down( act(up x) ) with ``activation`` one of "relu2" (the square of relu), "gelu_tanh", "silu".  Tensor names:
    ``<prefix><up_name>`` [I, d] and ``<prefix><down_name>`` [d, I]."""

    def __init__(self, prefix: str, width: int, intermediate: int, activation: str = "relu2", up_name: str = "up",
                 down_name: str = "down"):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation '{activation}'; known: {', '.join(ops.ACTIVATIONS)}")
        self.prefix, self.width, self.intermediate, self.activation = prefix, int(width), int(intermediate), activation
        self.up_name, self.down_name = up_name, down_name
        self.w_up = self.w_down = None

    def tensor_specs(self):
        p, d, i = self.prefix, self.width, self.intermediate
        return [TensorSpec(p + self.up_name, (i, d)), TensorSpec(p + self.down_name, (d, i))]

    def bind(self, tensors):
        self.w_up = tensors[self.prefix + self.up_name]
        self.w_down = tensors[self.prefix + self.down_name]

    def forward(self, ctx, x):
        h = linear.linear(ctx, x, self.w_up)
        ops.activation(h, h, self.activation)
        return linear.linear(ctx, h, self.w_down)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """down( g' * sigmoid(alpha (g' + cubic g'^3)) * (u' + shift) ) with g' = min(gate x, limit) and u' = clamp(up x, -limit, limit)
    (``limit`` None: unclamped).  ``SILU_GATE`` and ``GELU_TANH_GATE`` are the constants of silu(g) u and of the tanh form of gelu,
    gelu(g) u.  Tensor names: ``<prefix>gate``, ``<prefix>up`` [I, d] and ``<prefix>down`` [d, I]."""

    def __init__(self, prefix: str, width: int, intermediate: int, limit=None, alpha: float = 1.702, shift: float = 1.0,
                 cubic: float = 0.0):
        self.prefix, self.width, self.intermediate = prefix, int(width), int(intermediate)
        if limit is not None and float(limit) < 0:
            raise ValueError(f"a clamp at {limit} is no limit")
        self.limit, self.alpha, self.shift, self.cubic = (-1.0 if limit is None else float(limit)), float(alpha), float(shift), float(cubic)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        p, d, i = self.prefix, self.width, self.intermediate
        return [TensorSpec(p + "gate", (i, d)), TensorSpec(p + "up", (i, d)), TensorSpec(p + "down", (d, i))]

    def bind(self, tensors):
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate"], tensors[p + "up"]], dim=0).contiguous()
        self.w_down = tensors[p + "down"]

    def forward(self, ctx, x):
        gu = linear.linear(ctx, x, self.w_gate_up)
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ops.glu_clamped(gu, act, self.limit, self.alpha, self.shift, self.cubic)
        return linear.linear(ctx, act, self.w_down)
