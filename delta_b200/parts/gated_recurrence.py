"""A recurrent block with a gated diagonal linear recurrence (the real-gated linear recurrent unit of Griffin).

With mixer input h, C = ``channels``, a convolution of ``conv`` taps and ``blocks`` equal groups of channels:
    y = gelu_tanh(W_y h + b_y)                            the gate branch
    u = causal_conv(W_x h + b_x) + b_conv                 per channel over the request's tokens, no activation
    r = sigmoid(R_b u_b + rb_b),  i = sigmoid(I_b u_b + ib_b)      per group b, R_b and I_b square
    a = exp(-``decay_scale`` * r * softplus(lam))         per channel
    S <- a S + sqrt(1 - a^2) (i u)                        from S = 0, the first token like every other
    out = W_o (S * y)
A request's state is the last ``conv - 1`` inputs of the convolution and S, both 32 bit and one pair per run of the layer; a
step continues from what the request's earlier steps left.  The two projections are one product, the two gates' matrices of
a group one product per group (batched); gates, decays and the state are 32 bit whatever the compute type.  Long portions
are cut into segments that run in parallel (the recurrence is linear in S) and are stitched together in order.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import linear
from .base import MIXERS, Mixer, StateSpec, TensorSpec

SEGMENT = 16            # tokens of a segment when a long portion's recurrence runs in parallel pieces
CONV_STATE = "conv"
SCAN_STATE = "recurrence"


@MIXERS.register("gated_recurrence")
class GatedRecurrence(Mixer):
    """Tensor names under ``prefix``: ``x``, ``y`` [C, d] with ``x.b``, ``y.b`` [C]; ``conv`` [C, taps], ``conv.b`` [C]; ``ra``, ``ri``
    [blocks, C/blocks, C/blocks] with ``ra.b``, ``ri.b`` [blocks, C/blocks]; ``lam`` [C]; ``o`` [d, C]."""

    def __init__(self, prefix: str, width: int, channels: int, conv: int, blocks: int, decay_scale: float = 8.0,
                 wide_output: bool = False):
        self.prefix, self.width = prefix, int(width)
        self.channels, self.taps, self.blocks = int(channels), int(conv), int(blocks)
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        if self.blocks < 1 or self.channels % self.blocks:
            raise ValueError(f"{self.channels} channels do not split into {self.blocks} equal groups")
        self.block_size = self.channels // self.blocks
        self.decay_scale, self.wide_output = float(decay_scale), bool(wide_output)
        self.w_in = self.w_gates = self.w_o = None
        self.x_bias = self.y_bias = self.conv_w = self.conv_b = self.r_bias = self.i_bias = self.decay = None

    def tensor_specs(self):
        p, d, C, nb, sz = self.prefix, self.width, self.channels, self.blocks, self.block_size
        vec = dict(kind="vector", init="uniform:-0.1:0.1")
        return [TensorSpec(p + "y", (C, d)), TensorSpec(p + "y.b", (C,), **vec), TensorSpec(p + "x", (C, d)), TensorSpec(p + "x.b", (C,), **vec),
                TensorSpec(p + "conv", (C, self.taps), kind="vector", init="uniform:-0.5:0.5"), TensorSpec(p + "conv.b", (C,), **vec),
                TensorSpec(p + "ra", (nb, sz, sz)), TensorSpec(p + "ra.b", (nb, sz), **vec),
                TensorSpec(p + "ri", (nb, sz, sz)), TensorSpec(p + "ri.b", (nb, sz), **vec),
                TensorSpec(p + "lam", (C,), kind="vector", init="uniform:-4:-1"), TensorSpec(p + "o", (d, C))]

    def bind(self, tensors):
        p = self.prefix
        f = lambda n: tensors[p + n].float().contiguous()   # noqa: E731  (what the recurrence reads is kept in 32 bit)
        self.w_in = torch.cat([tensors[p + "x"], tensors[p + "y"]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors[p + "ra"], tensors[p + "ri"]], dim=1).contiguous()      # [blocks, 2 sz, sz]
        self.w_o = tensors[p + "o"]
        self.x_bias, self.y_bias, self.conv_w, self.conv_b = f("x.b"), f("y.b"), f("conv"), f("conv.b")
        self.r_bias, self.i_bias = f("ra.b").reshape(-1), f("ri.b").reshape(-1)
        self.decay = (-self.decay_scale * torch.nn.functional.softplus(tensors[p + "lam"].double())).float().contiguous()

    def run_state_specs(self):
        return {CONV_STATE: StateSpec((max(self.taps - 1, 1), self.channels), torch.float32, 0.0),
                SCAN_STATE: StateSpec((self.channels,), torch.float32, 0.0)}

    def _gates(self, ctx, u):
        """The two gates' products of every group, 32 bit: [T, 2C], or [blocks, T, 2 sz] from the library's batched product."""
        T, C, nb, sz = u.shape[0], self.channels, self.blocks, self.block_size
        if u.dtype == torch.bfloat16 and T > linear.SMALL_M and "products" not in ctx.plain_kernels:
            ops.count_launch()
            g = torch.bmm(u.view(T, nb, sz).transpose(0, 1), self.w_gates.transpose(1, 2), out_dtype=torch.float32)
            ops.count_library()
            return g
        g = torch.empty((T, 2 * C), dtype=torch.float32, device=u.device)
        ops.gemm_nt_plain_batched(u.data_ptr(), self.w_gates.data_ptr(), g.data_ptr(), T, 2 * sz, sz, C, sz, 2 * C, nb, sz, 2 * sz * sz,
                                  2 * sz, u.dtype, torch.float32)
        return g

    def forward(self, ctx, x, cache):
        C = self.channels
        T = x.shape[0]
        rows = dict(row_slot=ctx.row_slot, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len)
        xy = linear.linear(ctx, x, self.w_in)                                   # [T, 2C]: x | y, before biases and activations
        u = torch.empty((T, C), dtype=x.dtype, device=x.device)
        ops.conv_silu(xy, 2 * C, self.conv_w, self.conv_b, cache.state[CONV_STATE], u, tok_row=ctx.tok_row, in_bias=self.x_bias,
                      silu=False, **rows)
        gates = self._gates(ctx, u)
        seg = {}
        if not ctx.replayable and ctx.max_q_len > SEGMENT:
            segs = -(-ctx.max_q_len // SEGMENT)
            n = ctx.num_rows * segs * C
            seg = dict(seg_len=SEGMENT, segs=segs, seg_state=ctx.scratch("gated_recurrence.segments", (n,), torch.float32),
                       seg_decay=ctx.scratch("gated_recurrence.segment_decays", (n,), torch.float32))
        h = torch.empty((T, C), dtype=x.dtype, device=x.device)
        ops.gated_recurrence(u, gates, self.block_size, self.r_bias, self.i_bias, self.decay, xy.data_ptr() + C * xy.element_size(),
                             2 * C, self.y_bias, cache.state[SCAN_STATE], h, gelu=True, **rows, **seg)
        return linear.linear(ctx, h, self.w_o, out_dtype=torch.float32 if self.wide_output else None)
