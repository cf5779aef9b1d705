"""A mixture of experts: every token runs ``top`` of ``experts`` small gated feed-forwards, chosen by a router.

    z = W_router h                                   router logits, 32 bit
    the ``top`` largest z pick the experts; their weights are the softmax over the chosen logits only
    expert e:  y = act(W_gate,e h, W_up,e h),  W_down,e y          (the gated activation of ``clamped_glu``)
    out = sum over the chosen experts of weight * expert(h)  (+ sigmoid(w_sg . h) * shared(h) when there is a shared expert,
          a feed-forward of the same form that every token runs)
Nothing about the routing is read on the host: the (token, choice) pairs are sorted by expert on the device into tiles of
rows of one expert, and the two products of all experts are one launch each: warp-level MMA over tiles of 64 rows
(``csrc/experts.cu``), or, when a step brings many rows an expert, the tcgen05 product over tiles of 128 rows gathered side
by side (``csrc/gemm_tc.cu``).  The router's rows and
the shared expert's gate row are one matrix, so one product gives both.

Options: ``scoring`` "sigmoid": scores s = sigmoid(z); the ``top`` largest of s + correction (a tensor ``correction`` [E] when
``correction`` is set) are chosen, and the weights are the chosen s (without the correction) divided by their sum (+ 1e-20), times
``route_scale``; ``normalize`` False: the chosen s themselves, times ``route_scale``.  ``weight_input``: a choice's weight multiplies
what its expert reads, out = sum expert(weight * h), not what it gives: since (w h) W^T = w (h W^T), the first product's result is
multiplied by the weight before the activation (the tcgen05 path multiplies the rows as it gathers them).  ``shared`` {intermediate, limit, alpha, shift, gate}: ``gate`` False leaves the shared expert's sigmoid gate (and the
tensor ``shared.sg``) out, so it is added as it is.  ``activation`` "relu_squared": an expert is  W_down relu(W_up h)^2  with no gate branch.  ``wide_output``: the
weighted sum is handed on in 32 bit (for a 32-bit residual stream), not rounded to the compute type.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .feed_forward import ClampedGLU


TC_TILE = 128               # rows of a tile on the tcgen05 path
TC_ROWS_PER_EXPERT = 96     # from this many rows an expert on average, the products go to the tcgen05 kernel


@FEED_FORWARDS.register("experts")
class Experts(FeedForward):
    """Tensor names under ``prefix``: ``router`` [E, d]; ``e<i>.gate|up`` [F, d], ``e<i>.down`` [d, F]; with a shared expert
    ``shared.gate|up|down`` and ``shared.sg`` [1, d]."""

    def __init__(self, prefix: str, width: int, experts: int, top: int, intermediate: int, limit=None, alpha: float = 1.702,
                 shift: float = 1.0, shared: Optional[dict] = None, scoring: str = "softmax", correction: bool = False,
                 route_scale: float = 1.0, activation: str = "clamped_glu", wide_output: bool = False, normalize: bool = True,
                 weight_input: bool = False):
        self.prefix, self.width = prefix, int(width)
        self.experts, self.top, self.intermediate = int(experts), int(top), int(intermediate)
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"{self.top} of {self.experts} experts cannot be chosen")
        if limit is not None and float(limit) < 0:
            raise ValueError(f"a clamp at {limit} is no limit")
        self.limit, self.alpha, self.shift = (-1.0 if limit is None else float(limit)), float(alpha), float(shift)
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown router scoring '{scoring}' (softmax, sigmoid)")
        if activation not in ("clamped_glu", "relu_squared"):
            raise ValueError(f"unknown expert activation '{activation}' (clamped_glu, relu_squared)")
        if correction and scoring != "sigmoid":
            raise ValueError("a correction of the choice belongs to sigmoid scores")
        self.scoring, self.has_correction, self.route_scale = scoring, bool(correction), float(route_scale)
        self.gated = activation == "clamped_glu"
        self.wide_output = bool(wide_output)
        if self.wide_output and shared:
            raise ValueError("the 32-bit output is for experts without a shared expert (whose output has the compute type)")
        self.normalize, self.weight_input = bool(normalize), bool(weight_input)
        if not self.normalize and scoring != "sigmoid":
            raise ValueError("weights that are not normalised belong to sigmoid scores")
        self.correction = None
        self.shared = None
        self.shared_gate = bool(shared.get("gate", True)) if shared else False
        if shared:
            self.shared = ClampedGLU(prefix + "shared.", width, int(shared["intermediate"]), limit=shared.get("limit"),
                                     alpha=shared.get("alpha", alpha), shift=shared.get("shift", shift))
        self.w_router = self.w1 = self.w2 = None

    def tensor_specs(self):
        p, d, F = self.prefix, self.width, self.intermediate
        specs = [TensorSpec(p + "router", (self.experts, d))]
        if self.has_correction:
            specs.append(TensorSpec(p + "correction", (self.experts,), kind="vector", init="uniform:-0.2:0.2"))
        for e in range(self.experts):
            specs += ([TensorSpec(f"{p}e{e}.gate", (F, d))] if self.gated else []) + [TensorSpec(f"{p}e{e}.up", (F, d)),
                                                                                     TensorSpec(f"{p}e{e}.down", (d, F))]
        if self.shared is not None:
            specs += self.shared.tensor_specs() + ([TensorSpec(p + "shared.sg", (1, d))] if self.shared_gate else [])
        return specs

    def bind(self, tensors):
        p = self.prefix
        rows = [tensors[p + "router"]] + ([tensors[p + "shared.sg"]] if self.shared_gate else [])
        self.w_router = torch.cat(rows, dim=0).contiguous()
        if self.gated:
            self.w1 = torch.stack([torch.cat([tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"]], dim=0) for e in range(self.experts)]).contiguous()
        else:
            self.w1 = torch.stack([tensors[f"{p}e{e}.up"] for e in range(self.experts)]).contiguous()
        self.correction = tensors[p + "correction"].float().contiguous() if self.has_correction else None
        self.w2 = torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def forward(self, ctx, x):
        T, d, E, top, F = x.shape[0], self.width, self.experts, self.top, self.intermediate
        dev, i32, f32 = x.device, torch.int32, torch.float32
        z = torch.empty((T, self.w_router.shape[0]), dtype=f32, device=dev)        # [T, E (+1)]
        choice = torch.empty((T, top), dtype=i32, device=dev)
        weight = torch.empty((T, top), dtype=f32, device=dev)
        ops.router(x, self.w_router, E, top, z, choice, weight, scoring=self.scoring, correction=self.correction, scale=self.route_scale,
                   normalize=self.normalize)
        act = "gated" if self.gated else "relu_squared"
        slots = T * top
        # weight_input: a slot's weight goes into the first product (or into the gathered rows), and the sum at the end has none
        row_scale = weight.view(-1) if self.weight_input else None
        # many rows an expert (prompt portions): tiles of 128 rows through the tcgen05 product; else tiles of 64 through warp-level MMA
        many = (x.dtype == torch.bfloat16 and "products" not in ctx.plain_kernels and slots >= TC_ROWS_PER_EXPERT * E and
                ops.experts_gemm_tc_supported(F, d, self.gated) and ops.experts_gemm_tc_supported(d, F, False))
        tile = TC_TILE if many else ops.experts_tile_rows()
        capacity = -(-(slots + (tile - 1) * min(E, slots)) // tile) * tile
        sorted_slots = torch.empty(capacity, dtype=i32, device=dev)
        tile_expert = torch.empty(capacity // tile, dtype=i32, device=dev)
        ops.experts_align(choice, E, sorted_slots, tile_expert, tile)
        y = torch.empty((capacity, F), dtype=x.dtype, device=dev)
        out_slots = torch.empty((slots, d), dtype=f32, device=dev)
        if many:
            rows = ops.experts_gather(x, sorted_slots, top, torch.empty((capacity, d), dtype=x.dtype, device=dev), row_scale=row_scale)
            ops.experts_gemm_tc(rows, self.w1, y, tile_expert, tile, n=F, glu=True if self.gated else act, limit=self.limit, alpha=self.alpha, shift=self.shift,
                                err=ctx.err)
            ops.experts_gemm_tc(y, self.w2, out_slots, tile_expert, tile, n=d, row_map=sorted_slots, err=ctx.err)
        else:
            ops.experts_gemm(x, self.w1, y, sorted_slots, tile_expert, top=top, n=F, k=d, act=act, limit=self.limit, alpha=self.alpha,
                             shift=self.shift, row_scale=row_scale)
            ops.experts_gemm(y, self.w2, out_slots, sorted_slots, tile_expert, top=top, n=d, k=F)
        out = torch.empty((T, d), dtype=f32 if self.wide_output else x.dtype, device=dev)     # wide: the weighted sum unrounded
        if self.weight_input:
            weight = None
        if self.shared is not None:
            s = self.shared.forward(ctx, x)
            ops.experts_combine(out_slots, weight, out, shared=s, gate_logit=(z.data_ptr() + E * 4) if self.shared_gate else None,
                                gate_stride=z.shape[1], top=top)
        else:
            ops.experts_combine(out_slots, weight, out, top=top)
        return out
