"""A residual stream of one copy kept in 32 bit, and the block whose sublayers run side by side on it.

``residual_f32``: x [T, d] float32.  It starts as
    x = table[token] * scale  (+ pair_table[(previous token * mul_prev + token * mul_cur) mod buckets])
where the pair table ("bigram embedding") is optional; a request's first token takes the table's last row, and the
token before a portion's first one is per-request state (``stream.prev_token``).  What a layer hands on as ``pending`` is
a ``Pending``: the outputs of its sublayers, not yet added, and what a re-entry adds.  The next norm adds them while it
reads the stream (one kernel, ``ops.residual_norm``): x <- x + (y1 + y2), then + the embedding output, then + the pass's
vector.  ``reentry`` describes a span of layers that runs several times: before every pass but the first the embedding
output (x as ``start`` made it) is added, and before every pass t the row t of the tensor ``reentry["name"]``
[passes, d].

A re-entry may instead be a projection (``reentry["project"]`` names a matrix W [d, 2 d]): before EVERY pass, the first
too, x <- W [x ; x0] with x0 the embedding output.  The matrix is cut into its two halves W = [A | B]: B x0 is the same for
every pass and is computed once per step; a pass then computes A x and hands B x0 on as the pending 32-bit stream that the
next norm adds, so the sum costs no kernel.

``parallel`` block: h = norm1(x); x <- x + (mixer(h) + feed_forward(h)); one norm, both sublayers read it; the
feed-forward may be absent.

``residual_pre_norm`` block: x <- x + mixer(norm1(x)); x <- x + feed_forward(norm2(x)); the second sublayer may be absent.

``sublayer_norm`` block: the norms sit on the sublayers' outputs and the sublayers read the stream itself,
x <- x + norm1(mixer(x)); x <- x + norm2(feed_forward(x)) (a norm may carry a scale per column behind it, "layer scale"); the second
sublayer may be absent.  Norm and sum are one kernel (``ops.sublayer_norm_add``), which also leaves the new stream in the compute
type for the next sublayer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..kernels import ops
from . import linear
from .base import BLOCKS, STREAMS, Block, StateSpec, Stream, TensorSpec

PREV_TOKEN = "stream.prev_token"
KEPT = "residual.embedding_output"
PROJECTED = "residual.projected_embedding"


@dataclass
class Pending:
    """What has not been added to the stream yet."""
    updates: tuple = ()                       # outputs of the last layer's sublayers [T, d], compute type
    extra: Optional[torch.Tensor] = None      # float32 [T, d]
    vec: Optional[torch.Tensor] = None        # float32 [d]
    rounded: Optional[torch.Tensor] = None    # the settled stream in the compute type, when nothing above is pending and a kernel
                                              # made it on its way (a block whose sublayers read the stream itself takes it)

    def empty(self) -> bool:
        return not self.updates and self.extra is None and self.vec is None


def read(ctx, x, pending: Optional[Pending], norm, rows=None, write_back=True):
    """Settles ``pending`` into x and returns norm(x) in the compute type (``norm``: a part with ``weight32()``, ``eps`` and
    ``kind``; None: the settled x itself in float32)."""
    p = pending or Pending()
    n = x.shape[0] if rows is None else rows.shape[0]
    if norm is None:
        out = torch.empty((n, x.shape[1]), dtype=torch.float32, device=x.device)
        return ops.residual_norm(x, out, updates=p.updates, extra=p.extra, vec=p.vec, rows=rows, write_back=write_back)
    out = torch.empty((n, x.shape[1]), dtype=ctx.dtype, device=x.device)
    bias = norm.bias32() if hasattr(norm, "bias32") else None
    return ops.residual_norm(x, out, updates=p.updates, extra=p.extra, vec=p.vec, weight=norm.weight32(), bias=bias, eps=norm.eps, kind=norm.kind,
                             rows=rows, write_back=write_back)


@STREAMS.register("residual_f32")
class ResidualStream(Stream):
    def __init__(self, width: int, scale: float = 1.0, pair: Optional[dict] = None, reentry: Optional[dict] = None,
                 rounded_start: bool = False):
        """``pair``: {name, buckets, mul_prev, mul_cur} of the hashed pair table [buckets + 1, d] (None: none).
        ``reentry``: {name, passes, add_embedding}, or {project, passes} (None: no span runs more than once).
        ``rounded_start``: the embedding kernel also leaves the stream in the compute type and ``initial_pending`` hands it to the
        first block (for blocks whose sublayers read the stream itself)."""
        self.rounded_start = bool(rounded_start)
        self._rounded = None
        self.width, self.scale = int(width), float(scale)
        self.pair = dict(pair) if pair else None
        self.reentry = dict(reentry) if reentry else None
        self.projects = bool(self.reentry and self.reentry.get("project"))
        self.pair_table = self.pass_vectors = self.w_stream = self.w_embed = None

    def tensor_specs(self):
        specs = []
        if self.pair:
            specs.append(TensorSpec(self.pair["name"], (int(self.pair["buckets"]) + 1, self.width), kind="table"))
        if self.projects:
            specs.append(TensorSpec(self.reentry["project"], (self.width, 2 * self.width), init="eye2"))
        elif self.reentry:
            specs.append(TensorSpec(self.reentry["name"], (int(self.reentry["passes"]), self.width), kind="vector", init="normal"))
        return specs

    def bind(self, tensors):
        if self.pair:
            self.pair_table = tensors[self.pair["name"]]
        if self.projects:
            w = tensors[self.reentry["project"]]
            self.w_stream, self.w_embed = w[:, :self.width].contiguous(), w[:, self.width:].contiguous()
        elif self.reentry:
            self.pass_vectors = tensors[self.reentry["name"]].float().contiguous()

    def state_specs(self):
        return {PREV_TOKEN: StateSpec((1,), torch.int32, -1)} if self.pair else {}

    def _keeps(self) -> bool:
        if self.projects:
            return True
        return bool(self.reentry and self.reentry.get("add_embedding", True) and int(self.reentry["passes"]) > 1)

    def start(self, ctx, table):
        T = ctx.num_tokens
        x = torch.empty((T, self.width), dtype=torch.float32, device=ctx.device)
        keep = None
        if self._keeps():
            keep = ctx.scratch(KEPT, (T, self.width), torch.float32, bound=(ctx.max_step_tokens, self.width))
        pair = self.pair or {}
        state = ctx.state(PREV_TOKEN) if self.pair else None
        self._rounded = None
        if self.rounded_start and ctx.dtype != torch.float32:
            self._rounded = torch.empty((T, self.width), dtype=ctx.dtype, device=ctx.device)
        ops.embedding_pair(ctx.tokens, table, x, scale=self.scale, pair_table=self.pair_table, buckets=pair.get("buckets", 0),
                           mul_prev=pair.get("mul_prev", 0), mul_cur=pair.get("mul_cur", 0), prev_state=state, tok_row=ctx.tok_row,
                           tok_pos=ctx.tok_pos, row_q_start=ctx.row_q_start, row_slot=ctx.row_slot, keep=keep, rounded=self._rounded, err=ctx.err)
        if self.pair:
            ops.remember_tokens(ctx.tokens, state, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len, row_slot=ctx.row_slot)
        self._kept = keep
        self._projected = None
        return x

    def initial_pending(self):
        return Pending(rounded=self._rounded) if self._rounded is not None else None

    def _enter_projected(self, ctx, x, pending):
        """x <- A x + B x0: the settled stream goes through A here, B x0 (made once per step) is left pending."""
        T = x.shape[0]
        if self._projected is None:
            e = torch.empty((T, self.width), dtype=ctx.dtype, device=x.device)
            ops.residual_norm(self._kept, e, write_back=False)          # the embedding output in the compute type
            self._projected = linear.linear_f32(ctx, e, self.w_embed)
        h = torch.empty((T, self.width), dtype=ctx.dtype, device=x.device)
        p = pending or Pending()
        ops.residual_norm(x, h, updates=p.updates, extra=p.extra, vec=p.vec, write_back=False)   # the settled stream, rounded once
        return linear.linear_f32(ctx, h, self.w_stream), Pending((), self._projected, None)

    def enter_pass(self, ctx, x, pending, number: int):
        if not self.reentry:
            raise ValueError("the stream was built without a re-entry and is told that a pass starts")
        if self.projects:
            return self._enter_projected(ctx, x, pending)
        p = pending or Pending()
        if p.extra is not None or p.vec is not None:      # two re-entries without a layer between them: settle the first
            ops.residual_norm(x, None, updates=p.updates, extra=p.extra, vec=p.vec)
            p = Pending()
        extra = self._kept if (number > 0 and self._keeps()) else None
        return x, Pending(p.updates, extra, self.pass_vectors[number])

    def finish(self, ctx, x, pending, norm, rows):
        return read(ctx, x, pending, norm, rows=rows, write_back=False)

    def total(self, ctx, x, pending):
        return read(ctx, x, pending, None, write_back=False)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    """One norm whose output the mixer and the feed-forward both read; their outputs are summed into the stream."""
    roles = ("norm1", "mixer")
    optional_roles = ("feed_forward",)

    def forward(self, ctx, x, pending, cache):
        h = read(ctx, x, pending, self.norm1)
        ys = (self.mixer.forward(ctx, h, cache),)
        if self.feed_forward is not None:
            ys = ys + (self.feed_forward.forward(ctx, h),)
        return x, Pending(ys)


@BLOCKS.register("residual_pre_norm")
class ResidualPreNormBlock(Block):
    """The pre-norm arrangement on the 32-bit stream; a layer may have no feed-forward (then it has no second norm either)."""
    roles = ("norm1", "mixer")
    optional_roles = ("norm2", "feed_forward")

    def __init__(self, parts):
        super().__init__(parts)
        if (self.norm2 is None) != (self.feed_forward is None):
            raise ValueError("the second norm and the feed-forward come together or not at all")

    def forward(self, ctx, x, pending, cache):
        h = read(ctx, x, pending, self.norm1)
        y = self.mixer.forward(ctx, h, cache)
        if self.feed_forward is None:
            return x, Pending((y,))
        f = read(ctx, x, Pending((y,)), self.norm2)
        return x, Pending((self.feed_forward.forward(ctx, f),))


@BLOCKS.register("sublayer_norm")
class SublayerNormBlock(Block):
    """Norms on the sublayers' outputs; a scale per column behind a norm is the norm's own (``layer_norm`` with ``scale``)."""
    roles = ("norm1", "mixer")
    optional_roles = ("norm2", "feed_forward")

    def __init__(self, parts):
        super().__init__(parts)
        if (self.norm2 is None) != (self.feed_forward is None):
            raise ValueError("the second norm and the feed-forward come together or not at all")

    def _settle(self, ctx, x, y, norm):
        out = None
        if ctx.dtype != torch.float32:
            out = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
        ops.sublayer_norm_add(x, y, out, weight=norm.weight32(), bias=norm.bias32() if hasattr(norm, "bias32") else None, eps=norm.eps,
                              kind=norm.kind)
        return x if out is None else out

    def forward(self, ctx, x, pending, cache):
        if pending is not None and pending.rounded is not None and pending.empty():
            h = pending.rounded
        elif ctx.dtype == torch.float32 and (pending is None or pending.empty()):
            h = x
        else:
            h = torch.empty(x.shape, dtype=ctx.dtype, device=x.device)
            p = pending or Pending()
            ops.residual_norm(x, h, updates=p.updates, extra=p.extra, vec=p.vec)      # settles what is pending; h = x rounded once
        h = self._settle(ctx, x, self.mixer.forward(ctx, h, cache), self.norm1)
        if self.feed_forward is not None:
            h = self._settle(ctx, x, self.feed_forward.forward(ctx, h), self.norm2)
        return x, Pending(rounded=h if h is not x else None)
