"""A matrix memory per head with exponential gates and a running maximum (the mLSTM of xLSTM).

With mixer input h, H heads, key size dk and value size dv:
    q = W_q h / sqrt(dk),  k = W_k h   [H, dk],    v = W_v h   [H, dv]
    li = cap tanh((W_i h + b_i) / cap),   lf = logsigmoid(cap tanh((W_f h + b_f) / cap))      one pair per head, 32 bit
    m' = max(lf + m, li);   S <- exp(lf + m - m') S + exp(li - m') k v^T;   z likewise from k alone
    o = S^T q / (max(|z . q|, exp(-m')) + guard)
    out = W_o ( o / rms(o per head) * w * sigmoid(W_g h) )
S [H, dk, dv], z [H, dk] and m [H] start at zero (m too: not at minus infinity), live in 32 bit, one set per run of the layer,
and are carried from step to step, so a prompt may be cut anywhere.  q, k, v and the output gate are one product; the two
gates' rows are a second, small product whose sums stay 32 bit.  Steps of single tokens stream the memory through registers once, one block per
(row, head); short portions and mixed steps take a row's tokens in turn, one block per (row, head, slice of the value entries)
(both in ``csrc/gated_recurrence.cu``); long portions run their chunks of 32 tokens in parallel (``csrc/matrix_memory_chunked.cu``).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from . import linear
from .base import MIXERS, Mixer, StateSpec, TensorSpec

PARALLEL_FROM = 65      # portions of at least this many tokens run their chunks in parallel
MEMORY = "memory"
NORMALIZER = "normalizer"
MAXIMUM = "maximum"


@MIXERS.register("matrix_memory")
class MatrixMemory(Mixer):
    """Tensor names under ``prefix``: ``q``, ``k`` [H*dk, d]; ``v``, ``g`` [H*dv, d]; ``i``, ``f`` [H, d] with ``i.b``, ``f.b`` [H];
    ``norm`` [H*dv]; ``o`` [d, H*dv]."""

    def __init__(self, prefix: str, width: int, heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 guard: float = 1e-6, wide_output: bool = False):
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dk, self.dv = int(heads), int(head_dim), int(value_dim)
        self.cap, self.eps, self.guard = float(gate_cap), float(eps), float(guard)
        if self.cap <= 0:
            raise ValueError("the gates' cap must be positive")
        self.wide_output = bool(wide_output)
        self.w_in = self.w_gates = self.w_o = self.gate_bias = self.norm_w = None

    def tensor_specs(self):
        p, d, H, dk, dv = self.prefix, self.width, self.heads, self.dk, self.dv
        return [TensorSpec(p + "q", (H * dk, d)), TensorSpec(p + "k", (H * dk, d)), TensorSpec(p + "v", (H * dv, d)),
                TensorSpec(p + "g", (H * dv, d)), TensorSpec(p + "i", (H, d)), TensorSpec(p + "f", (H, d)),
                TensorSpec(p + "i.b", (H,), kind="vector", init="uniform:-2:0"), TensorSpec(p + "f.b", (H,), kind="vector", init="uniform:1:4"),
                TensorSpec(p + "norm", (H * dv,), kind="vector", init="norm"), TensorSpec(p + "o", (d, H * dv))]

    def bind(self, tensors):
        p = self.prefix
        self.w_in = torch.cat([tensors[p + "q"], tensors[p + "k"], tensors[p + "v"], tensors[p + "g"]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors[p + "i"], tensors[p + "f"]], dim=0).contiguous()         # [2H, d]: input gates, forget gates
        self.gate_bias = torch.cat([tensors[p + "i.b"].float(), tensors[p + "f.b"].float()]).contiguous()
        self.w_o = tensors[p + "o"]
        self.norm_w = tensors[p + "norm"].float().contiguous()

    def run_state_specs(self):
        H, dk, dv = self.heads, self.dk, self.dv
        return {MEMORY: StateSpec((H, dk, dv), torch.float32, 0.0), NORMALIZER: StateSpec((H, dk), torch.float32, 0.0),
                MAXIMUM: StateSpec((H,), torch.float32, 0.0)}

    def forward(self, ctx, x, cache):
        H, dk, dv = self.heads, self.dk, self.dv
        T = x.shape[0]
        qkvg = linear.linear(ctx, x, self.w_in)                       # [T, 2 H dk + 2 H dv]: q | k | v | g
        gates = linear.linear_f32(ctx, x, self.w_gates)               # [T, 2H], before bias, cap and logsigmoid
        o = torch.empty((T, H * dv), dtype=torch.float32, device=x.device)
        st = cache.state
        rows = dict(row_slot=ctx.row_slot, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len)
        if not ctx.replayable and ctx.max_q_len >= PARALLEL_FROM and ops.matrix_memory_chunked_supported(dk, dv):
            # long portions: once the running maxima are known the recurrence is linear in the memory, so a row's chunks run in
            # parallel and are stitched together in order
            chunk = ops.matrix_memory_chunk()

            def layout():
                counts = [-(-n // chunk) for n in ctx.host["q_lens"]]
                base = [sum(counts[:i]) for i in range(len(counts))]
                return torch.tensor(base, dtype=torch.int32).to(x.device, non_blocking=True), sum(counts), max(counts)
            base, total, most = ctx.memo(("matrix_memory chunks", chunk), layout)
            bound = ops.matrix_memory_chunked_work(-(-ctx.max_step_tokens // chunk) + ctx.max_rows, H, dk, dv)
            work = ctx.scratch("matrix_memory.chunks", (ops.matrix_memory_chunked_work(total, H, dk, dv),), torch.float32, bound=(bound,))
            ops.matrix_memory_chunked(qkvg, 0, H * dk, 2 * H * dk, dk ** -0.5, gates, self.gate_bias, self.cap, self.guard, st[MEMORY],
                                      st[NORMALIZER], st[MAXIMUM], o, work, base, total, most, H=H, dk=dk, dv=dv, **rows)
        elif ctx.decode_only and ops.matrix_memory_step_supported(dk, dv):
            ops.matrix_memory_step(qkvg, 0, H * dk, 2 * H * dk, dk ** -0.5, gates, self.gate_bias, self.cap, self.guard, st[MEMORY],
                                   st[NORMALIZER], st[MAXIMUM], o, H=H, dk=dk, dv=dv, row_slot=ctx.row_slot, row_q_start=ctx.row_q_start)
        else:
            ops.matrix_memory(qkvg, 0, H * dk, 2 * H * dk, dk ** -0.5, gates, self.gate_bias, self.cap, self.guard, st[MEMORY],
                              st[NORMALIZER], st[MAXIMUM], o, H=H, dk=dk, dv=dv, **rows)
        y = torch.empty((T, H * dv), dtype=x.dtype, device=x.device)
        g_at = qkvg.data_ptr() + (2 * H * dk + H * dv) * qkvg.element_size()
        ops.gated_rms_norm(o, g_at, qkvg.shape[1], self.norm_w, y, self.eps, group=dv)
        return linear.linear(ctx, y, self.w_o, out_dtype=torch.float32 if self.wide_output else None)
