"""Latent attention: keys and values of all heads are linear maps of one small latent vector per token, and
only that vector (with one short rotated key part that all heads share) is cached.

Per token with mixer input h (H heads; per head ``head_dim`` plain and ``rot_dim`` rotated query/key entries,
value size ``value_dim``, latent size R):
    q_h          = [q_h^plain | q_h^rot]            rows of W_q h, head by head
    [low | r]    = W_dkv h                          R + rot_dim entries
    c            = rmsnorm(low) * w_c               the latent, cached
    r            rotated by its position            the shared key part, cached
    k_h^plain    = U_h^K c ,   v_h = U_h^V c
    s_h(i, j)    = (q_h^plain(i) . k_h^plain(j) + rot(q_h^rot(i)) . r(j)) * scale ,  causal softmax over j <= i
With ``q_rank`` Rq the queries go through a latent of their own, c_q = rmsnorm(W_dq h) * w_q, q = W_uq c_q (tensors ``dq``, ``dq.norm``,
``uq`` instead of ``q``): W_dq rides with W_dkv in the first product, and a second product makes the heads' queries.
The keys are never made: since q^plain . (U^K c) = ((U^K)^T q^plain) . c, the query is carried into the latent
space once per new token (one product per head), attention then runs with one shared key-value head whose key is the
cached row [c | r] and whose value is c, and U^V is applied to the attended latent afterwards.  So a step's cost
does not grow with the products that would rebuild keys and values of the whole context.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from . import linear, row_attention
from .base import MIXERS, PAGE, POSITION_ENCODINGS, CacheSpec, Mixer, PartSpec, TensorSpec


LIBRARY_BATCHED = True      # bfloat16 prompt portions: the library's batched product on strided views


def heads_product(ctx, a, a_off, lda, sa, w, n, k, c, c_off, ldc, sc, heads):
    """For every head b: C_b[T, n] = A_b[T, k] W_b[n, k]^T, where A_b starts ``a_off + b*sa`` elements into ``a`` with
    rows ``lda`` apart, W_b = w[b], and C_b starts ``c_off + b*sc`` elements into ``c`` with rows ``ldc`` apart."""
    T = a.shape[0]
    if T == 0:
        return
    es = a.element_size()
    if LIBRARY_BATCHED and a.dtype == torch.bfloat16 and "products" not in ctx.plain_kernels and T >= 16 and lda % 8 == 0 and ldc % 8 == 0 \
            and a_off % 8 == 0 and c_off % 8 == 0 and sa % 8 == 0 and sc % 8 == 0:
        # the library's batched product on strided views of the same memory
        ops.count_launch()
        av = torch.as_strided(a, (heads, T, k), (sa, lda, 1), a.storage_offset() + a_off)
        cv = torch.as_strided(c, (heads, T, n), (sc, ldc, 1), c.storage_offset() + c_off)
        torch.bmm(av, w.transpose(1, 2), out=cv)
        ops.count_library("library batched product")
        return
    ops.gemm_nt_plain_batched(a.data_ptr() + a_off * es, w.data_ptr(), c.data_ptr() + c_off * es, T, n, k, lda, k, ldc, heads,
                              sa, n * k, sc, a.dtype, c.dtype)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Tensor names under ``prefix``: ``q`` [H*(head_dim+rot_dim), d] (with ``q_rank`` Rq instead ``dq`` [Rq, d], ``dq.norm`` [Rq],
    ``uq`` [H*(head_dim+rot_dim), Rq]), ``dkv`` [R+rot_dim, d], ``dkv.norm`` [R], ``uk`` [H*head_dim, R], ``uv`` [H*value_dim, R],
    ``o`` [d, H*value_dim]."""

    def __init__(self, prefix: str, width: int, heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int,
                 eps: float, scale: Optional[float] = None, position: Optional[PartSpec] = None, rot_dims: Optional[int] = None,
                 q_rank: Optional[int] = None):
        self.q_rank = int(q_rank) if q_rank else 0
        self.w_uq = self.q_norm_w = None
        self.prefix, self.width = prefix, int(width)
        self.heads, self.dq, self.dr, self.dv, self.rank = int(heads), int(head_dim), int(rot_dim), int(value_dim), int(kv_rank)
        self.eps = float(eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dq + self.dr)
        self.position = position.build(POSITION_ENCODINGS) if (position is not None and self.dr > 0) else None
        self.rot_dims = int(rot_dims) if rot_dims else self.dr
        if self.position is not None and self.rot_dims > self.dr:
            raise ValueError(f"{self.rot_dims} rotated entries do not fit a rotated part of {self.dr}")
        self.w_in = self.w_ukT = self.w_uv = self.w_o = self.norm_w = None

    def tensor_specs(self):
        p, d, H = self.prefix, self.width, self.heads
        if self.q_rank:
            queries = [TensorSpec(p + "dq", (self.q_rank, d)), TensorSpec(p + "dq.norm", (self.q_rank,), kind="vector", init="norm"),
                       TensorSpec(p + "uq", (H * (self.dq + self.dr), self.q_rank))]
        else:
            queries = [TensorSpec(p + "q", (H * (self.dq + self.dr), d))]
        return queries + [TensorSpec(p + "dkv", (self.rank + self.dr, d)),
                TensorSpec(p + "dkv.norm", (self.rank,), kind="vector", init="norm"),
                TensorSpec(p + "uk", (H * self.dq, self.rank)), TensorSpec(p + "uv", (H * self.dv, self.rank)),
                TensorSpec(p + "o", (d, H * self.dv))]

    def bind(self, tensors):
        p, H = self.prefix, self.heads
        first = tensors[p + "dq"] if self.q_rank else tensors[p + "q"]
        self.w_in = torch.cat([first, tensors[p + "dkv"]], dim=0).contiguous()      # one product for q (or its latent) and the latent
        if self.q_rank:
            self.w_uq = tensors[p + "uq"]
            self.q_norm_w = tensors[p + "dq.norm"]
        self.norm_w = tensors[p + "dkv.norm"].float().contiguous()
        self.w_ukT = tensors[p + "uk"].view(H, self.dq, self.rank).transpose(1, 2).contiguous()  # [H, R, dq]: q^plain -> latent space
        self.w_uv = tensors[p + "uv"].view(H, self.dv, self.rank).contiguous()                   # [H, dv, R]
        self.w_o = tensors[p + "o"]

    def cache_spec(self):
        # a page of a layer: [one shared head][offset in the page][latent | rotated key part]
        return CacheSpec((1, PAGE, self.rank + self.dr), None, run_tokens=128)

    def forward(self, ctx, x, cache):
        H, dq, dr, dv, R = self.heads, self.dq, self.dr, self.dv, self.rank
        T = x.shape[0]
        width = R + dr
        src = linear.linear(ctx, x, self.w_in)                       # [T, H*(dq+dr) + R + dr], or [T, Rq + R + dr]
        low, low_offset = None, 0
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
            ops.rms_norm_strided(src, src.shape[1], self.q_norm_w, self.eps, cq)      # the first Rq columns of every row
            low, low_offset = src, self.q_rank
            src = linear.linear(ctx, cq, self.w_uq)                  # [T, H*(dq+dr)]
        qabs = torch.empty((T, H, width), dtype=x.dtype, device=x.device)
        table = self.position.table(x.device) if self.position is not None else None
        ops.latent_prepare(src, ctx.tok_pos, ctx.tok_row, cache.block_table, cache.pages if cache.writes else None, qabs,
                           norm_weight=self.norm_w, eps=self.eps, H=H, dq=dq, dr=dr, R=R, ps=cache.page_size, table=table,
                           rot_dims=self.rot_dims, interleaved=bool(getattr(self.position, "interleaved", True)), low=low,
                           low_offset=low_offset, err=ctx.err)
        # the plain query parts, carried into the latent space: qabs[t, h, :R] = q_h^plain(t) U_h^K
        heads_product(ctx, src, 0, src.shape[1], dq + dr, self.w_ukT, R, dq, qabs, 0, H * width, width, H)
        lat = torch.empty((T, H * R), dtype=x.dtype, device=x.device)
        params = row_attention.make_params(ctx, q=qabs, q_stride=H * width, q_head_stride=width, out=lat, cache=cache, H=H, KV=1,
                                           dk=width, dv=R, row_width=width, k_off=0, v_off=0, scale=self.scale)
        row_attention.run(ctx, params)
        vals = torch.empty((T, H * dv), dtype=x.dtype, device=x.device)
        heads_product(ctx, lat, 0, H * R, R, self.w_uv, dv, R, vals, 0, H * dv, dv, H)
        return linear.linear(ctx, vals, self.w_o)
