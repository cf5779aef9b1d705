"""Attention over a paged cache of rows: every cached token of a key-value head is one row that holds its key
and its value, of sizes that may differ (``csrc/row_attention_params.h``).

``sink_attention``: grouped-query attention, H query heads on ``kv_heads`` key-value heads (query head h reads
key-value head h // (H / kv_heads)), with the options
  * ``window`` W: position i sees the keys j with i - W < j <= i (None: every j <= i);
  * ``sink``: a learned logit per head that joins the softmax's denominator and carries no value,
        p_j = exp(s_j) / (exp(sink_h) + sum_j' exp(s_j'));
  * ``position``: a rotary position encoding on the first ``rot_dims`` entries of every query and key head
    (None: positions do not enter the scores);
  * ``scale``: the factor on q . k (default 1 / sqrt(head_dim));
  * ``sink_logit``: a sink with this fixed logit for every head and no tensor (0: the softmax has one more in its
    denominator), instead of ``sink``;
  * ``unit_norm_eps``: after the rotation every query and key head is divided by its root mean square,
    sqrt(mean(x^2) + eps), with no weight (None: not);
  * ``value_from_key``: there is no value projection; a token's value is its key as projected, before rotation and norm.
  * ``bias``: the q, k, v and output projections have biases (``<name>.b``), added to the products in 32 bit;
  * ``qk_norm_eps``: before the rotation every query and key head goes through an RMS norm with a weight of the head's size
    (``q.norm`` / ``k.norm``, the same for every head): x / sqrt(mean(x^2) + eps) * w (None: not);
  * ``gate``: the heads' outputs are multiplied by sigmoid(W_g h) (``g`` [heads * value_dim, width], the mixer's own input h)
    before the output projection;
  * ``wide_output``: the output projection's result is handed on in 32 bit;
  * ``out_bias`` False (with ``bias``): only q, k and v have biases, the output projection has none;
  * ``qk_norm_whole`` (with ``qk_norm_eps``): one RMS norm over all columns of q at once and one over all of k, before they are cut into
    heads, with weights ``q.norm`` [heads * head_dim] and ``k.norm`` [kv_heads * head_dim];
  * ``q_temp`` {coef, every}: the query at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1);
  * ``softcap`` c: the scaled score s becomes c * tanh(s / c);
  * ``distance_bias`` {rows, far}: a learned table ``rel`` [rows, heads] whose row bucket(i - j) is added to the score of query i and
    key j (after the cap; the scale does not multiply it), with bucket(n) = n below rows/2 and
    min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))) from there on (``distance_buckets``);
  * ``shared_kv``: the layer has no key and value projections (nor their biases and norm); it reads the cache that another layer's
    run filled (the model's run order says which), with queries, sink and everything else of its own.
Scores and softmax weights are 32 bit in every kernel of the family.  ``run`` chooses the kernels for a batch.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from . import linear
from .base import MIXERS, PAGE, POSITION_ENCODINGS, CacheSpec, Mixer, PartSpec, TensorSpec


MAX_SPLITS = 32
SINGLE_WARP_BLOCKS_PER_SM = 6      # blocks of one warp (a tile of a single token's heads) that an SM holds at a time
PARTIALS = "row_attention.partials"


def plain(ctx) -> bool:
    return "attention" in ctx.plain_kernels or ctx.dtype != torch.bfloat16


def decode_splits(rows: int, kv_heads: int, group: int, max_keys: int, sm_count: int) -> int:
    """Blocks that share the keys of a (row, key-value head) in a step of single tokens: enough to fill the device (a group of
    up to 16 heads is one warp a block, of which an SM holds about six; larger groups take four warps a block, two blocks an SM),
    and so few that every block has two key tiles."""
    small = group <= 16
    blocks = max(1, rows * kv_heads * (1 if small else -(-group // 64)))
    tiles = max(1, -(-max_keys // (32 if small else 64)))
    return max(1, min((SINGLE_WARP_BLOCKS_PER_SM if small else 2) * sm_count // blocks, tiles // 2, MAX_SPLITS))


def run(ctx, params) -> None:
    """Runs attention over a cache of rows with the kernels that fit the batch.  bfloat16 with key and value sizes that
    are multiples of 16 goes to the tensor-core kernel: rows that bring several tokens in tiles of 64 query rows, rows
    that bring one token as a tile of their group's heads with the keys split over several blocks; a mixed step
    launches it once for each kind.  32 bit and other sizes go to the plain kernel.  In a replayable step nothing is
    chosen from the step's host data."""
    if plain(ctx) or not ops.attention_rows_mma_supported(params):
        params.row_filter = 0
        ops.attention_rows_plain(params)
        return
    group = params.H // params.KV
    singles = ctx.decode_only or any(n == 1 for n in ctx.host["q_lens"])
    several = not ctx.decode_only
    if singles:
        params.row_filter = 1 if several else 0
        splits, scratch = 1, None
        if not several:
            replay = getattr(ctx, "replayable", False)
            longest = ctx.cache.max_seq_len if replay else ctx.max_seq_len
            max_keys = min(longest, params.window + 64) if params.window else longest
            rows = params.rows
            splits = decode_splits(rows, params.KV, group, max_keys, ctx.sm_count)
            if splits > 1:
                n = ops.attention_rows_mma_scratch_floats(params.T, params.H, params.dv, splits)
                bound = ops.attention_rows_mma_scratch_floats(max(getattr(ctx, "max_rows", 0), rows), params.H, params.dv, MAX_SPLITS)
                scratch = ctx.scratch(PARTIALS + f".{params.dv}", (n,), torch.float32, bound=(bound,))
        ops.attention_rows_mma(params, group, splits, scratch)
    if several:
        params.row_filter = 2 if singles else 0
        ops.attention_rows_mma(params, ctx.max_q_len * group, 1, None)


def distance_buckets(rows: int, far: float) -> list:
    """bucket(n) for n = 0 .. ceil(far): from ceil(far) on every distance has the last bucket, so the list's last entry stands for
    all of them.  Distances below rows/2 have a bucket each; from there on the buckets' edges grow geometrically up to ``far``."""
    near = rows // 2
    if rows < 2 or far <= near:
        raise ValueError(f"a distance table of {rows} rows up to distance {far} has no room for its logarithmic half")
    out = []
    for n in range(int(math.ceil(far)) + 1):
        out.append(n if n < near else min(rows - 1, near + int(math.floor(math.log(n / near) / math.log(far / near) * (rows - near)))))
    return out


def make_params(ctx, *, q, q_stride, q_head_stride, out, cache, H, KV, dk, dv, row_width, k_off, v_off, scale, window=None,
                sink=None, softcap=None, dist_bias=None):
    return ops.row_attn_params(
        q=q, q_stride=q_stride, q_head_stride=q_head_stride, out=out, cache=cache.pages, block_table=cache.block_table,
        tok_row=ctx.tok_row, tok_pos=ctx.tok_pos, row_q_start=ctx.row_q_start, row_q_len=ctx.row_q_len,
        row_pos_start=ctx.row_pos_start, H=H, KV=KV, dk=dk, dv=dv, ps=cache.page_size, row_width=row_width, k_off=k_off,
        v_off=v_off, scale=scale, window=window or 0, sink=sink, softcap=softcap, dist_bias=dist_bias, err=ctx.err)


@MIXERS.register("sink_attention")
class SinkAttention(Mixer):
    """Tensor names: ``<prefix><q|k|v|o>`` (``names`` replaces them) and ``<prefix>sink`` [heads] when ``sink``."""

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 window: Optional[int] = None, sink: bool = False, scale: Optional[float] = None,
                 position: Optional[PartSpec] = None, rot_dims: Optional[int] = None, names: Optional[dict] = None,
                 sink_logit: Optional[float] = None, unit_norm_eps: Optional[float] = None, value_from_key: bool = False,
                 bias: bool = False, qk_norm_eps: Optional[float] = None, gate: bool = False, wide_output: bool = False,
                 out_bias: bool = True, qk_norm_whole: bool = False, q_temp: Optional[dict] = None, softcap: Optional[float] = None,
                 distance_bias: Optional[dict] = None, shared_kv: bool = False):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are no multiple of {kv_heads} key-value heads")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.kv_heads, self.dk = int(heads), int(kv_heads), int(head_dim)
        self.dv = int(value_dim) if value_dim else self.dk
        self.window = int(window) if window else None
        self.has_sink = bool(sink)
        self.sink_logit = float(sink_logit) if sink_logit is not None else None
        self.unit_norm_eps = float(unit_norm_eps) if unit_norm_eps is not None else None
        self.value_from_key = bool(value_from_key)
        self.has_bias, self.has_gate, self.wide_output = bool(bias), bool(gate), bool(wide_output)
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps is not None else None
        self.has_out_bias = self.has_bias and bool(out_bias)
        self.qk_norm_whole = bool(qk_norm_whole)
        if self.qk_norm_whole and self.qk_norm_eps is None:
            raise ValueError("a norm over all heads at once needs its eps (qk_norm_eps)")
        self.q_temp = (float(q_temp["coef"]), int(q_temp["every"])) if q_temp else None
        if self.q_temp and self.q_temp[1] < 1:
            raise ValueError(f"a query temperature that steps every {self.q_temp[1]} tokens")
        self.softcap = float(softcap) if softcap else None
        self.distance_bias = dict(rows=int(distance_bias["rows"]), far=float(distance_bias["far"])) if distance_bias else None
        if self.distance_bias:
            distance_buckets(**self.distance_bias)      # refuses sizes that make no table
        self.shared_kv = bool(shared_kv)
        if self.shared_kv and (value_from_key or gate):
            raise ValueError("a layer that reads another layer's keys and values has neither of its own to derive anything from")
        self.dist_table = None
        self.fold_out_bias = False      # set by a container that adds the output bias itself (``out_bias``) in a kernel of its own
        self.in_bias = self.out_bias = self.q_norm = self.k_norm = None
        if self.has_sink and self.sink_logit is not None:
            raise ValueError("a learned sink and a fixed sink logit exclude one another")
        if self.value_from_key and self.dv != self.dk:
            raise ValueError(f"values taken from keys have the keys' size: {self.dv} against {self.dk}")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.dk)
        self.position = position.build(POSITION_ENCODINGS) if position is not None else None
        self.rot_dims = int(rot_dims) if rot_dims else (self.dk if position is not None else 0)
        self.names = dict(q="q", k="k", v="v", o="o", sink="sink", g="g", rel="rel")
        self.names.update(names or {})
        self.w_qkv = self.w_o = self.sink = None

    def tensor_specs(self):
        p, n, d = self.prefix, self.names, self.width
        own_kv = not self.shared_kv
        has_v = own_kv and not self.value_from_key
        specs = [TensorSpec(p + n["q"], (self.heads * self.dk, d))]
        if own_kv:
            specs.append(TensorSpec(p + n["k"], (self.kv_heads * self.dk, d)))
        if has_v:
            specs.append(TensorSpec(p + n["v"], (self.kv_heads * self.dv, d)))
        specs.append(TensorSpec(p + n["o"], (d, self.heads * self.dv)))
        if self.has_sink:
            specs.append(TensorSpec(p + n["sink"], (self.heads,), kind="vector", init="uniform:-1:1"))
        if self.has_gate:
            specs.append(TensorSpec(p + n["g"], (self.heads * self.dv, d)))
        if self.has_bias:
            specs.append(TensorSpec(p + n["q"] + ".b", (self.heads * self.dk,), kind="vector", init="uniform:-0.1:0.1"))
            if own_kv:
                specs.append(TensorSpec(p + n["k"] + ".b", (self.kv_heads * self.dk,), kind="vector", init="uniform:-0.1:0.1"))
            if self.has_out_bias:
                specs.append(TensorSpec(p + n["o"] + ".b", (d,), kind="vector", init="uniform:-0.1:0.1"))
            if has_v:
                specs.append(TensorSpec(p + n["v"] + ".b", (self.kv_heads * self.dv,), kind="vector", init="uniform:-0.1:0.1"))
        if self.qk_norm_eps is not None:
            per = (lambda heads: heads * self.dk) if self.qk_norm_whole else (lambda heads: self.dk)
            specs.append(TensorSpec(p + n["q"] + ".norm", (per(self.heads),), kind="vector", init="norm"))
            if own_kv:
                specs.append(TensorSpec(p + n["k"] + ".norm", (per(self.kv_heads),), kind="vector", init="norm"))
        if self.distance_bias:
            specs.append(TensorSpec(p + n["rel"], (self.distance_bias["rows"], self.heads), kind="vector", init="uniform:-1:1"))
        return specs

    def bind(self, tensors):
        p, n = self.prefix, self.names
        own_kv = not self.shared_kv
        has_v = own_kv and not self.value_from_key
        mats = [tensors[p + n["q"]]] + ([tensors[p + n["k"]]] if own_kv else []) + ([tensors[p + n["v"]]] if has_v else [])
        if self.has_gate:      # the gate's rows ride behind q, k and v in one product
            mats.append(tensors[p + n["g"]])
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        if self.has_bias:
            parts = [tensors[p + n["q"] + ".b"]] + ([tensors[p + n["k"] + ".b"]] if own_kv else []) + ([tensors[p + n["v"] + ".b"]] if has_v else [])
            self.in_bias = torch.cat([t.float() for t in parts]).contiguous()
            self.out_bias = tensors[p + n["o"] + ".b"].float().contiguous() if self.has_out_bias else None
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[p + n["q"] + ".norm"].float().contiguous()
            self.k_norm = tensors[p + n["k"] + ".norm"].float().contiguous() if own_kv else None
        self.w_o = tensors[p + n["o"]]
        self.sink = tensors[p + n["sink"]].float().contiguous() if self.has_sink else None
        if self.sink_logit is not None:
            self.sink = torch.full((self.heads,), self.sink_logit, dtype=torch.float32, device=self.w_o.device)
        if self.distance_bias:      # the table by bucket, spread out by distance, a row a head: entry min(i - j, last) of [heads, last + 1]
            rel = tensors[p + n["rel"]].float()
            buckets = torch.tensor(distance_buckets(**self.distance_bias), dtype=torch.long, device=rel.device)
            self.dist_table = rel[buckets].t().contiguous()

    def cache_spec(self):
        # a page of a layer: [kv head][offset in the page][key | value]
        return CacheSpec((self.kv_heads, PAGE, self.dk + self.dv), self.window, run_tokens=128)

    def forward(self, ctx, x, cache):
        H, KV, dk, dv = self.heads, self.kv_heads, self.dk, self.dv
        if self.shared_kv and cache.writes:
            raise ValueError("a layer without keys and values of its own was given a cache to fill")
        qkv = linear.linear(ctx, x, self.w_qkv)
        table = self.position.table(x.device) if self.position is not None else None
        append = dict(H=H, KV=0 if self.shared_kv else KV, dk=dk, dv=dv, ps=cache.page_size, row_width=dk + dv, k_off=0, v_off=dk,
                      table=table, rot_dims=self.rot_dims, interleaved=bool(getattr(self.position, "interleaved", True)), err=ctx.err)
        pages = cache.pages if cache.writes else None
        if (self.unit_norm_eps is not None or self.value_from_key or self.has_bias or self.qk_norm_eps is not None or self.q_temp
                or self.shared_kv):
            ops.rows_append_unit(qkv, ctx.tok_pos, ctx.tok_row, cache.block_table, pages, unit_eps=self.unit_norm_eps,
                                 value_from_key=self.value_from_key, bias=self.in_bias, q_norm=self.q_norm, k_norm=self.k_norm,
                                 pre_eps=self.qk_norm_eps or 0.0, norm_whole=self.qk_norm_whole, q_temp=self.q_temp, **append)
        else:
            ops.rows_append(qkv, ctx.tok_pos, ctx.tok_row, cache.block_table, pages, **append)
        out = torch.empty((x.shape[0], H * dv), dtype=x.dtype, device=x.device)
        params = make_params(ctx, q=qkv, q_stride=qkv.shape[1], q_head_stride=dk, out=out, cache=cache, H=H, KV=KV, dk=dk, dv=dv,
                             row_width=dk + dv, k_off=0, v_off=dk, scale=self.scale, window=self.window, sink=self.sink,
                             softcap=self.softcap, dist_bias=self.dist_table)
        run(ctx, params)
        if self.has_gate:
            g_at = qkv.data_ptr() + ((H + KV) * dk + (0 if self.value_from_key else KV * dv)) * qkv.element_size()
            ops.sigmoid_gate(out, g_at, qkv.shape[1], out)
        y = linear.linear(ctx, out, self.w_o, out_dtype=torch.float32 if self.wide_output else None)
        if self.out_bias is not None and not self.fold_out_bias:
            ops.add_bias(y, self.out_bias)
        return y
