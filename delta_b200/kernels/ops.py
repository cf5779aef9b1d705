"""Tensor-level entry points of the CUDA kernels.

Each function checks that its tensors are CUDA tensors of the expected type and
layout, and launches on torch's current stream.  Sizes that a kernel does not
take are refused with an error by the launcher itself; nothing is computed on
the CPU and no library model code is called.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import lib as _l
from .lib import AttnParams, KernelError

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"the kernels take float32 and bfloat16, not {dt}")


def _ptr(t: Optional[torch.Tensor], name: str, dtype=None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} is on '{t.device}': the kernels run on CUDA tensors only and there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


def _stream():
    """The current stream's handle.  (``torch.cuda.current_stream().cuda_stream`` makes a Python object and looks up
    the device three times over: 15 us a launch, the largest part of the host's time in a step that is not replayed.)"""
    return _raw_stream(_current_device())


def _device_index() -> int:
    return _current_device() if _current_device is not None else torch.cuda.current_device()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:      # a torch without these entry points: the public, slower way
    def _stream():  # noqa: F811
        return torch.cuda.current_stream().cuda_stream


def launch_count() -> int:
    """Kernels launched through this module so far (library products included)."""
    return _l.LAUNCHES[0]


def count_launch(n: int = 1) -> None:
    _l.LAUNCHES[0] += n


def count_library(what: str = "library product") -> None:
    """To be called behind a library kernel on the hot path: counts it and, while launches are timed, marks it."""
    if _l.PROFILE is not None:
        _l.profile_mark(what)


profile_start, profile_stop = _l.profile_start, _l.profile_stop


def new_error_record(device) -> torch.Tensor:
    """Four ints the kernels write {code, a, b, c} into when they meet a bad index."""
    return torch.zeros(4, dtype=torch.int32, device=device)


_ERR_TEXT = {1: "page id out of range (token {0}, logical page {1}, page id {2})",
             2: "token id out of range (row {0}: id {1}, vocabulary {2})",
             3: "position out of range (token {0}: position {1}, limit {2})",
             4: "a wait inside a kernel ran out (block {0}, part {1}, {2} steps); its result was not stored"}


def error_text(code: int, a: int, b: int, c: int) -> str:
    return "a kernel met a bad index and skipped it: " + _ERR_TEXT.get(code, "code {3}").format(a, b, c, code)


def raise_if_error(err: torch.Tensor) -> None:
    """Reads the record (this waits for the device), clears it and raises when it is set."""
    code, a, b, c = err.tolist()
    if code != 0:
        err.zero_()
        raise KernelError(error_text(code, a, b, c))


def wait_check(err: torch.Tensor, limit_ms: float = 1.0) -> None:
    """Launches a kernel whose only wait, bounded by ``limit_ms`` (at most 10), can never be satisfied:
    it gives up, records it in ``err`` and returns.  For checking that path; nothing else uses it."""
    _l.check(_l.load().dk_wait_check(_ptr(err, "err", torch.int32), int(limit_ms * 1e6), _stream()), "wait_check")


# ---------------------------------------------------------------------------

def embedding(tokens, table, out, err=None):
    T, d = out.shape
    _l.check(_l.load().dk_embedding(_ptr(tokens, "tokens", torch.int32), _ptr(table, "table"), _ptr(out, "out", table.dtype),
                                    T, d, table.shape[0], dtype_code(table.dtype), _ptr(err, "err", torch.int32), _stream()),
             "embedding")
    return out


def rms_norm(x, weight, eps, out, add=None, rows=None, cast_first=False):
    """out[r] = rmsnorm(x[s]) * weight with s = rows[r] (or r); when ``add`` is
    given, x[s] += add[s] first, in place.  ``rows`` must not name a row twice
    together with ``add``."""
    n_rows = out.shape[0]
    d = x.shape[-1]
    if add is not None and add.dtype != x.dtype:
        raise KernelError("rms_norm: add and x differ in dtype")
    _l.check(_l.load().dk_rms_norm(_ptr(x, "x"), _ptr(add, "add"), _ptr(weight, "weight"), _ptr(out, "out", x.dtype),
                                   _ptr(rows, "rows", torch.int32), n_rows, d, float(eps), dtype_code(x.dtype),
                                   dtype_code(weight.dtype), int(bool(cast_first)), _stream()), "rms_norm")
    return out


def rms_norm_strided(x, ld, weight, eps, out):
    """out[r] = rmsnorm(x[r, :d]) * weight for rows of ``x`` that lie ``ld`` elements apart, d = out.shape[1] (the first columns of
    a wider product's result); statistics and weight in 32 bit, rounded once."""
    n, d = out.shape
    if x.shape[0] != n or ld < d or x.numel() < (n - 1) * ld + d:
        raise KernelError(f"rms_norm_strided: {n} rows of {d} columns, {ld} apart, do not lie in a tensor of shape {tuple(x.shape)}")
    _l.check(_l.load().dk_rms_norm_strided(_ptr(x, "x"), int(ld), _ptr(weight, "weight"), _ptr(out, "out", x.dtype), n, d, float(eps),
                                           dtype_code(x.dtype), dtype_code(weight.dtype), _stream()), "rms_norm_strided")
    return out


def silu_mul(gate_up, out):
    T, I2 = gate_up.shape
    _l.check(_l.load().dk_silu_mul(_ptr(gate_up, "gate_up"), _ptr(out, "out", gate_up.dtype), T, I2 // 2,
                                   dtype_code(gate_up.dtype), _stream()), "silu_mul")
    return out


def rope_append(qkv, tok_pos, tok_row, block_table, kv, table, H, KV, hd, ps, interleaved, err=None):
    """Rotates q and k inside ``qkv`` [T, (H+2KV)*hd] and appends k, v to the pages
    of ``kv`` [pages, 2, KV, ps, hd].  ``table`` [positions, hd/2, 2] float holds
    cos and sin; None leaves q and k unrotated.  ``kv`` None appends nothing."""
    T = qkv.shape[0]
    if qkv.shape[1] != (H + 2 * KV) * hd:
        raise KernelError(f"rope_append: qkv has width {qkv.shape[1]}, expected {(H + 2 * KV) * hd}")
    if kv is not None and (tuple(kv.shape[1:]) != (2, KV, ps, hd) or kv.dtype != qkv.dtype):
        raise KernelError(f"rope_append: cache has shape {tuple(kv.shape)} / {kv.dtype}, expected [pages, 2, {KV}, {ps}, {hd}] of {qkv.dtype}")
    if table is not None and (table.dim() != 3 or table.shape[1] != hd // 2 or table.shape[2] != 2):
        raise KernelError(f"rope_append: table has shape {tuple(table.shape)}, expected [positions, {hd // 2}, 2]")
    _l.check(_l.load().dk_rope_append(
        _ptr(qkv, "qkv"), _ptr(tok_pos, "tok_pos", torch.int32), _ptr(tok_row, "tok_row", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1] if block_table is not None else 0,
        _ptr(kv, "kv"), kv.shape[0] if kv is not None else 0, _ptr(table, "table", torch.float32),
        table.shape[0] if table is not None else 0, T, H, KV, hd, ps, int(bool(interleaved)), dtype_code(qkv.dtype),
        _ptr(err, "err", torch.int32), _stream()), "rope_append")


def gemm_nt_plain(a, w, out):
    """out[M,N] = a[M,K] @ w[N,K]^T on the FMA units with float accumulation."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N) or a.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_nt_plain(_ptr(a, "a"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, K, K, N,
                                        dtype_code(a.dtype), dtype_code(out.dtype), _stream()), "gemm_nt_plain")
    return out


def attn_step_params(*, tok_row, tok_pos, row_slot=None, row_flags=None, row_q_start=None, row_q_len=None, row_pos_start=None,
                     err=None) -> AttnParams:
    """The part of the attention kernels' parameters that is the same for every layer of a step (the step's
    tokens and rows): made once per step and handed to ``make_attn_params`` as ``step``."""
    p = AttnParams()
    i32 = torch.int32
    p.tok_row = _ptr(tok_row, "tok_row", i32)
    p.tok_pos = _ptr(tok_pos, "tok_pos", i32)
    p.row_slot = _ptr(row_slot, "row_slot", i32)
    p.row_flags = _ptr(row_flags, "row_flags", i32)
    p.row_q_start = _ptr(row_q_start, "row_q_start", i32)
    p.row_q_len = _ptr(row_q_len, "row_q_len", i32)
    p.row_pos_start = _ptr(row_pos_start, "row_pos_start", i32)
    p.err = _ptr(err, "err", i32)
    p.T = tok_row.shape[0]
    return p


def make_attn_params(*, q, q_stride, out, kv, block_table, tok_row=None, tok_pos=None, H, KV, hd, ps, scale, row_slot=None,
                     row_flags=None, row_q_start=None, row_q_len=None, row_pos_start=None, sel_pages=None,
                     sel_count=None, dump=None, lse=None, scratch=None, err=None, window=0, splits=0, row_filter=0,
                     fuse=0, rope_table=None, step: Optional[AttnParams] = None) -> AttnParams:
    i32 = torch.int32
    if step is not None:
        p = AttnParams.from_buffer_copy(step)
    else:
        p = AttnParams()
        p.tok_row = _ptr(tok_row, "tok_row", i32)
        p.tok_pos = _ptr(tok_pos, "tok_pos", i32)
        p.row_slot = _ptr(row_slot, "row_slot", i32)
        p.row_flags = _ptr(row_flags, "row_flags", i32)
        p.row_q_start = _ptr(row_q_start, "row_q_start", i32)
        p.row_q_len = _ptr(row_q_len, "row_q_len", i32)
        p.row_pos_start = _ptr(row_pos_start, "row_pos_start", i32)
        p.err = _ptr(err, "err", i32)
        p.T = tok_row.shape[0]
    p.q = _ptr(q, "q")
    p.out = _ptr(out, "out", q.dtype)
    p.kv = _ptr(kv, "kv", q.dtype)
    if tuple(kv.shape[1:]) != (2, KV, ps, hd):
        raise KernelError(f"attention: cache has shape {tuple(kv.shape)}, expected [pages, 2, {KV}, {ps}, {hd}]")
    p.block_table = _ptr(block_table, "block_table", i32)
    p.sel_pages = _ptr(sel_pages, "sel_pages", i32)
    p.sel_count = _ptr(sel_count, "sel_count", i32)
    p.dump = _ptr(dump, "dump", torch.float32)
    p.lse = _ptr(lse, "lse", torch.float32)
    p.scratch = _ptr(scratch, "scratch")
    p.rows = block_table.shape[0]
    p.H, p.KV, p.hd, p.ps = H, KV, hd, ps
    p.max_pages = block_table.shape[1]
    p.num_pages = kv.shape[0]
    p.q_stride = q_stride
    p.window = int(window or 0)
    p.sel_stride = sel_pages.shape[1] if sel_pages is not None else 0
    p.dump_stride = dump.shape[-1] if dump is not None else 0
    p.dtype = dtype_code(q.dtype)
    p.splits = splits
    p.row_filter = row_filter
    p.fuse = fuse
    p.rope_table = _ptr(rope_table, "rope_table", torch.float32)
    p.rope_positions = rope_table.shape[0] if rope_table is not None else 0
    p.scale = float(scale)
    return p


def attention_plain(params: AttnParams):
    _l.check(_l.load().dk_attention_plain(C.byref(params), _stream()), "attention_plain")


def attention_decode_supported(dtype, H, KV, hd, ps) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_decode_supported(BF16, H, KV, hd, ps))


_decode_occupancy = {}


def attention_decode_blocks_per_sm(H, KV, hd, block_entries) -> int:
    """Blocks of the decode kernel one SM of the current device holds at once (asked of the runtime once)."""
    key = (_device_index(), H, KV, hd, block_entries)
    if key not in _decode_occupancy:
        n = int(_l.load().dk_attention_decode_blocks_per_sm(H, KV, hd, block_entries))
        if n < 1:
            raise KernelError("attention_decode: " + _l.load().dk_last_error().decode("utf-8", "replace"))
        _decode_occupancy[key] = n
    return _decode_occupancy[key]


def attention_decode_max_clusters(H, KV, hd, block_entries, splits) -> int:
    """Clusters of ``splits`` blocks of the decode kernel that the current device holds at once (asked of the runtime once)."""
    key = (_device_index(), H, KV, hd, block_entries, splits)
    if key not in _decode_occupancy:
        n = int(_l.load().dk_attention_decode_max_clusters(H, KV, hd, block_entries, splits))
        if n < 1:
            raise KernelError("attention_decode: " + _l.load().dk_last_error().decode("utf-8", "replace"))
        _decode_occupancy[key] = n
    return _decode_occupancy[key]


def attention_decode_scratch_floats(rows, H, hd, splits) -> int:
    return int(_l.load().dk_attention_decode_scratch_floats(rows, H, hd, splits))


def attention_decode(params: AttnParams):
    """One new token per row; ``params.splits`` blocks share a request's keys and, when there
    is more than one, ``params.scratch`` holds their partial results."""
    _l.check(_l.load().dk_attention_decode(C.byref(params), _stream()), "attention_decode", 2 if params.splits > 1 else 1)


def attention_prefill_supported(dtype, H, KV, hd, ps) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_prefill_supported(BF16, H, KV, hd, ps))


def attention_prefill(params: AttnParams, max_q_len: int):
    """Rows that bring several tokens (``params.row_filter`` 2 leaves single tokens to the
    decode kernel); ``max_q_len`` is the most tokens any row brings."""
    _l.check(_l.load().dk_attention_prefill(C.byref(params), int(max_q_len), _stream()), "attention_prefill")


def attention_prefill_tc_supported(dtype, H, KV, hd, ps, q_stride) -> bool:
    if dtype != torch.bfloat16:
        return False
    return bool(_l.load().dk_attention_prefill_tc_supported(BF16, H, KV, hd, ps, int(q_stride)))


def attention_prefill_tc(params: AttnParams, max_q_len: int):
    """The same rows as ``attention_prefill`` on the tcgen05 tensor cores: 128 queries a block,
    accumulators in tensor memory, pages fetched by TMA."""
    _l.check(_l.load().dk_attention_prefill_tc(C.byref(params), int(max_q_len), _stream()), "attention_prefill_tc")


def gemm_small_m_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_small_m_supported(M, N, K, int(swiglu)))


def gemm_small_m(x, w, out, swiglu=False):
    """out = x @ w^T for up to 64 rows of bfloat16 x, streaming w once.  ``swiglu``: w holds
    gate rows then up rows, and out [M, N/2] = silu(x gate^T) * (x up^T)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_small_m: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_small_m(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                       out.stride(0), dtype_code(out.dtype), int(swiglu), _stream()), "gemm_small_m")
    return out


def gemm_tc_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_tc_supported(M, N, K, int(swiglu)))


def gemm_tc_many_rows_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_tc_many_rows_supported(M, N, K, int(swiglu)))


def gemm_tc(x, w, out, swiglu=False, splits=1, err=None, per_sm=1):
    """out = x @ w^T for up to 128 rows of bfloat16 x on the tcgen05 tensor cores; the weights
    stream through shared memory by TMA.  ``splits`` blocks (1, 2, 4, 8) share K as a cluster.
    ``swiglu``: w holds gate rows then up rows, out [M, N/2] = silu(x gate^T) * (x up^T).
    ``per_sm`` 2: shorter stages, so that two blocks fit on an SM.
    More than 128 rows are taken in chunks of up to 256 (``splits`` and ``per_sm`` 1)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tc: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    _l.check(_l.load().dk_gemm_tc(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                  out.stride(0), dtype_code(out.dtype), int(swiglu), int(splits), int(per_sm),
                                  _ptr(err, "err", torch.int32), _stream()), "gemm_tc")
    return out


def gemm_stream_k_supported(M, N, K, swiglu=False) -> bool:
    return bool(_l.load().dk_gemm_stream_k_supported(M, N, K, int(swiglu)))


_stream_k_workspace = {}


def gemm_stream_k(x, w, out, swiglu=False, err=None):
    """out = x @ w^T for up to 128 rows of bfloat16 x as one persistent tcgen05 kernel: the
    (tile, K step) sequence is cut into one equal piece per SM, tiles that two pieces share are
    summed through a workspace in block order.  The workspace (partials and flags, zero at first)
    belongs to the device and is used by one stream at a time.
    ``swiglu``: w holds gate rows then up rows, out [M, N/2] = silu(x gate^T) * (x up^T)."""
    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if w.shape[1] != K or tuple(out.shape) != (M, n_out) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_stream_k: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} or dtypes do not fit")
    ws = _stream_k_workspace.get(x.device)
    if ws is None:
        ws = torch.zeros(int(_l.load().dk_gemm_stream_k_workspace_bytes(128)), dtype=torch.uint8, device=x.device)
        _stream_k_workspace[x.device] = ws
    _l.check(_l.load().dk_gemm_stream_k(_ptr(x, "x"), _ptr(w, "w"), _ptr(out, "out"), M, N, K, x.stride(0), w.stride(0),
                                        out.stride(0), dtype_code(out.dtype), int(swiglu), _ptr(ws, "workspace", torch.uint8),
                                        _ptr(err, "err", torch.int32), _stream()), "gemm_stream_k")
    return out


def recent_pages(row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count, ps, ratio, page_ahead=False):
    """``page_ahead``: a request whose newest page is exactly full counts one more, empty page (see delta_select.cu)."""
    i32 = torch.int32
    _l.check(_l.load().dk_recent_pages(_ptr(row_slot, "row_slot", i32), _ptr(row_flags, "row_flags", i32),
                                       _ptr(row_pos_start, "row_pos_start", i32), _ptr(row_q_len, "row_q_len", i32),
                                       _ptr(sel_pages, "sel_pages", i32), _ptr(sel_count, "sel_count", i32),
                                       row_slot.shape[0], sel_pages.shape[1], ps, float(ratio), int(page_ahead), _stream()), "recent_pages")


def page_scores(dump, lse, row_flags, row_q_start, row_pos_start, row_q_len, scores, ps, k, ratio, page_ahead=False):
    rows, H, stride = dump.shape
    i32 = torch.int32
    _l.check(_l.load().dk_page_scores(_ptr(dump, "dump", torch.float32), _ptr(lse, "lse", torch.float32),
                                      _ptr(row_flags, "row_flags", i32), _ptr(row_q_start, "row_q_start", i32),
                                      _ptr(row_pos_start, "row_pos_start", i32), _ptr(row_q_len, "row_q_len", i32),
                                      _ptr(scores, "scores", torch.float32), rows, H, ps, stride, scores.shape[1], k,
                                      float(ratio), int(page_ahead), _stream()), "page_scores")


def select_pages(scores, row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count, keep_last, ps, bias, ratio,
                 page_ahead=False):
    i32 = torch.int32
    _l.check(_l.load().dk_select_pages(_ptr(scores, "scores", torch.float32), _ptr(row_slot, "row_slot", i32),
                                       _ptr(row_flags, "row_flags", i32), _ptr(row_pos_start, "row_pos_start", i32),
                                       _ptr(row_q_len, "row_q_len", i32), _ptr(sel_pages, "sel_pages", i32),
                                       _ptr(sel_count, "sel_count", i32), scores.shape[0], scores.shape[1],
                                       sel_pages.shape[1], keep_last, ps, float(bias), float(ratio), int(page_ahead),
                                       _stream()), "select_pages")


def sample(logits, out, temperature=None, top_p=None, seeds=None, positions=None, err=None):
    """One token per row of float ``logits`` [R, V]: greedy where temperature is 0
    (or not given), else a draw from softmax(logits / temperature).  With ``err`` (the kernels'
    error record) ``out`` has four more ints than rows, and the record is copied behind the tokens."""
    R, V = logits.shape
    if err is not None:
        if out.shape[0] != R + 4:
            raise KernelError(f"sample: with an error record the output holds rows + 4 ints, got {out.shape[0]} for {R} rows")
        if R == 0:
            out.copy_(err)
            return out
    _l.check(_l.load().dk_sample(_ptr(logits, "logits", torch.float32), logits.stride(0) if R else V, R, V,
                                 _ptr(temperature, "temperature", torch.float32), _ptr(top_p, "top_p", torch.float32),
                                 _ptr(seeds, "seeds", torch.int64), _ptr(positions, "positions", torch.int32),
                                 _ptr(out, "out", torch.int32), _ptr(err, "err", torch.int32), _stream()), "sample")
    return out


# ---- a residual stream in 32 bit, one copy or several mixed ones ------------------------------------------

def embedding_streams(tokens, table, X, err=None):
    """X[t, s, :] = table[tokens[t]] for every copy s; X is float32 [T, S, d]."""
    T, S, d = X.shape
    _l.check(_l.load().dk_embedding_streams(_ptr(tokens, "tokens", torch.int32), _ptr(table, "table"), _ptr(X, "X", torch.float32),
                                            T, S, d, table.shape[0], dtype_code(table.dtype), _ptr(err, "err", torch.int32), _stream()),
             "embedding_streams")
    return X


def stream_norm(X, out, *, weight=None, eps=0.0, read=None, update=None, rows=None, write_back=True):
    """The step between two sublayers on a stream X [T, S, d] (float32).  ``update`` = (y, mix, out_w): the
    copies first become  X_t <- sum_s mix[s, t] X_s + out_w[t] y  (stored when ``write_back``); then
    u = sum_s read[s] X_s (``read`` None: the plain sum) and ``out`` = rmsnorm(u) * weight (``weight`` None: u
    itself).  ``rows``: only these tokens, in this order.  ``out`` None: only the update is done."""
    T, S, d = X.shape
    n = (rows.shape[0] if rows is not None else T)
    y = mix = out_w = None
    if update is not None:
        y, mix, out_w = update
        if tuple(y.shape) != (T, d):
            raise KernelError(f"stream_norm: the update has shape {tuple(y.shape)}, the stream rows {(T, d)}")
    if out is not None and tuple(out.shape) != (n, d):
        raise KernelError(f"stream_norm: the output has shape {tuple(out.shape)}, expected {(n, d)}")
    f32 = torch.float32
    _l.check(_l.load().dk_stream_norm(
        _ptr(X, "X", f32), _ptr(y, "y"), _ptr(mix, "mix", f32), _ptr(out_w, "out_w", f32), _ptr(read, "read", f32),
        _ptr(weight, "weight", f32), _ptr(out, "out"), _ptr(rows, "rows", torch.int32), n, S, d, float(eps),
        int(bool(write_back)), dtype_code(y.dtype) if y is not None else (dtype_code(out.dtype) if out is not None else F32),
        dtype_code(out.dtype) if out is not None else F32, _stream()), "stream_norm")
    return out


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2}


def activation(x, out, kind: str):
    """Element by element: relu(x)^2, gelu in its tanh form, or silu."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"unknown activation '{kind}'; known: {', '.join(ACTIVATIONS)}")
    _l.check(_l.load().dk_activation(_ptr(x, "x"), _ptr(out, "out", x.dtype), x.numel(), ACTIVATIONS[kind], dtype_code(x.dtype),
                                     _stream()), "activation")
    return out


def softcap(logits, cap: Optional[float], scale: float = 1.0):
    """logits <- logits * scale, then logits <- cap * tanh(logits / cap) (``cap`` None: no cap), in place (float32)."""
    _l.check(_l.load().dk_softcap(_ptr(logits, "logits", torch.float32), logits.numel(), float(cap or 0.0), float(scale), _stream()), "softcap")
    return logits


# ---- the selective state-space mixer ----------------------------------------------------------------------

def conv_silu(xin, in_stride, weight, bias, conv_state, out, *, tok_row, row_slot, row_q_start, row_q_len, in_bias=None, silu=True):
    """Causal convolution over each row's tokens and silu; ``xin`` holds a token's C inputs at the start of rows of
    ``in_stride`` elements.  ``conv_state`` [slots, taps-1, C] (float32) supplies the inputs before the step's first
    token and is left holding the last taps-1 inputs of every row.  ``in_bias`` (float32 [C]) is added to every input
    as it is read (the zeros before a request's first token stay zeros); ``silu`` False: no activation."""
    T, C_ = out.shape
    taps = weight.shape[1]
    i32, f32 = torch.int32, torch.float32
    _l.check(_l.load().dk_conv_silu(
        _ptr(xin, "xin", out.dtype), int(in_stride), _ptr(weight, "weight", f32), _ptr(bias, "bias", f32),
        _ptr(conv_state, "conv_state", f32), _ptr(out, "out"), _ptr(tok_row, "tok_row", i32), _ptr(row_slot, "row_slot", i32),
        _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32), T, row_slot.shape[0], C_, taps,
        _ptr(in_bias, "in_bias", f32), int(bool(silu)), dtype_code(out.dtype), _stream()), "conv_silu", 2 if taps > 1 else 1)
    return out


def selective_scan(x, dtraw, bc, b_off, c_off, z, z_stride, A_log, D, dt_bias, scan_state, out, *, row_slot, row_q_start,
                   row_q_len, seg_len=0, segs=1, seg_state=None, seg_dt=None):
    """The recurrence of the selective state-space mixer over each row's tokens, from and into ``scan_state``
    [slots, C, N] (float32).  ``bc`` [T, stride] holds a token's input map at ``b_off`` and output map at ``c_off``
    (N each); ``z`` points at the gate's C values in rows of ``z_stride`` elements.  ``seg_len`` > 0: rows are cut into
    segments of that many tokens which run in parallel (three kernels: every segment from zero, the segments' start states
    in order, every segment again from its start); ``segs`` is the most segments of any row, ``seg_state``
    [rows * segs, C, N] and ``seg_dt`` [rows * segs, C] (float32) are working memory."""
    T, C_ = x.shape
    N = A_log.shape[1]
    i32, f32 = torch.int32, torch.float32
    _l.check(_l.load().dk_selective_scan(
        _ptr(x, "x"), _ptr(dtraw, "dtraw", x.dtype), _ptr(bc, "bc", x.dtype), bc.shape[1], int(b_off), int(c_off), z, int(z_stride),
        _ptr(A_log, "A_log", f32), _ptr(D, "D", f32), _ptr(dt_bias, "dt_bias", f32), _ptr(scan_state, "scan_state", f32),
        _ptr(out, "out", x.dtype), _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32),
        _ptr(row_q_len, "row_q_len", i32), row_slot.shape[0], C_, N, dtype_code(x.dtype), int(segs), int(seg_len),
        _ptr(seg_state, "seg_state", f32), _ptr(seg_dt, "seg_dt", f32), _stream()), "selective_scan", 3 if seg_len else 1)
    return out


# ---- attention over a cache of rows -----------------------------------------------------------------------

RowAttnParams = _l.RowAttnParams


def row_attn_params(*, q, q_stride, q_head_stride, out, cache, block_table, tok_row, tok_pos, row_q_start, row_q_len,
                    row_pos_start, H, KV, dk, dv, ps, row_width, k_off, v_off, scale, window=0, sink=None, softcap=None, dist_bias=None,
                    err=None) -> RowAttnParams:
    """``softcap`` c: the scaled score s becomes c tanh(s / c).  ``dist_bias`` float32 [H, D + 1]: entry min(i - j, D) of a head's row
    is added to the scores of query i and key j (after the cap; the scale does not multiply it)."""
    i32 = torch.int32
    if tuple(cache.shape[1:]) != (KV, ps, row_width) or cache.dtype != q.dtype:
        raise KernelError(f"attention_rows: cache has shape {tuple(cache.shape)} / {cache.dtype}, expected [pages, {KV}, {ps}, {row_width}] of {q.dtype}")
    p = RowAttnParams()
    p.q, p.out, p.cache = _ptr(q, "q"), _ptr(out, "out", q.dtype), _ptr(cache, "cache")
    p.block_table = _ptr(block_table, "block_table", i32)
    p.tok_row, p.tok_pos = _ptr(tok_row, "tok_row", i32), _ptr(tok_pos, "tok_pos", i32)
    p.row_q_start, p.row_q_len = _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32)
    p.row_pos_start = _ptr(row_pos_start, "row_pos_start", i32)
    p.sink = _ptr(sink, "sink", torch.float32)
    if dist_bias is not None:
        if dist_bias.dim() != 2 or dist_bias.shape[0] != H or dist_bias.shape[1] < 1:
            raise KernelError(f"attention_rows: the distance biases have shape {tuple(dist_bias.shape)}, expected [{H}, distances]")
        p.dist_bias, p.dist_max = _ptr(dist_bias, "dist_bias", torch.float32), dist_bias.shape[1] - 1
    p.softcap = float(softcap or 0.0)
    p.err = _ptr(err, "err", i32)
    p.T, p.rows = tok_row.shape[0], block_table.shape[0]
    p.H, p.KV, p.dk, p.dv, p.ps = H, KV, dk, dv, ps
    p.max_pages, p.num_pages = block_table.shape[1], cache.shape[0]
    p.q_stride, p.q_head_stride = int(q_stride), int(q_head_stride)
    p.row_width, p.k_off, p.v_off = row_width, k_off, v_off
    p.window = int(window or 0)
    p.dtype = dtype_code(q.dtype)
    p.scale = float(scale)
    return p


def attention_rows_plain(params: RowAttnParams):
    _l.check(_l.load().dk_attention_rows_plain(C.byref(params), _stream()), "attention_rows_plain")


def rows_append(src, tok_pos, tok_row, block_table, cache, *, H, KV, dk, dv, ps, row_width, k_off, v_off, table=None,
                rot_dims=0, interleaved=True, err=None):
    """``src`` [T, (H+KV)*dk + KV*dv] holds q, k and v of every token.  q and k get rotary positions on the first
    ``rot_dims`` entries of each head (``table`` [positions, rot_dims/2, 2] of cos and sin; None: none), q in place;
    k and v are written to the token's rows of ``cache`` [pages, KV, ps, row_width] (None: nothing is appended)."""
    T = src.shape[0]
    if cache is not None and (tuple(cache.shape[1:]) != (KV, ps, row_width) or cache.dtype != src.dtype):
        raise KernelError(f"rows_append: cache has shape {tuple(cache.shape)} / {cache.dtype}, expected [pages, {KV}, {ps}, {row_width}] of {src.dtype}")
    if table is not None and tuple(table.shape[1:]) != (rot_dims // 2, 2):
        raise KernelError(f"rows_append: table has shape {tuple(table.shape)}, expected [positions, {rot_dims // 2}, 2]")
    i32 = torch.int32
    _l.check(_l.load().dk_rows_append(
        _ptr(src, "src"), src.shape[1], _ptr(tok_pos, "tok_pos", i32), _ptr(tok_row, "tok_row", i32),
        _ptr(block_table, "block_table", i32), block_table.shape[1] if block_table is not None else 0, _ptr(cache, "cache"),
        cache.shape[0] if cache is not None else 0, _ptr(table, "table", torch.float32), table.shape[0] if table is not None else 0,
        int(rot_dims), int(bool(interleaved)), T, H, KV, dk, dv, ps, row_width, k_off, v_off, dtype_code(src.dtype),
        _ptr(err, "err", i32), _stream()), "rows_append")


def latent_prepare(src, tok_pos, tok_row, block_table, cache, qabs, *, norm_weight, eps, H, dq, dr, R, ps, table=None, rot_dims=0,
                   interleaved=True, low=None, low_offset=0, err=None):
    """``src`` [T, H*(dq+dr) + R + dr]: per head the plain and the rotated query part, then the latent and the shared
    rotated key part; with ``low`` [T, >= low_offset + R + dr] the latent and the key part are read from its columns from
    ``low_offset`` on and ``src`` [T, H*(dq+dr)] holds the queries only.  Writes the normalised latent and the rotated key part to the token's row of ``cache``
    [pages, 1, ps, R+dr] and the heads' rotated query parts to ``qabs`` [T, H, R+dr] at [R, R+dr)."""
    T = src.shape[0]
    if cache is not None and (tuple(cache.shape[1:]) != (1, ps, R + dr) or cache.dtype != src.dtype):
        raise KernelError(f"latent_prepare: cache has shape {tuple(cache.shape)} / {cache.dtype}, expected [pages, 1, {ps}, {R + dr}] of {src.dtype}")
    if low is not None and (low.shape[0] != T or low.shape[1] - int(low_offset) < R + dr):
        raise KernelError(f"latent_prepare: rows of {low.shape[1]} entries do not hold the latent from column {low_offset} on")
    if tuple(qabs.shape) != (T, H, R + dr):
        raise KernelError(f"latent_prepare: qabs has shape {tuple(qabs.shape)}, expected {(T, H, R + dr)}")
    i32 = torch.int32
    _l.check(_l.load().dk_latent_prepare(
        _ptr(src, "src"), src.shape[1], _ptr(tok_pos, "tok_pos", i32), _ptr(tok_row, "tok_row", i32),
        _ptr(block_table, "block_table", i32), block_table.shape[1] if block_table is not None else 0, _ptr(cache, "cache"),
        cache.shape[0] if cache is not None else 0, _ptr(table, "table", torch.float32), table.shape[0] if table is not None else 0,
        int(rot_dims), int(bool(interleaved)), _ptr(norm_weight, "norm_weight", torch.float32), float(eps),
        _ptr(qabs, "qabs", src.dtype), T, H, dq, dr, R, ps,
        (_ptr(low, "low", src.dtype) + int(low_offset) * low.element_size()) if low is not None else None,
        low.shape[1] if low is not None else 0, dtype_code(src.dtype), _ptr(err, "err", i32), _stream()), "latent_prepare")


def gemm_nt_plain_batched(a_ptr, w_ptr, c_ptr, M, N, K, lda, ldw, ldc, batch, sa, sw, sc, in_dtype, out_dtype):
    """``batch`` products C_b[M,N] = A_b[M,K] W_b[N,K]^T on the FMA units with float accumulation; the operands of product b
    lie b*sa, b*sw and b*sc elements behind the given addresses (raw addresses: the operands may be interleaved views)."""
    _l.check(_l.load().dk_gemm_nt_plain_batched(a_ptr, w_ptr, c_ptr, M, N, K, lda, ldw, ldc, batch, sa, sw, sc,
                                                dtype_code(in_dtype), dtype_code(out_dtype), _stream()), "gemm_nt_plain_batched")


def attention_rows_mma_supported(params: RowAttnParams) -> bool:
    """True when the tensor-core kernel of the family takes these sizes (bfloat16; key and value sizes multiples of 16)."""
    return bool(_l.load().dk_attention_rows_mma_supported(C.byref(params)))


def attention_rows_mma_scratch_floats(T, H, dv, splits) -> int:
    return int(_l.load().dk_attention_rows_mma_scratch_floats(T, H, dv, splits))


def attention_rows_mma(params: RowAttnParams, max_m: int, splits: int = 1, scratch=None):
    """``max_m``: the most query rows (new tokens times heads of a group) of any batch row that ``params.row_filter`` lets
    through.  ``splits`` > 1: that many blocks share a row's keys and ``scratch`` (float32) takes their partial results."""
    _l.check(_l.load().dk_attention_rows_mma(C.byref(params), int(max_m), int(splits), _ptr(scratch, "scratch", torch.float32),
                                             _stream()), "attention_rows_mma", 2 if splits > 1 else 1)


def rows_append_unit(src, tok_pos, tok_row, block_table, cache, *, H, KV, dk, dv, ps, row_width, k_off, v_off, table=None,
                     rot_dims=0, interleaved=True, unit_eps=None, value_from_key=False, bias=None, q_norm=None, k_norm=None,
                     pre_eps=0.0, norm_whole=False, q_temp=None, err=None):
    """As ``rows_append``, one warp per head in 32 bit: after the rotation every query and key head is divided by its root
    mean square, sqrt(mean(x^2) + ``unit_eps``) (None: not), and rounded once.  ``value_from_key``: ``src`` holds no v;
    the value is the key as it was projected, before rotation and norm.  ``bias`` (float32, one entry per column of q, k
    and v) is added as the heads are read; ``q_norm`` / ``k_norm`` (float32 [dk]): the RMS norm with this weight and
    ``pre_eps`` on every query / key head before the rotation; ``norm_whole``: one norm over all of q's columns and one over
    all of k's, with weights [H*dk] and [KV*dk].  ``q_temp`` (coef, every): the query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1).  ``KV`` 0 with no cache: ``src`` holds queries only."""
    T = src.shape[0]
    if cache is not None and (tuple(cache.shape[1:]) != (KV, ps, row_width) or cache.dtype != src.dtype):
        raise KernelError(f"rows_append_unit: cache has shape {tuple(cache.shape)} / {cache.dtype}, expected [pages, {KV}, {ps}, {row_width}] of {src.dtype}")
    if table is not None and tuple(table.shape[1:]) != (rot_dims // 2, 2):
        raise KernelError(f"rows_append_unit: table has shape {tuple(table.shape)}, expected [positions, {rot_dims // 2}, 2]")
    i32 = torch.int32
    _l.check(_l.load().dk_rows_append_unit(
        _ptr(src, "src"), src.shape[1], _ptr(tok_pos, "tok_pos", i32), _ptr(tok_row, "tok_row", i32),
        _ptr(block_table, "block_table", i32), block_table.shape[1] if block_table is not None else 0, _ptr(cache, "cache"),
        cache.shape[0] if cache is not None else 0, _ptr(table, "table", torch.float32), table.shape[0] if table is not None else 0,
        int(rot_dims), int(bool(interleaved)), T, H, KV, dk, dv, ps, row_width, k_off, v_off, int(unit_eps is not None),
        float(unit_eps or 0.0), int(bool(value_from_key)), _ptr(bias, "bias", torch.float32), _ptr(q_norm, "q_norm", torch.float32),
        _ptr(k_norm, "k_norm", torch.float32), float(pre_eps), int(bool(norm_whole)), float(q_temp[0]) if q_temp else 0.0,
        int(q_temp[1]) if q_temp else 0, dtype_code(src.dtype), _ptr(err, "err", i32), _stream()), "rows_append_unit")


# ---- a residual stream of one 32-bit copy whose sublayers run side by side ---------------------------------------

NORM_KINDS = {"rms": 0, "layer": 1}


def embedding_pair(tokens, table, X, *, scale=1.0, pair_table=None, buckets=0, mul_prev=0, mul_cur=0, prev_state=None, tok_row=None,
                   tok_pos=None, row_q_start=None, row_slot=None, keep=None, rounded=None, err=None):
    """X[t] = table[tokens[t]] * scale (+ pair_table[(previous token * mul_prev + token * mul_cur) mod buckets]; a request's
    first token takes row ``buckets``; the token before a portion's first comes from ``prev_state`` [slots, 1]).  X, and
    ``keep`` when given (a second copy), are float32 [T, d]; ``rounded`` when given takes X in the table's type."""
    T, d = X.shape
    i32 = torch.int32
    _l.check(_l.load().dk_embedding_pair(
        _ptr(tokens, "tokens", i32), _ptr(tok_row, "tok_row", i32), _ptr(tok_pos, "tok_pos", i32), _ptr(row_q_start, "row_q_start", i32),
        _ptr(row_slot, "row_slot", i32), _ptr(prev_state, "prev_state", i32), _ptr(table, "table"), float(scale),
        _ptr(pair_table, "pair_table", table.dtype), int(buckets), int(mul_prev), int(mul_cur), _ptr(X, "X", torch.float32),
        _ptr(keep, "keep", torch.float32), _ptr(rounded, "rounded", table.dtype), T, d, table.shape[0], dtype_code(table.dtype), _ptr(err, "err", i32), _stream()), "embedding_pair")
    return X


def remember_tokens(tokens, prev_state, *, row_q_start, row_q_len, row_slot):
    """prev_state[slot of row] = the row's last token of this step."""
    i32 = torch.int32
    _l.check(_l.load().dk_remember_tokens(_ptr(tokens, "tokens", i32), _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32),
                                          _ptr(row_slot, "row_slot", i32), _ptr(prev_state, "prev_state", i32), row_slot.shape[0], _stream()),
             "remember_tokens")


def residual_norm(X, out, *, updates=(), extra=None, vec=None, weight=None, bias=None, eps=0.0, kind="layer", rows=None, write_back=True):
    """The step between two layers on a 32-bit stream X [T, d]:  X <- X + (y1 + y2) (``updates``: none, one or two tensors
    of the compute type), X <- X + ``extra`` (float32 [T, d]), X <- X + ``vec`` (float32 [d]), stored when ``write_back``;
    then ``out`` = norm(X) * weight with the layer norm without bias or the RMS norm (``weight`` None: X itself).
    ``bias`` (float32 [d]) is added behind the weight.  ``rows``: only these tokens, in this order.  ``out`` None: only the sums
    are done."""
    T, d = X.shape
    n = rows.shape[0] if rows is not None else T
    if len(updates) > 2:
        raise KernelError("residual_norm takes at most two updates")
    for y in updates:
        if tuple(y.shape) != (T, d):
            raise KernelError(f"residual_norm: an update has shape {tuple(y.shape)}, the stream {(T, d)}")
    if out is not None and tuple(out.shape) != (n, d):
        raise KernelError(f"residual_norm: the output has shape {tuple(out.shape)}, expected {(n, d)}")
    y1 = updates[0] if len(updates) > 0 else None
    y2 = updates[1] if len(updates) > 1 else None
    f32 = torch.float32
    ydt = dtype_code(y1.dtype) if y1 is not None else (dtype_code(out.dtype) if out is not None and out.dtype != f32 else F32)
    _l.check(_l.load().dk_residual_norm(
        _ptr(X, "X", f32), _ptr(y1, "update"), _ptr(y2, "update", y1.dtype if y1 is not None else None), _ptr(extra, "extra", f32),
        _ptr(vec, "vec", f32), _ptr(weight, "weight", f32), _ptr(bias, "bias", f32) if weight is not None else None, _ptr(out, "out"),
        _ptr(rows, "rows", torch.int32), n, d, float(eps),
        NORM_KINDS[kind], int(bool(write_back)), ydt, dtype_code(out.dtype) if out is not None else F32, _stream()), "residual_norm")
    return out


def sublayer_norm_add(X, y, out, *, weight, bias=None, eps=0.0, kind="layer"):
    """X <- X + norm(y) * weight + bias on a 32-bit stream X [T, d], with the norm of the sublayer's output y (compute type or
    float32) over the width; ``bias`` (float32 [d]) may be absent.  ``out`` (or None) takes the new X rounded to its type."""
    T, d = X.shape
    if tuple(y.shape) != (T, d) or (out is not None and tuple(out.shape) != (T, d)):
        raise KernelError(f"sublayer_norm_add: the stream is {(T, d)}, the sublayer's output {tuple(y.shape)}")
    f32 = torch.float32
    _l.check(_l.load().dk_sublayer_norm_add(
        _ptr(X, "X", f32), _ptr(y, "y"), _ptr(weight, "weight", f32), _ptr(bias, "bias", f32), _ptr(out, "out"),
        T, d, float(eps), NORM_KINDS[kind], dtype_code(y.dtype), dtype_code(out.dtype) if out is not None else F32, _stream()),
        "sublayer_norm_add")
    return out


# ---- linear attention with a decay per head ---------------------------------------------------------------------

def decay_attention_slice(rows, H, dk, dv) -> int:
    return int(_l.load().dk_decay_attention_slice(int(rows), H, dk, dv))


def decay_attention(src, q_off, k_off, v_off, decays, state, out, *, H, dk, dv, row_slot, row_q_start, row_q_len, silu=True, slice_=None):
    """Per row and head the recurrence  S <- decay_h S + k v^T,  o = S^T q  over the row's new tokens, from and into
    ``state`` [slots, H, dk, dv] (float32).  ``src`` [T, stride] holds a token's q at ``q_off``, k at ``k_off`` (H*dk each) and
    v at ``v_off`` (H*dv), before the activation when ``silu``; ``decays`` [H] float64; ``out`` float32 [T, H*dv]."""
    rows = row_slot.shape[0]
    if tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError(f"decay_attention: the state has shape {tuple(state.shape)}, expected [slots, {H}, {dk}, {dv}]")
    if tuple(out.shape) != (src.shape[0], H * dv):
        raise KernelError(f"decay_attention: the output has shape {tuple(out.shape)}, expected {(src.shape[0], H * dv)}")
    dvs = slice_ or decay_attention_slice(rows, H, dk, dv)
    i32 = torch.int32
    _l.check(_l.load().dk_decay_attention(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), int(bool(silu)), _ptr(decays, "decays", torch.float64),
        _ptr(state, "state", torch.float32), _ptr(out, "out", torch.float32), _ptr(row_slot, "row_slot", i32),
        _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32), rows, H, dk, dv, dvs, dtype_code(src.dtype),
        _stream()), "decay_attention")
    return out


def decay_attention_step_supported(dk, dv) -> bool:
    return bool(_l.load().dk_decay_attention_step_supported(int(dk), int(dv)))


def decay_attention_step(src, q_off, k_off, v_off, decays, state, out, *, H, dk, dv, row_slot, row_q_start, silu=True):
    """``decay_attention`` for steps in which every row brings one token: the state streams through registers once."""
    if tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError(f"decay_attention_step: the state has shape {tuple(state.shape)}, expected [slots, {H}, {dk}, {dv}]")
    i32 = torch.int32
    _l.check(_l.load().dk_decay_attention_step(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), int(bool(silu)), _ptr(decays, "decays", torch.float64),
        _ptr(state, "state", torch.float32), _ptr(out, "out", torch.float32), _ptr(row_slot, "row_slot", i32),
        _ptr(row_q_start, "row_q_start", i32), row_slot.shape[0], H, dk, dv, dtype_code(src.dtype), _stream()), "decay_attention_step")
    return out


def decay_attention_chunk() -> int:
    """Tokens of a chunk on the path that runs a row's chunks in parallel."""
    return int(_l.load().dk_decay_attention_chunk())


def decay_attention_chunked_supported(dk, dv) -> bool:
    return bool(_l.load().dk_decay_attention_chunked_supported(int(dk), int(dv)))


def decay_attention_chunked(src, q_off, k_off, v_off, decays, state, out, work, chunk_base, max_chunks, *, H, dk, dv, row_slot,
                            row_q_start, row_q_len, silu=True):
    """``decay_attention`` for long portions: every row is cut into chunks that run in parallel (three kernels: every chunk's own
    state, the states before the chunks in order, every chunk's outputs).  ``chunk_base`` [rows] int32: the chunks of all rows
    before each row; ``work`` float32 with room for (all chunks) x H x dk x dv; ``max_chunks``: the most chunks of a row."""
    rows = row_slot.shape[0]
    if tuple(state.shape[1:]) != (H, dk, dv):
        raise KernelError(f"decay_attention_chunked: the state has shape {tuple(state.shape)}, expected [slots, {H}, {dk}, {dv}]")
    i32 = torch.int32
    _l.check(_l.load().dk_decay_attention_chunked(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), int(bool(silu)), _ptr(decays, "decays", torch.float64),
        _ptr(state, "state", torch.float32), _ptr(out, "out", torch.float32), _ptr(work, "work", torch.float32),
        _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32),
        _ptr(chunk_base, "chunk_base", i32), rows, int(max_chunks), H, dk, dv, dtype_code(src.dtype), _stream()),
        "decay_attention_chunked", 3)
    return out


def gated_rms_norm(o, gate_ptr, gate_stride, weight, out, eps, group=None):
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate) per token; ``o`` float32 [T, n]; the gate's n values of a token
    lie at ``gate_ptr`` + t * ``gate_stride`` elements of the type of ``out``.  ``group``: the mean is taken over every ``group``
    consecutive entries (one head) instead of the whole row."""
    T, n = o.shape
    _l.check(_l.load().dk_gated_rms_norm(_ptr(o, "o", torch.float32), gate_ptr, int(gate_stride), _ptr(weight, "weight", torch.float32),
                                         _ptr(out, "out"), T, n, float(eps), int(group or n), dtype_code(out.dtype), _stream()), "gated_rms_norm")
    return out


# ---- sublayers side by side, an output gate, and two recurrent mixers ------------------------------------------------

def normed_sum(branches, out, eps, factor=1.0):
    """out = ``factor`` * sum over ``branches`` [(y, bias or None, weight)] of rms_norm(y + bias) * weight; one or two
    branches, everything float32, y [T, d]."""
    if not 1 <= len(branches) <= 2:
        raise KernelError("normed_sum takes one or two branches")
    f32 = torch.float32
    T, d = branches[0][0].shape
    args = []
    for y, b, w in list(branches) + [(None, None, None)] * (2 - len(branches)):
        if y is not None and tuple(y.shape) != (T, d):
            raise KernelError(f"normed_sum: a branch has shape {tuple(y.shape)}, another {(T, d)}")
        args += [_ptr(y, "branch", f32), _ptr(b, "bias", f32), _ptr(w, "weight", f32)]
    _l.check(_l.load().dk_normed_sum(*args, _ptr(out, "out", f32), T, d, float(eps), float(factor), _stream()), "normed_sum")
    return out


def add_bias(y, bias):
    """y[t] += bias (float32 [n]) in place; y [T, n] float32 or bfloat16."""
    T, n = y.shape
    _l.check(_l.load().dk_add_bias(_ptr(y, "y"), _ptr(bias, "bias", torch.float32), T, n, dtype_code(y.dtype), _stream()), "add_bias")
    return y


def sigmoid_gate(a, gate_ptr, gate_stride, out):
    """out = a * sigmoid(g) element by element; the gate's values of token t lie at ``gate_ptr`` + t * ``gate_stride``
    elements of the type of ``a``."""
    T, n = a.shape
    _l.check(_l.load().dk_sigmoid_gate(_ptr(a, "a"), gate_ptr, int(gate_stride), _ptr(out, "out", a.dtype), T, n, dtype_code(a.dtype),
                                       _stream()), "sigmoid_gate")
    return out


def gated_recurrence(u, gates, block_size, r_bias, i_bias, decay, y_ptr, y_stride, y_bias, state, out, *, row_slot, row_q_start, row_q_len,
                     gelu=True, seg_len=0, segs=1, seg_state=None, seg_decay=None):
    """The gated diagonal recurrence over each row's tokens, from and into ``state`` [slots, C] (float32):
    a = exp(decay * sigmoid(gr + r_bias)), S <- a S + sqrt(1 - a^2) sigmoid(gi + i_bias) u, out = S * act(y + y_bias).
    ``gates`` float32, [T, 2C] (per block of ``block_size`` channels the decay gate's products, then the input gate's) or
    [blocks, T, 2 block_size]; ``y_ptr``
    addresses the gate branch in rows of ``y_stride`` elements of the type of ``u``.  ``seg_len`` > 0: rows are cut into segments
    that run in parallel (three kernels), ``seg_state`` / ``seg_decay`` float32 [rows * segs * C] are working memory."""
    T, C_ = u.shape
    f32, i32 = torch.float32, torch.int32
    if tuple(gates.shape) == (T, 2 * C_):
        g_tok, g_block = 2 * C_, 2 * block_size
    elif tuple(gates.shape) == (C_ // block_size, T, 2 * block_size):
        g_tok, g_block = 2 * block_size, T * 2 * block_size
    else:
        raise KernelError(f"gated_recurrence: gates of shape {tuple(gates.shape)} do not fit {T} tokens of {C_} channels")
    if tuple(state.shape[1:]) != (C_,):
        raise KernelError(f"gated_recurrence: the state has shape {tuple(state.shape)}, expected [slots, {C_}]")
    _l.check(_l.load().dk_gated_recurrence(
        _ptr(u, "u"), _ptr(gates, "gates", f32), g_tok, g_block, int(block_size), _ptr(r_bias, "r_bias", f32), _ptr(i_bias, "i_bias", f32),
        _ptr(decay, "decay", f32), y_ptr, int(y_stride), _ptr(y_bias, "y_bias", f32), int(bool(gelu)), _ptr(state, "state", f32),
        _ptr(out, "out", u.dtype), _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32),
        row_slot.shape[0], C_, int(seg_len), int(segs), _ptr(seg_state, "seg_state", f32), _ptr(seg_decay, "seg_decay", f32),
        dtype_code(u.dtype), _stream()), "gated_recurrence", 3 if seg_len > 0 else 1)
    return out


def matrix_memory_slice(rows, H, dk, dv) -> int:
    return int(_l.load().dk_matrix_memory_slice(int(rows), H, dk, dv))


def matrix_memory(src, q_off, k_off, v_off, q_scale, gates, gate_bias, cap, guard, S, z, m, out, *, H, dk, dv, row_slot, row_q_start,
                  row_q_len, slice_=None):
    """The matrix memory with exponential gates over each row's tokens, from and into ``S`` [slots, H, dk, dv], ``z`` [slots, H, dk]
    and ``m`` [slots, H] (float32).  ``src`` [T, stride] holds a token's q, k (H*dk each) and v (H*dv) at the given offsets;
    ``gates`` float32 [T, 2H] the input gates' products, then the forget gates'; ``gate_bias`` [2H]; ``out`` float32 [T, H*dv]."""
    rows = row_slot.shape[0]
    T = src.shape[0]
    f32, i32 = torch.float32, torch.int32
    if tuple(S.shape[1:]) != (H, dk, dv) or tuple(z.shape[1:]) != (H, dk) or tuple(m.shape[1:]) != (H,):
        raise KernelError(f"matrix_memory: states of shapes {tuple(S.shape)}, {tuple(z.shape)}, {tuple(m.shape)} do not fit H={H} dk={dk} dv={dv}")
    if tuple(out.shape) != (T, H * dv) or tuple(gates.shape) != (T, 2 * H):
        raise KernelError(f"matrix_memory: out {tuple(out.shape)} or gates {tuple(gates.shape)} do not fit {T} tokens")
    dvs = slice_ or matrix_memory_slice(rows, H, dk, dv)
    _l.check(_l.load().dk_matrix_memory(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), float(q_scale), _ptr(gates, "gates", f32),
        _ptr(gate_bias, "gate_bias", f32), float(cap), float(guard), _ptr(S, "S", f32), _ptr(z, "z", f32), _ptr(m, "m", f32),
        _ptr(out, "out", f32), _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32), _ptr(row_q_len, "row_q_len", i32),
        rows, H, dk, dv, dvs, dtype_code(src.dtype), _stream()), "matrix_memory")
    return out


def matrix_memory_step_supported(dk, dv) -> bool:
    return bool(_l.load().dk_matrix_memory_step_supported(int(dk), int(dv)))


def matrix_memory_step(src, q_off, k_off, v_off, q_scale, gates, gate_bias, cap, guard, S, z, m, out, *, H, dk, dv, row_slot, row_q_start):
    """``matrix_memory`` for steps in which every row brings one token: one block per (row, head) streams the memory through
    registers once.  The value size is a multiple of 4."""
    rows = row_slot.shape[0]
    T = src.shape[0]
    f32, i32 = torch.float32, torch.int32
    if tuple(S.shape[1:]) != (H, dk, dv) or tuple(z.shape[1:]) != (H, dk) or tuple(m.shape[1:]) != (H,):
        raise KernelError(f"matrix_memory_step: states of shapes {tuple(S.shape)}, {tuple(z.shape)}, {tuple(m.shape)} do not fit H={H} dk={dk} dv={dv}")
    if tuple(out.shape) != (T, H * dv) or tuple(gates.shape) != (T, 2 * H):
        raise KernelError(f"matrix_memory_step: out {tuple(out.shape)} or gates {tuple(gates.shape)} do not fit {T} tokens")
    _l.check(_l.load().dk_matrix_memory_step(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), float(q_scale), _ptr(gates, "gates", f32),
        _ptr(gate_bias, "gate_bias", f32), float(cap), float(guard), _ptr(S, "S", f32), _ptr(z, "z", f32), _ptr(m, "m", f32),
        _ptr(out, "out", f32), _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32), rows, H, dk, dv,
        dtype_code(src.dtype), _stream()), "matrix_memory_step")
    return out


def matrix_memory_chunk() -> int:
    """Tokens of a chunk on the path that runs a row's chunks in parallel."""
    return int(_l.load().dk_matrix_memory_chunk())


def matrix_memory_chunked_supported(dk, dv) -> bool:
    return bool(_l.load().dk_matrix_memory_chunked_supported(int(dk), int(dv)))


def matrix_memory_chunked_work(total_chunks, H, dk, dv) -> int:
    """Floats of work space for that many chunks: every chunk's memory, keys' sum and four numbers."""
    return int(total_chunks) * H * (dk * dv + dk + 4)


def matrix_memory_chunked(src, q_off, k_off, v_off, q_scale, gates, gate_bias, cap, guard, S, z, m, out, work, chunk_base, total_chunks,
                          max_chunks, *, H, dk, dv, row_slot, row_q_start, row_q_len):
    """``matrix_memory`` for long portions: every row is cut into chunks that run in parallel (three kernels: every chunk alone from
    an empty memory, the memories and maxima before the chunks in order, every chunk's outputs).  ``chunk_base`` [rows] int32: the
    chunks of all rows before each row; ``work`` float32 of ``matrix_memory_chunked_work(total_chunks, ...)`` entries."""
    rows = row_slot.shape[0]
    T = src.shape[0]
    f32, i32 = torch.float32, torch.int32
    if tuple(S.shape[1:]) != (H, dk, dv) or tuple(z.shape[1:]) != (H, dk) or tuple(m.shape[1:]) != (H,):
        raise KernelError(f"matrix_memory_chunked: states of shapes {tuple(S.shape)}, {tuple(z.shape)}, {tuple(m.shape)} do not fit H={H} dk={dk} dv={dv}")
    if tuple(out.shape) != (T, H * dv) or tuple(gates.shape) != (T, 2 * H):
        raise KernelError(f"matrix_memory_chunked: out {tuple(out.shape)} or gates {tuple(gates.shape)} do not fit {T} tokens")
    if work.numel() < matrix_memory_chunked_work(total_chunks, H, dk, dv):
        raise KernelError(f"matrix_memory_chunked: {work.numel()} floats of work space are too few for {total_chunks} chunks")
    _l.check(_l.load().dk_matrix_memory_chunked(
        _ptr(src, "src"), src.shape[1], int(q_off), int(k_off), int(v_off), float(q_scale), _ptr(gates, "gates", f32),
        _ptr(gate_bias, "gate_bias", f32), float(cap), float(guard), _ptr(S, "S", f32), _ptr(z, "z", f32), _ptr(m, "m", f32),
        _ptr(out, "out", f32), _ptr(work, "work", f32), _ptr(row_slot, "row_slot", i32), _ptr(row_q_start, "row_q_start", i32),
        _ptr(row_q_len, "row_q_len", i32), _ptr(chunk_base, "chunk_base", i32), rows, int(total_chunks), int(max_chunks), H, dk, dv,
        dtype_code(src.dtype), _stream()), "matrix_memory_chunked", 3)
    return out


# ---- gated feed-forwards and a mixture of experts ---------------------------------------------------------------

def glu_clamped(gate_up, out, limit=-1.0, alpha=1.702, shift=1.0, cubic=0.0):
    """out = g' * sigmoid(alpha (g' + cubic g'^3)) * (u' + shift) from rows [g | u], g' = min(g, limit), u' = clamp(u, -limit, limit)
    (``limit`` negative: unclamped)."""
    rows, F2 = gate_up.shape
    _l.check(_l.load().dk_glu_clamped(_ptr(gate_up, "gate_up"), _ptr(out, "out", gate_up.dtype), rows, F2 // 2, float(limit), float(alpha),
                                      float(shift), float(cubic), dtype_code(gate_up.dtype), _stream()), "glu_clamped")
    return out


def router_topk(logits, experts, top, choice, weight):
    """Per token the ``top`` largest of the first ``experts`` columns of float32 ``logits`` and the softmax over them."""
    T = logits.shape[0]
    _l.check(_l.load().dk_router_topk(_ptr(logits, "logits", torch.float32), logits.shape[1], _ptr(choice, "choice", torch.int32),
                                      _ptr(weight, "weight", torch.float32), T, int(experts), int(top), _stream()), "router_topk")


def router(x, w, experts, top, logits, choice, weight, scoring="softmax", correction=None, scale=1.0, normalize=True):
    """logits = x w^T in 32 bit ([T, rows of w]; the first ``experts`` rows are the experts'), and per token the ``top`` largest of
    the experts' logits with the softmax over them.  ``scoring`` "sigmoid": scores s = sigmoid(logit); the ``top`` largest of
    s + ``correction`` (float32 [experts] or None) are chosen; the weights are the chosen s divided by their sum (``normalize``
    False: the chosen s themselves), times ``scale``."""
    T, d = x.shape
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"router: unknown scoring '{scoring}'")
    _l.check(_l.load().dk_router(_ptr(x, "x"), _ptr(w, "w", x.dtype), _ptr(logits, "logits", torch.float32), _ptr(choice, "choice", torch.int32),
                                 _ptr(weight, "weight", torch.float32), T, d, w.shape[0], int(experts), int(top),
                                 _ptr(correction, "correction", torch.float32), float(scale),
                                 (1 if normalize else 2) if scoring == "sigmoid" else 0,
                                 dtype_code(x.dtype), _stream()), "router")


def experts_tile_rows() -> int:
    return int(_l.load().dk_experts_tile_rows())


def experts_align(choice, experts, sorted_slots, tile_expert, tile_rows=None):
    """Sorts the (token, choice) slots by expert into tiles of ``tile_rows`` rows of one expert each: ``sorted_slots`` [tiles *
    tile_rows] holds slot numbers (token * top + choice) or -1, ``tile_expert`` [tiles] the expert of every tile or -1."""
    tile_rows = tile_rows or experts_tile_rows()
    _l.check(_l.load().dk_experts_align(_ptr(choice, "choice", torch.int32), choice.numel(), int(experts),
                                        _ptr(sorted_slots, "sorted_slots", torch.int32), sorted_slots.numel(),
                                        _ptr(tile_expert, "tile_expert", torch.int32), tile_expert.numel(), int(tile_rows), _stream()),
             "experts_align")


def experts_gather(x, sorted_slots, top, rows, row_scale=None):
    """rows[p] = x[sorted_slots[p] // top] (zeros where the slot is -1); bfloat16, the width a multiple of 8.  ``row_scale`` (float32,
    one entry a slot): rows[p] = row_scale[slot] * x[slot // top], rounded once."""
    _l.check(_l.load().dk_experts_gather(_ptr(x, "x", torch.bfloat16), _ptr(sorted_slots, "sorted_slots", torch.int32), int(top),
                                         _ptr(rows, "rows", torch.bfloat16), rows.shape[0], x.shape[1],
                                         _ptr(row_scale, "row_scale", torch.float32), _stream()), "experts_gather")
    return rows


def experts_gemm_tc_supported(n, k, glu=False) -> bool:
    return bool(_l.load().dk_experts_gemm_tc_supported(int(n), int(k), int(bool(glu))))


def experts_gemm_tc(rows, w, out, tile_expert, tile_rows, *, n, row_map=None, glu=False, limit=-1.0, alpha=1.702, shift=1.0, err=None):
    """The experts' products on the tcgen05 tensor cores: ``rows`` [tiles * tile_rows, k] (bfloat16, tiles of 128 or 256 rows of
    one expert each), ``w`` [E, n (2n with ``glu``: gate rows, then up rows), k]; ``out`` row r (or ``row_map[r]``; negative: not
    stored) takes the n results of row r, after the gated activation when ``glu``; ``glu`` "relu_squared": ``w`` [E, n, k] and
    relu(result)^2."""
    E, k = w.shape[0], w.shape[2]
    _l.check(_l.load().dk_experts_gemm_tc(_ptr(rows, "rows", torch.bfloat16), _ptr(w, "w", torch.bfloat16), _ptr(out, "out"),
                                          _ptr(tile_expert, "tile_expert", torch.int32), _ptr(row_map, "row_map", torch.int32),
                                          rows.shape[0], int(tile_rows), int(n), int(k), int(E), out.stride(0), dtype_code(out.dtype),
                                          2 if glu == "relu_squared" else int(bool(glu)), float(limit), float(alpha), float(shift),
                                          _ptr(err, "err", torch.int32), _stream()), "experts_gemm_tc")
    return out


def experts_gemm(a, w, out, sorted_slots, tile_expert, *, top, n, k, act=False, limit=-1.0, alpha=1.702, shift=1.0, row_scale=None):
    """For every tile of rows its expert's product (see ``csrc/experts.cu``).  ``act`` False: ``a`` holds the rows in sorted order, the
    result goes to the slots in 32 bit.  ``act`` True / "gated": rows gathered from the tokens, ``w`` [E, 2n, k] (gate rows, then up rows),
    the gated activation.  ``act`` "relu_squared": rows gathered, ``w`` [E, n, k], relu(product)^2.  ``row_scale`` (float32, one entry a
    slot; with an activation only): the product of slot s is multiplied by row_scale[s] before the activation, which is what an expert
    that read row_scale[s] * x would have got."""
    if row_scale is not None and not act:
        raise KernelError("experts_gemm: a scale per row belongs to the first product")
    code = {False: 0, True: 1, "gated": 1, "relu_squared": 2}.get(act)
    if code is None:
        raise KernelError(f"experts_gemm: unknown activation '{act}'")
    _l.check(_l.load().dk_experts_gemm(_ptr(a, "a"), _ptr(w, "w", a.dtype), _ptr(out, "out"), _ptr(sorted_slots, "sorted_slots", torch.int32),
                                       _ptr(tile_expert, "tile_expert", torch.int32), tile_expert.numel(), int(top), int(n), int(k),
                                       code, float(limit), float(alpha), float(shift), _ptr(row_scale, "row_scale", torch.float32),
                                       dtype_code(a.dtype), _stream()), "experts_gemm")


def experts_combine(z, weight, out, shared=None, gate_logit=None, gate_stride=0, top=None):
    """out[t] = sum_j weight[t, j] z[t*top + j] (+ sigmoid(gate logit of t) * shared[t]; no gate logit: + shared[t]); ``gate_logit``: an
    address (float32).  ``weight`` None with ``top``: every weight is 1."""
    T, d = out.shape
    _l.check(_l.load().dk_experts_combine(_ptr(z, "z", torch.float32), _ptr(weight, "weight", torch.float32),
                                          weight.shape[1] if weight is not None else int(top),
                                          _ptr(shared, "shared", out.dtype), gate_logit, int(gate_stride), _ptr(out, "out"), T, d,
                                          dtype_code(out.dtype), _stream()), "experts_combine")
    return out
