"""Loads the CUDA library and declares the C signature of every launcher.

There is one code path: the hand-written kernels.  If the library cannot be
built or loaded, or a tensor handed to a kernel is not on a CUDA device, the
call raises; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

import ctypes as C
import threading

from .build import build

_lock = threading.Lock()
_lib = None

P = C.c_void_p
I = C.c_int
F = C.c_float
D = C.c_double


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


class AttnParams(C.Structure):
    """Mirror of ``DkAttnParams`` in csrc/attention_params.h."""
    _fields_ = [
        ("q", P), ("out", P), ("kv", P), ("block_table", P), ("tok_row", P), ("tok_pos", P),
        ("row_slot", P), ("row_flags", P), ("row_q_start", P), ("row_q_len", P), ("row_pos_start", P),
        ("sel_pages", P), ("sel_count", P), ("dump", P), ("lse", P), ("scratch", P), ("err", P), ("rope_table", P),
        ("T", I), ("rows", I), ("H", I), ("KV", I), ("hd", I), ("ps", I), ("max_pages", I), ("num_pages", I),
        ("q_stride", I), ("window", I), ("sel_stride", I), ("dump_stride", I), ("dtype", I), ("splits", I),
        ("scale", F), ("block_entries", I), ("row_filter", I), ("fuse", I), ("rope_positions", I), ("reserved", I),
    ]


class RowAttnParams(C.Structure):
    """Mirror of ``DkRowAttnParams`` in csrc/row_attention_params.h."""
    _fields_ = [
        ("q", P), ("out", P), ("cache", P), ("block_table", P), ("tok_row", P), ("tok_pos", P), ("row_q_start", P),
        ("row_q_len", P), ("row_pos_start", P), ("sink", P), ("dist_bias", P), ("scratch", P), ("err", P),
        ("T", I), ("rows", I), ("H", I), ("KV", I), ("dk", I), ("dv", I), ("ps", I), ("max_pages", I), ("num_pages", I),
        ("q_stride", I), ("q_head_stride", I), ("row_width", I), ("k_off", I), ("v_off", I), ("window", I), ("dtype", I),
        ("splits", I), ("row_filter", I), ("scale", F), ("softcap", F), ("dist_max", I), ("reserved", I),
    ]


L = C.c_longlong

_SIGNATURES = {
    "dk_embedding_streams": [P, P, P, I, I, I, I, I, P, P],
    "dk_stream_norm": [P, P, P, P, P, P, P, P, I, I, I, F, I, I, I, P],
    "dk_activation": [P, P, L, I, I, P],
    "dk_softcap": [P, L, F, F, P],
    "dk_conv_silu": [P, I, P, P, P, P, P, P, P, P, I, I, I, I, P, I, I, P],
    "dk_selective_scan": [P, P, P, I, I, I, P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P, P],
    "dk_attention_rows_plain": [C.POINTER(RowAttnParams), P],
    "dk_rows_append": [P, I, P, P, P, I, P, I, P, I, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
    "dk_latent_prepare": [P, I, P, P, P, I, P, I, P, I, I, I, P, F, P, I, I, I, I, I, I, P, I, I, P, P],
    "dk_attention_rows_mma_supported": [C.POINTER(RowAttnParams)],
    "dk_attention_rows_mma": [C.POINTER(RowAttnParams), I, I, P, P],
    "dk_gemm_nt_plain_batched": [P, P, P, I, I, I, I, I, I, I, L, L, L, I, I, P],
    "dk_embedding": [P, P, P, I, I, I, I, P, P],
    "dk_rms_norm": [P, P, P, P, P, I, I, F, I, I, I, P],
    "dk_rms_norm_strided": [P, I, P, P, I, I, F, I, I, P],
    "dk_silu_mul": [P, P, I, I, I, P],
    "dk_rope_append": [P, P, P, P, I, P, I, P, I, I, I, I, I, I, I, I, P, P],
    "dk_gemm_nt_plain": [P, P, P, I, I, I, I, I, I, I, I, P],
    "dk_attention_plain": [C.POINTER(AttnParams), P],
    "dk_recent_pages": [P, P, P, P, P, P, I, I, I, D, I, P],
    "dk_page_scores": [P, P, P, P, P, P, P, I, I, I, I, I, I, D, I, P],
    "dk_select_pages": [P, P, P, P, P, P, P, I, I, I, I, I, F, D, I, P],
    "dk_sample": [P, I, I, I, P, P, P, P, P, P, P],
    "dk_attention_decode": [C.POINTER(AttnParams), P],
    "dk_attention_decode_supported": [I, I, I, I, I],
    "dk_attention_decode_blocks_per_sm": [I, I, I, I],
    "dk_attention_decode_max_clusters": [I, I, I, I, I],
    "dk_attention_prefill": [C.POINTER(AttnParams), I, P],
    "dk_attention_prefill_supported": [I, I, I, I, I],
    "dk_attention_prefill_tc": [C.POINTER(AttnParams), I, P],
    "dk_attention_prefill_tc_supported": [I, I, I, I, I, I],
    "dk_gemm_small_m": [P, P, P, I, I, I, I, I, I, I, I, P],
    "dk_gemm_small_m_supported": [I, I, I, I],
    "dk_gemm_tc": [P, P, P, I, I, I, I, I, I, I, I, I, I, P, P],
    "dk_gemm_tc_supported": [I, I, I, I],
    "dk_gemm_tc_many_rows_supported": [I, I, I, I],
    "dk_gemm_stream_k_supported": [I, I, I, I],
    "dk_gemm_stream_k": [P, P, P, I, I, I, I, I, I, I, I, P, P, P],
    "dk_wait_check": [P, C.c_longlong, P],
    "dk_embedding_pair": [P, P, P, P, P, P, P, F, P, L, L, L, P, P, P, I, I, I, I, P, P],
    "dk_remember_tokens": [P, P, P, P, P, I, P],
    "dk_residual_norm": [P, P, P, P, P, P, P, P, P, I, I, F, I, I, I, I, P],
    "dk_sublayer_norm_add": [P, P, P, P, P, I, I, F, I, I, I, P],
    "dk_rows_append_unit": [P, I, P, P, P, I, P, I, P, I, I, I, I, I, I, I, I, I, I, I, I, I, F, I, P, P, P, F, I, F, I, I, P, P],
    "dk_decay_attention_slice": [I, I, I, I],
    "dk_decay_attention": [P, I, I, I, I, I, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "dk_decay_attention_chunk": [],
    "dk_decay_attention_chunked_supported": [I, I],
    "dk_decay_attention_chunked": [P, I, I, I, I, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "dk_decay_attention_step_supported": [I, I],
    "dk_decay_attention_step": [P, I, I, I, I, I, P, P, P, P, P, I, I, I, I, I, P],
    "dk_normed_sum": [P, P, P, P, P, P, P, I, I, F, F, P],
    "dk_add_bias": [P, P, I, I, I, P],
    "dk_sigmoid_gate": [P, P, I, P, I, I, I, P],
    "dk_gated_recurrence": [P, P, L, L, I, P, P, P, P, I, P, I, P, P, P, P, P, I, I, I, I, P, P, I, P],
    "dk_matrix_memory_slice": [I, I, I, I],
    "dk_matrix_memory": [P, I, I, I, I, F, P, P, F, F, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "dk_matrix_memory_step_supported": [I, I],
    "dk_matrix_memory_step": [P, I, I, I, I, F, P, P, F, F, P, P, P, P, P, P, I, I, I, I, I, P],
    "dk_matrix_memory_chunk": [],
    "dk_matrix_memory_chunked_supported": [I, I],
    "dk_matrix_memory_chunked": [P, I, I, I, I, F, P, P, F, F, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    "dk_gated_rms_norm": [P, P, I, P, P, I, I, F, I, I, P],
    "dk_glu_clamped": [P, P, L, I, F, F, F, F, I, P],
    "dk_router_topk": [P, I, P, P, I, I, I, P],
    "dk_router": [P, P, P, P, P, I, I, I, I, I, P, F, I, I, P],
    "dk_experts_align": [P, I, I, P, I, P, I, I, P],
    "dk_experts_gather": [P, P, I, P, I, I, P, P],
    "dk_experts_gemm_tc_supported": [I, I, I],
    "dk_experts_gemm_tc": [P, P, P, P, P, I, I, I, I, I, I, I, I, F, F, F, P, P],
    "dk_experts_gemm": [P, P, P, P, P, I, I, I, I, I, F, F, F, P, I, P],
    "dk_experts_combine": [P, P, I, P, P, I, P, I, I, I, P],
    "dk_experts_tile_rows": [],
}


def load():
    """The loaded library (built at the first call)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build()
        lib = C.CDLL(str(path))
        lib.dk_last_error.restype = C.c_char_p
        lib.dk_last_error.argtypes = []
        lib.dk_sizeof_attn_params.restype = I
        lib.dk_attention_decode_scratch_floats.restype = C.c_longlong
        lib.dk_attention_decode_scratch_floats.argtypes = [I, I, I, I]
        lib.dk_gemm_stream_k_workspace_bytes.restype = C.c_longlong
        lib.dk_gemm_stream_k_workspace_bytes.argtypes = [I]
        lib.dk_sizeof_row_attn_params.restype = I
        lib.dk_attention_rows_mma_scratch_floats.restype = C.c_longlong
        lib.dk_attention_rows_mma_scratch_floats.argtypes = [I, I, I, I]
        if lib.dk_sizeof_row_attn_params() != C.sizeof(RowAttnParams):
            raise KernelError(f"RowAttnParams is {C.sizeof(RowAttnParams)} bytes in Python and "
                              f"{lib.dk_sizeof_row_attn_params()} in the library: the two declarations differ")
        if lib.dk_sizeof_attn_params() != C.sizeof(AttnParams):
            raise KernelError(f"AttnParams is {C.sizeof(AttnParams)} bytes in Python and "
                              f"{lib.dk_sizeof_attn_params()} in the library: the two declarations differ")
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = I
            fn.argtypes = args
        _lib = lib
    return _lib


def declare(name: str, argtypes: list) -> None:
    """Adds a launcher's signature (used by kernel files that come later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = I
        fn.argtypes = argtypes


LAUNCHES = [0]
PROFILE = None      # a list while launches are being timed: (name of the launcher, event recorded behind it)


def profile_start() -> None:
    """From now on an event is recorded behind every launcher (and every library product that is counted), so that the
    device time between two of them can be read afterwards with ``profile_stop``.  For measurements only: nothing is
    synchronised, but a recorded step cannot be captured into a graph meanwhile."""
    global PROFILE
    import torch
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    PROFILE = [("start", ev)]


def profile_mark(what: str) -> None:
    if PROFILE is not None:
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        PROFILE.append((what, ev))


def profile_stop() -> dict:
    """Stops timing and returns {launcher: (calls, milliseconds)}: the device time from the end of the launcher before
    to the end of this one, summed over its calls (launch gaps included; waits for the device)."""
    global PROFILE
    import torch
    marks, PROFILE = PROFILE or [], None
    torch.cuda.synchronize()
    out = {}
    for (_, e0), (what, e1) in zip(marks, marks[1:]):
        n, ms = out.get(what, (0, 0.0))
        out[what] = (n + 1, ms + e0.elapsed_time(e1))
    return out


def check(code: int, what: str, kernels: int = 1) -> None:
    """Raises when a launcher returned an error; counts the kernels it launched."""
    LAUNCHES[0] += kernels
    if PROFILE is not None:
        profile_mark(what)
    if code != 0:
        msg = load().dk_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg} (code {code})")
