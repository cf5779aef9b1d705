"""A plain, slow implementation of the Mufalix design in float64, one function per mechanism.

It shares no code with the engine: whole sequences at once, no cache, no pages, a loop over tokens
where a recurrence runs.  ``forward`` takes the dict of config.json, a dict name -> tensor and the
token ids of one sequence, and returns the logits of every position and the residual stream after
every layer run.

Notation: T tokens, d width, H heads, G key-value heads, C channels of the recurrent branch.
"""
from __future__ import annotations

import math

import torch

F = torch.float64

# With ``rounding("bfloat16")`` active every product's result and every activation between products is
# rounded to bfloat16 once, as a 16-bit engine does; what the design keeps in 32 bit is not.
_round = [lambda x: x]


class rounding:
    def __init__(self, kind):
        self.fn = (lambda x: x.to(torch.bfloat16).to(F)) if kind == "bfloat16" else (lambda x: x)

    def __enter__(self):
        self.old = _round[0]
        _round[0] = self.fn

    def __exit__(self, *a):
        _round[0] = self.old


def rnd(x):
    return _round[0](x)


def lin(h, w, b=None):
    y = h @ w.to(F).T
    if b is not None:
        y = y + b.to(F)
    return rnd(y)


# ---------------------------------------------------------------- norms and activations

def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w.to(F)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


# ---------------------------------------------------------------- positions

def scaled_frequencies(base, dims, scaling):
    """Frequencies base^(-2i/dims), i < dims/2; with ``scaling`` {factor, low, high, original} long wavelengths are
    stretched by ``factor``, short ones kept, and those between blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / hi:
                pass
            elif wave > orig / lo:
                f = f / fac
            else:
                s = (orig / wave - lo) / (hi - lo)
                f = (1.0 - s) * f / fac + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate_half(x, positions, freq):
    """x [T, heads, n]: entry i of the first 2 len(freq) is paired with entry i + len(freq); the pair (a, b) at position p
    becomes (a cos - b sin, b cos + a sin) of the angle p freq_i.  The rest passes."""
    half = freq.numel()
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)


# ---------------------------------------------------------------- the windowed attention with a sink

def sink_window_attention(q, k, v, scale, window, sink):
    """q [T, H, n], k [T, G, n], v [T, G, m], sink [H] -> [T, H, m].  Query i sees keys j with 0 <= i - j < window; the
    softmax's denominator also holds exp(sink_h), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale                     # [T, T]
        i = torch.arange(T)
        seen = (i[:, None] - i[None, :] >= 0) & (i[:, None] - i[None, :] < window)
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(-1).values, sink[h].to(F).expand(T))
        e = torch.exp(s - top[:, None])
        den = e.sum(-1) + torch.exp(sink[h].to(F) - top)
        out[:, h] = (e / den[:, None]) @ v[:, g]
    return out


def gated_window_attention(cfg_m, W, p, h, positions, eps):
    H, G, n, m = cfg_m["heads"], cfg_m["kv_heads"], cfg_m["dim"], cfg_m["vdim"]
    T = h.shape[0]
    q = lin(h, W[p + "q"], W[p + "q.b"]).view(T, H, n)
    k = lin(h, W[p + "k"], W[p + "k.b"]).view(T, G, n)
    v = lin(h, W[p + "v"], W[p + "v.b"]).view(T, G, m)
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    rot = cfg_m.get("rot")
    if rot and rot["dims"]:
        freq = scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = rotate_half(q, positions, freq), rotate_half(k, positions, freq)
    q, k = rnd(q), rnd(k)
    window = (cfg_m.get("mask") or {}).get("size") or T + 1
    a = sink_window_attention(q, k, v, float(cfg_m["scale"]), int(window), W[p + "sink"])
    a = rnd(a).reshape(T, H * m)
    gate = torch.sigmoid(lin(h, W[p + "g"]))
    return lin(rnd(a * gate), W[p + "o"], W[p + "o.b"])


# ---------------------------------------------------------------- the gated linear recurrence

def causal_conv(x, w, b):
    """x [T, C], w [C, taps] whose last column meets the current token, zeros before the first token."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], dim=0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + padded[j:j + T] * w.to(F)[:, j]
    return y + b.to(F)


def block_diagonal(u, w, b):
    """u [T, C] in ``blocks`` equal parts; part j goes through the square matrix w[j] ([out, in]) and gets b[j]."""
    nb, sz, _ = w.shape
    T = u.shape[0]
    parts = u.view(T, nb, sz)
    return (torch.einsum("tbi,boi->tbo", parts, w.to(F)) + b.to(F)).reshape(T, nb * sz)


def gated_linear_recurrence(u, r, i, lam):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, with log a_t = -8 r_t softplus(lam)."""
    T, C = u.shape
    log_a = -8.0 * r * torch.nn.functional.softplus(lam.to(F))
    a = torch.exp(log_a)
    S = torch.zeros(C, dtype=F)
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] * a[t]) * i[t] * u[t]
        out[t] = S
    return out


def recurrent_branch(cfg_m, W, p, h):
    y = rnd(gelu_tanh(lin(h, W[p + "y"], W[p + "y.b"])))
    u = rnd(causal_conv(lin(h, W[p + "x"], W[p + "x.b"]), W[p + "conv"], W[p + "conv.b"]))
    r = torch.sigmoid(block_diagonal(u, W[p + "ra"], W[p + "ra.b"]))
    i = torch.sigmoid(block_diagonal(u, W[p + "ri"], W[p + "ri.b"]))
    S = gated_linear_recurrence(u, r, i, W[p + "lam"])
    return lin(rnd(S * y), W[p + "o"])


def side_by_side(cfg_m, W, p, h, positions, eps):
    """Both mixers read h; each output is RMS-normed over the width with its own weight; half their sum."""
    left = gated_window_attention(cfg_m["left"], W, p + "left.", h, positions, eps)
    right = recurrent_branch(cfg_m["right"], W, p + "right.", h)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


# ---------------------------------------------------------------- the matrix memory

def capped(z, cap):
    return cap * torch.tanh(z / cap)


def matrix_memory(q, k, v, log_i, log_f, with_condition=False):
    """q, k [T, H, n], v [T, H, m], log gates [T, H] -> [T, H, m].  Per head, with a running maximum mx that starts at 0:
    mx' = max(log_f + mx, log_i);  S' = exp(log_f + mx - mx') S + exp(log_i - mx') k v^T;  z likewise from k alone;
    out = S'^T q / (max(|z' . q|, exp(-mx')) + 1e-6)."""
    T, H, n = q.shape
    m = v.shape[-1]
    out = torch.zeros(T, H, m, dtype=F)
    cond = torch.zeros(T, H, dtype=F)
    for h in range(H):
        S = torch.zeros(n, m, dtype=F)
        z = torch.zeros(n, dtype=F)
        mx = torch.zeros((), dtype=F)
        for t in range(T):
            new = torch.maximum(log_f[t, h] + mx, log_i[t, h])
            keep, take = torch.exp(log_f[t, h] + mx - new), torch.exp(log_i[t, h] - new)
            S = keep * S + take * torch.outer(k[t, h], v[t, h])
            z = keep * z + take * k[t, h]
            mx = new
            den = torch.maximum((z @ q[t, h]).abs(), torch.exp(-mx)) + 1e-6
            out[t, h] = (S.T @ q[t, h]) / den
            cond[t, h] = (z * q[t, h]).abs().sum() / den
    return (out, cond) if with_condition else out


def matrix_memory_mixer(cfg_m, W, p, h, eps):
    H, n, m, cap = cfg_m["heads"], cfg_m["dim"], cfg_m["vdim"], float(cfg_m["gate_cap"])
    T = h.shape[0]
    q = rnd(lin(h, W[p + "q"]) * n ** -0.5).view(T, H, n)
    k = lin(h, W[p + "k"]).view(T, H, n)
    v = lin(h, W[p + "v"]).view(T, H, m)
    log_i = capped(h @ W[p + "i"].to(F).T + W[p + "i.b"].to(F), cap)
    log_f = torch.nn.functional.logsigmoid(capped(h @ W[p + "f"].to(F).T + W[p + "f.b"].to(F), cap))
    o = matrix_memory(q, k, v, log_i, log_f)
    o = rms(o, eps).reshape(T, H * m) * W[p + "norm"].to(F)
    return lin(rnd(o * torch.sigmoid(lin(h, W[p + "g"]))), W[p + "o"])


# ---------------------------------------------------------------- the experts

MARGINS = None      # a list: every call of ``route`` appends its tokens' margins [T] here and their choices [T, top] to CHOICES
CHOICES = []


def route(h, w_router, correction, top, scale):
    """Sigmoid scores; the ``top`` largest of score + correction are chosen (lowest index among equals); their weights are
    the scores without the correction, divided by their sum, times ``scale``.  Returns (choice [T, top], weight [T, top])."""
    s = torch.sigmoid(h @ w_router.to(F).T)
    pick = s + correction.to(F)
    ranked = torch.sort(pick, dim=-1, descending=True, stable=True)
    order = ranked.indices[:, :top]
    if MARGINS is not None:      # how far the last chosen expert is ahead of the first one left out, and the choice as a set
        MARGINS.append(ranked.values[:, top - 1] - ranked.values[:, top] if top < pick.shape[-1] else torch.full_like(pick[:, 0], 9.0))
        CHOICES.append(torch.sort(order, dim=-1).values)
    w = torch.gather(s, 1, order)
    return order, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def experts(cfg_mlp, W, p, h):
    r = cfg_mlp["router"]
    choice, weight = route(h, W[p + "router"], W[p + "correction"], int(r["top"]), float(r.get("scale", 1.0)))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(choice.shape[1]):
            e = int(choice[t, j])
            mid = rnd(relu_squared(lin(h[t:t + 1], W[f"{p}e{e}.up"])))
            out[t] += weight[t, j] * (mid @ W[f"{p}e{e}.down"].to(F).T)[0]
    return out


# ---------------------------------------------------------------- the whole model

def run_order(cfg):
    """[(layer, starts a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(a)]
    for _ in range(times):
        order += [(i, i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def forward(cfg, W, tokens):
    """(logits [T, vocab], stream after every layer run [runs, T, d]) of one sequence, float64."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    positions = torch.arange(T)
    eps = float(cfg["norm"]["eps"])
    x0 = W["embed"].to(F)[tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = x0
    after = []
    for i, starts in run_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if starts:
            x = (torch.cat([rnd(x), rnd(x0)], dim=-1) @ W["loop.in"].to(F).T)
        h = rnd(rms_norm(x, W[p + "norm1"], eps))
        if L["type"] == "parallel":
            x = x + side_by_side(L["mixer"], W, p + "mix.", h, positions, eps)
        elif L["type"] == "mlstm":
            x = x + matrix_memory_mixer(L["mixer"], W, p + "mix.", h, eps)
        else:
            raise KeyError(L["type"])
        if L.get("mlp"):
            x = x + experts(L["mlp"], W, p + "mlp.", rnd(rms_norm(x, W[p + "norm2"], eps)))
        after.append(x)
    logits = rnd(rms_norm(x, W["final.norm"], eps)) @ W["head"].to(F).T
    return logits, torch.stack(after)
