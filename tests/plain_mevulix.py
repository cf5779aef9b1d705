"""A plain, slow implementation of the Mevulix design in float64, one function per mechanism.

It shares no code with the engine: whole sequences at once, no cache, no pages, dense score matrices.
``forward`` takes the dict of config.json, a dict name -> tensor and the token ids of one sequence, and
returns the logits of every position and the residual stream after every layer.

Notation: T tokens, d width, H query heads, G key-value heads, R latent size, E experts.
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

def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w.to(F) + b.to(F)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# ---------------------------------------------------------------- positions

def yarn_frequencies(dims, base, scaling):
    """[dims/2] angles per position and the factor on cos and sin."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn(t):      # the (fractional) pair index whose wave makes t turns over the original length
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, rot):
    """x [T, ..., n]: entries (2i, 2i+1) of the first rot.dims are turned by pos * f_i; the rest pass."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    ang = pos.to(F)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mag).view(shape), (torch.sin(ang) * mag).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def distance_bucket(n, rows, far):
    """Row of the bias table for distance n >= 0: one row per distance below rows/2, then logarithmic steps up to ``far``."""
    near = rows // 2
    if n < near:
        return n
    return min(rows - 1, near + math.floor(math.log(n / near) / math.log(far / near) * (rows - near)))


# ---------------------------------------------------------------- mixers

def softmax_with_sink(scores, visible, sink=None):
    """scores [H, T, T]; ``sink`` [H]: one more term exp(sink_h) in every denominator, with no value."""
    s = scores.masked_fill(~visible, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(F)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(F)[:, None, None] - m)
    return e / den


def attention_keys_values(h, W, p, m, eps):
    """What a layer's cache holds: keys after the norm [T, G, dk] and values [T, G, dv]."""
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = lin(h, W[p + "k"], W[p + "k.b"])
    v = lin(h, W[p + "v"], W[p + "v.b"])
    k = rnd(rms_norm(k, W[p + "k.norm"], eps))
    return k.view(-1, G, dk), v.view(-1, G, dv)


def attention(h, W, p, m, eps, kv):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = lin(h, W[p + "q"], W[p + "q.b"])
    q = rms_norm(q, W[p + "q.norm"], eps)
    qt = m.get("q_temp")
    if qt:
        q = q * (1.0 + float(qt["coef"]) * torch.log(torch.floor((pos.to(F) + 1.0) / float(qt["every"])) + 1.0))[:, None]
    q = rnd(q).view(T, H, dk)
    k, v = kv
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    if m.get("bias_max") is not None:
        rel = W[p + "rel"].to(F)
        rows = rel.shape[0]
        by_distance = [distance_bucket(n, rows, float(m["bias_max"])) for n in range(T)]
        bucket = torch.tensor([[by_distance[i - j] if j <= i else 0 for j in range(T)] for i in range(T)])
        s = s + rel[bucket].permute(2, 0, 1)
    visible = (pos[None, :] <= pos[:, None])[None]
    w = softmax_with_sink(s, visible, W[p + "sink"])
    y = rnd(torch.einsum("hij,jhd->ihd", w, v)).reshape(T, H * dv)
    return lin(y, W[p + "o"])


def latent_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, dq, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rnd(rms_norm(lin(h, W[p + "dq"]), W[p + "dq.norm"], eps))
    q = lin(cq, W[p + "uq"]).view(T, H, dq + dr)
    low = lin(h, W[p + "dkv"])
    c = rnd(rms_norm(low[:, :R], W[p + "dkv.norm"], eps))
    shared = low[:, R:]
    q_plain, q_rot = q[..., :dq], q[..., dq:]
    if dr:
        q_rot = rnd(rotate_pairs(q_rot, pos, m["rot"]))
        shared = rnd(rotate_pairs(shared, pos, m["rot"]))
    k_plain = lin(c, W[p + "uk"]).view(T, H, dq)
    v = lin(c, W[p + "uv"]).view(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q_plain, k_plain)
    if dr:
        s = s + torch.einsum("ihd,jd->hij", q_rot, shared)
    s = s * float(m["scale"])
    visible = (pos[None, :] <= pos[:, None])[None]
    w = softmax_with_sink(s, visible)
    y = rnd(torch.einsum("hij,jhd->ihd", w, v)).reshape(T, H * dv)
    return lin(y, W[p + "o"])


# ---------------------------------------------------------------- feed-forwards

def gated(h, W, p, act):
    return lin(rnd(act(lin(h, W[p + "gate"])) * lin(h, W[p + "up"])), W[p + "down"])


MARGINS = None      # a list: every call of ``experts`` appends its tokens' margins [T] here and their choices [T, top] to CHOICES
CHOICES = []


def experts(h, W, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ W[p + "router"].to(F).T
    score = torch.sigmoid(z)
    ranked = torch.sort(z, dim=-1, descending=True, stable=True)      # the order of z is the order of sigmoid(z)
    chosen = ranked.indices[:, :top]
    if MARGINS is not None:      # how far the last chosen expert is ahead of the first one left out, and the choice as a set
        MARGINS.append(ranked.values[:, top - 1] - ranked.values[:, top] if top < E else torch.full_like(z[:, 0], 9.0))
        CHOICES.append(torch.sort(chosen, dim=-1).values)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += gated(rnd(score[t, e] * h[t])[None], W, f"{p}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + gated(h, W, p + "shared.", silu)
    return out


def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return gated(h, W, p, gelu_tanh)
    return experts(h, W, p, mlp)


# ---------------------------------------------------------------- the model

def forward(cfg: dict, W: dict, tokens):
    """(logits [T, vocab], stream after every layer [layers, T, d]), both float64."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    after = []
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = rnd(x)
        if L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(h, W, p + "mix.", m, eps)
                src = i
            y = attention(h, W, p + "mix.", m, eps, kept[src])
        elif L["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, W[p + "norm1"], W[p + "norm1.b"], eps) * W[p + "ls1"].to(F)
        if L.get("mlp"):
            f = feed_forward(rnd(x), W, p + "mlp.", L["mlp"])
            x = x + layer_norm(f, W[p + "norm2"], W[p + "norm2.b"], eps) * W[p + "ls2"].to(F)
        after.append(x.clone())
    h = rnd(layer_norm(x, W["final.norm"], W["final.norm.b"], eps))
    logits = (h @ W["head"].to(F).T) * float(cfg.get("logit_scale", 1.0))
    return logits, torch.stack(after)
