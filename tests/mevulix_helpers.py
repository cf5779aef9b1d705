"""Small Mevulix configurations and weights for the tests.  Tensor names and shapes are written out here from the
configuration, independently of the engine's own list, so a name or shape the engine gets wrong shows as a loading
error."""
from __future__ import annotations

import math

import torch

from roletar_helpers import write_folder  # noqa: F401  (the folder writer knows no design)


def attention(heads, kv_heads, dim, vdim, scale, rows=None, far=None, softcap=None, temp=None, kv_from=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if rows is not None:
        m["bias_max"] = far
        m["_rows"] = rows        # the rows of the bias table: not in config.json (the tensor's shape says it); taken out by ``config``
    if softcap is not None:
        m["softcap"] = softcap
    if temp is not None:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, dims=None, scaling=None):
    rot = dict(base=base, dims=dims or rot_dim)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
                                                    scale=scale, rot=rot))


def dense(layer, ff):
    return dict(layer, mlp=dict(kind="dense", ff=ff))


def moe(layer, experts, top, ff, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        mlp["shared"] = dict(ff=shared)
    return dict(layer, mlp=mlp)


def bare(layer):
    return dict(layer, mlp=None)


def _named(which: str) -> dict:
    base = dict(architecture="Mevulix", norm=dict(eps=1e-5))
    if which == "mix":      # both mixers, every feed-forward, a layer that reads another's keys and values, a layer without feed-forward
        return dict(base, vocab=300, width=96, logit_scale=0.7, layers=[
            dense(latent(3, 16, 8, 24, 40, 24, 0.2, base=1000.0, scaling=(4.0, 64, 8.0, 1.0)), 128),
            moe(attention(4, 2, 24, 16, 0.2, rows=12, far=40, softcap=8.0, temp=(0.5, 16)), 6, 2, 40, shared=24),
            moe(latent(2, 24, 16, 16, 24, 40, 0.15, base=50.0), 5, 3, 24),
            dense(attention(4, 2, 24, 16, 0.3, rows=8, far=21, softcap=30.0, temp=(0.2, 7), kv_from=1), 80),
            bare(attention(2, 1, 16, 32, 0.25, rows=20, far=100))])
    if which == "odd":      # no size a multiple of 4; a table with an odd count of rows; every expert is chosen; pages of two tokens
        return dict(base, vocab=61, width=50, norm=dict(eps=1e-6), logit_scale=1.3, layers=[
            moe(attention(3, 1, 10, 6, 0.35, rows=7, far=9.5, softcap=3.0, temp=(0.9, 5)), 5, 5, 9, shared=7),
            dense(latent(3, 6, 6, 10, 14, 10, 0.3, base=300.0, dims=6, scaling=(3.0, 40, 2.0, 0.5)), 34),
            moe(attention(3, 1, 10, 6, 0.5, rows=5, far=30, kv_from=0), 3, 2, 11)])
    if which == "one":      # what other models make larger is 1 or absent here: one head, one expert, a step every token, two rows,
        return dict(base, vocab=128, width=48, layers=[     # no cap, no temperature, no scaling, no logit scale
            moe(attention(1, 1, 8, 8, 0.6, rows=2, far=2, temp=(0.3, 1)), 1, 1, 20, shared=8),
            bare(latent(1, 8, 2, 8, 12, 6, 0.4, base=10.0)),
            dense(attention(4, 4, 12, 4, 0.25, rows=4, far=3), 16)])
    if which == "sharp":    # a large scale: single keys carry most of the weight; tiny pages
        return dict(base, vocab=97, width=64, logit_scale=0.5, layers=[
            bare(attention(4, 2, 16, 16, 1.2, rows=16, far=60, softcap=25.0, temp=(0.4, 32))),
            bare(latent(2, 16, 8, 16, 24, 16, 1.0, base=100.0, scaling=(8.0, 32, 4.0, 1.0))),
            dense(attention(2, 2, 32, 8, 1.0, rows=6, far=200), 48)])
    if which == "wide":     # sizes that the tensor-core kernels take (multiples of 16 and 64)
        return dict(base, vocab=200, width=128, logit_scale=0.8, layers=[
            moe(latent(4, 32, 32, 32, 64, 48, 0.12, base=5000.0, scaling=(2.0, 128, 16.0, 2.0)), 4, 2, 64, shared=64),
            dense(attention(4, 2, 64, 32, 0.15, rows=32, far=150, softcap=20.0, temp=(0.3, 50)), 256),
            moe(attention(8, 2, 64, 32, 0.1, rows=16, far=64, kv_from=1), 3, 1, 128)])
    if which == "larger":   # widths, heads and experts that the tcgen05 products and the warp-MMA attention take in long portions
        return dict(base, vocab=1000, width=512, logit_scale=0.6, layers=[
            moe(latent(8, 64, 32, 64, 128, 192, 0.1, base=100000.0, scaling=(4.0, 256, 16.0, 1.0)), 8, 2, 256, shared=256),
            moe(attention(8, 2, 64, 64, 0.125, rows=32, far=300, softcap=40.0, temp=(0.25, 100)), 8, 2, 256),
            dense(attention(8, 2, 64, 64, 0.125, rows=24, far=90, kv_from=1), 1024)])
    if which == "only_attention":
        return dict(base, vocab=97, width=40, layers=[bare(attention(4, 2, 16, 8, 0.4, rows=10, far=25, softcap=6.0, temp=(0.6, 9)))])
    if which == "only_latent":
        return dict(base, vocab=97, width=40, layers=[bare(latent(2, 16, 8, 12, 20, 12, 0.3, base=100.0, scaling=(6.0, 24, 3.0, 0.8)))])
    if which == "only_dense":     # the mixer is tiny, the feed-forward dominates
        return dict(base, vocab=97, width=40, layers=[dense(attention(1, 1, 4, 4, 0.5, rows=2, far=2), 56), dense(attention(1, 1, 4, 4, 0.5, rows=2, far=2), 24)])
    if which == "only_experts":
        return dict(base, vocab=97, width=40, layers=[moe(attention(1, 1, 4, 4, 0.5, rows=2, far=2), 7, 3, 24, shared=12),
                                                      moe(attention(1, 1, 4, 4, 0.5, rows=2, far=2), 4, 2, 12)])
    if which == "only_shared_kv":     # three layers read the first one's keys and values
        return dict(base, vocab=97, width=40, layers=[bare(attention(2, 1, 8, 8, 0.4, rows=6, far=12))] +
                    [bare(attention(2 * k, 1, 8, 8, 0.4, rows=4 + k, far=10 * k, temp=(0.2 * k, 3), kv_from=0)) for k in (1, 2, 3)])
    raise KeyError(which)


def bias_rows(cfg_with_rows: dict) -> dict:
    """layer -> rows of its bias table, from a configuration as ``_named`` makes it."""
    return {i: L["mixer"]["_rows"] for i, L in enumerate(cfg_with_rows["layers"]) if "_rows" in L["mixer"]}


def strip(cfg_with_rows: dict) -> dict:
    """config.json as a model folder holds it: the bias tables' rows are left to the tensors' shapes."""
    return dict(cfg_with_rows, layers=[dict(L, mixer={k: v for k, v in L["mixer"].items() if k != "_rows"}) for L in cfg_with_rows["layers"]])


def config(which: str) -> dict:
    return strip(_named(which))


PAGE_SIZE = {"larger": 16, "wide": 16, "mix": 16, "odd": 2, "one": 4, "sharp": 4, "only_attention": 8, "only_latent": 8, "only_dense": 16,
             "only_experts": 16, "only_shared_kv": 4}


def make_weights(cfg: dict, seed: int, rows: dict) -> dict:
    """name -> float32 tensor whose values are all representable in bfloat16.  ``rows``: layer -> rows of its bias table."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def uni(shape, a, b):
        return a + (b - a) * torch.rand(shape, generator=g)

    def gated(p, ff):
        W[p + "gate"], W[p + "up"], W[p + "down"] = mat(ff, d, 1.5), mat(ff, d, 1.5), mat(d, ff)

    W = {"embed": torch.randn(cfg["vocab"], d, generator=g), "head": mat(cfg["vocab"], d, 2.0), "final.norm": uni((d,), 0.8, 1.2),
         "final.norm.b": uni((d,), -0.2, 0.2)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"], W[p + "norm1.b"], W[p + "ls1"] = uni((d,), 0.8, 1.2), uni((d,), -0.2, 0.2), uni((d,), 0.3, 1.0)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[q + "q"], W[q + "q.b"], W[q + "q.norm"] = mat(H * dk, d, 2.0), uni((H * dk,), -0.3, 0.3), uni((H * dk,), 0.7, 1.4)
            if m.get("kv_from") is None:
                W[q + "k"], W[q + "k.b"], W[q + "k.norm"] = mat(G * dk, d, 2.0), uni((G * dk,), -0.3, 0.3), uni((G * dk,), 0.7, 1.4)
                W[q + "v"], W[q + "v.b"] = mat(G * dv, d, 1.5), uni((G * dv,), -0.3, 0.3)
            if i in rows:
                W[q + "rel"] = uni((rows[i], H), -2.0, 2.0)
            W[q + "sink"], W[q + "o"] = uni((H,), -1.0, 2.0), mat(d, H * dv)
        else:
            H, dk, dr, dv, R, Rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            W[q + "dq"], W[q + "dq.norm"], W[q + "uq"] = mat(Rq, d, 2.0), uni((Rq,), 0.8, 1.2), mat(H * (dk + dr), Rq, 2.0)
            W[q + "dkv"], W[q + "dkv.norm"] = mat(R + dr, d, 2.0), uni((R,), 0.8, 1.2)
            W[q + "uk"], W[q + "uv"], W[q + "o"] = mat(H * dk, R, 2.0), mat(H * dv, R), mat(d, H * dv)
        mlp = L.get("mlp")
        if not mlp:
            continue
        W[p + "norm2"], W[p + "norm2.b"], W[p + "ls2"] = uni((d,), 0.8, 1.2), uni((d,), -0.2, 0.2), uni((d,), 0.3, 1.0)
        if mlp["kind"] == "dense":
            gated(p + "mlp.", mlp["ff"])
            continue
        E = mlp["router"]["experts"]
        W[p + "mlp.router"] = mat(E, d, 3.0)
        for e in range(E):
            gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
        if mlp.get("shared"):
            gated(p + "mlp.shared.", mlp["shared"]["ff"])
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}


def build(which: str, seed: int):
    """(config.json's dict, weights) of a named test model."""
    full = _named(which)
    return strip(full), make_weights(full, seed, bias_rows(full))
