"""Small Mufalix configurations and weights for the tests.  Tensor names and shapes are written out here from the
configuration, independently of the engine's own list, so a name or shape the engine gets wrong shows as a loading
error."""
from __future__ import annotations

import math

import torch

from roletar_helpers import write_folder  # noqa: F401  (the folder writer knows no design)


def left(heads, kv_heads, dim, vdim, scale, window=None, rot_dims=None, base=10000.0, scaling=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if window:
        m["mask"] = dict(size=window)
    if rot_dims:
        m["rot"] = dict(base=base, dims=rot_dims)
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def parallel(left_cfg, width, conv, blocks):
    return dict(type="parallel", mixer=dict(left=left_cfg, right=dict(width=width, conv=conv, blocks=blocks)))


def mlstm(heads, dim, vdim, cap):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def moe(layer, experts, top, ff, scale=None):
    router = dict(experts=experts, top=top)
    if scale is not None:
        router["scale"] = scale
    return dict(layer, mlp=dict(kind="moe", router=router, expert=dict(ff=ff)))


def bare(layer):
    return dict(layer, mlp=None)


def config(which: str) -> dict:
    base = dict(architecture="Mufalix", norm=dict(eps=1e-5))
    if which == "mix":      # both mixers, layers with and without experts, a loop in the middle, a window that cuts pages
        return dict(base, vocab=300, width=96, embedding=dict(scale=3.0), loop=dict(start=1, stop=3, times=2), layers=[
            moe(mlstm(3, 16, 24, 15.0), 6, 2, 40, 1.5),
            moe(parallel(left(4, 2, 24, 16, 0.2, window=37, rot_dims=16, base=1000.0, scaling=(8.0, 1.0, 4.0, 64)), 64, 4, 2), 5, 3, 24, 2.5),
            bare(mlstm(2, 24, 16, 9.0)),
            bare(parallel(left(2, 2, 16, 24, 0.3, rot_dims=16), 48, 2, 4))])
    if which == "odd":      # no size a multiple of 4; the loop starts at layer 0 and runs three times; every expert is chosen
        return dict(base, vocab=61, width=50, norm=dict(eps=1e-6), embedding=dict(scale=1.7), loop=dict(start=0, stop=2, times=3), layers=[
            moe(parallel(left(3, 1, 10, 6, 0.35, window=5, rot_dims=6, base=300.0, scaling=(3.0, 0.5, 2.0, 40)), 30, 3, 3), 5, 5, 9, 0.7),
            moe(mlstm(3, 6, 10, 7.5), 3, 2, 11),
            bare(parallel(left(2, 2, 6, 10, 0.5, window=11, rot_dims=2, base=50.0), 18, 5, 1))])
    if which == "one":      # what other models make larger is 1 or absent here: one head, one expert chosen, one pass, a window of
        return dict(base, vocab=128, width=48, loop=dict(start=1, stop=2, times=1), layers=[    # one token, one tap, no rotation
            moe(parallel(left(1, 1, 8, 8, 0.6, window=1), 16, 1, 1), 3, 1, 16),
            bare(mlstm(1, 8, 8, 3.0)),
            moe(parallel(left(4, 4, 12, 4, 0.25, rot_dims=8), 8, 2, 8), 1, 1, 20, 1.0)])
    if which == "sharp":    # a large scale: single keys carry most of the weight; tiny pages; windows that end inside pages
        return dict(base, vocab=97, width=64, embedding=dict(scale=2.0), layers=[
            bare(parallel(left(4, 2, 16, 16, 1.5, window=50, rot_dims=8, base=100.0), 32, 4, 2)),
            bare(parallel(left(2, 1, 32, 8, 1.0, window=9, rot_dims=32, base=20000.0, scaling=(4.0, 1.0, 4.0, 32)), 64, 3, 4))])
    if which == "wide":     # sizes that the tensor-core kernels take (multiples of 64); long portions go to the library's batched
        return dict(base, vocab=200, width=128, embedding=dict(scale=2.0), loop=dict(start=0, stop=2, times=2), layers=[   # product
            moe(parallel(left(4, 2, 64, 32, 0.15, window=70, rot_dims=32, base=5000.0, scaling=(2.0, 1.0, 2.0, 128)), 128, 4, 2), 4, 2, 64, 2.0),
            moe(mlstm(2, 64, 64, 10.0), 3, 1, 128)])
    if which == "larger":   # heads, experts and widths that the tcgen05 products, the warp-MMA attention and the chunked kernels take in long
        return dict(base, vocab=1000, width=512, embedding=dict(scale=4.0), loop=dict(start=0, stop=2, times=2), layers=[   # portions
            moe(mlstm(4, 64, 128, 12.0), 8, 2, 256, 2.0),
            moe(parallel(left(8, 2, 64, 64, 0.125, window=300, rot_dims=32, base=100000.0, scaling=(4.0, 1.0, 4.0, 256)), 512, 4, 4), 8, 2, 256, 1.5)])
    if which == "only_memory":
        return dict(base, vocab=97, width=40, layers=[bare(mlstm(2, 16, 8, 4.0))])
    if which == "only_pair":
        return dict(base, vocab=97, width=40, layers=[bare(parallel(left(4, 2, 16, 8, 0.4, window=20, rot_dims=12, base=500.0), 24, 4, 3))])
    if which == "only_experts":   # the mixer is tiny, the experts dominate
        return dict(base, vocab=97, width=40, layers=[moe(mlstm(1, 4, 4, 5.0), 7, 3, 24, 3.0), moe(mlstm(1, 4, 4, 5.0), 4, 2, 12)])
    if which == "only_loop":      # the projection at the start of a pass dominates: one small layer run four times
        return dict(base, vocab=97, width=40, embedding=dict(scale=0.5), loop=dict(start=0, stop=1, times=4), layers=[bare(mlstm(1, 8, 8, 6.0))])
    raise KeyError(which)


PAGE_SIZE = {"larger": 16, "wide": 16, "mix": 16, "odd": 2, "one": 4, "sharp": 4, "only_memory": 16, "only_pair": 8, "only_experts": 16, "only_loop": 8}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> float32 tensor whose values are all representable in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def uni(shape, a, b):
        return a + (b - a) * torch.rand(shape, generator=g)

    W = {"embed": torch.randn(cfg["vocab"], d, generator=g), "head": mat(cfg["vocab"], d, 2.0), "final.norm": uni((d,), 0.8, 1.2)}
    if cfg.get("loop"):
        W["loop.in"] = torch.cat([torch.eye(d) * 0.6, torch.eye(d) * 0.4], dim=1) + mat(d, 2 * d, 0.5)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = uni((d,), 0.8, 1.2)
        if L["type"] == "mlstm":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            q = p + "mix."
            W[q + "q"], W[q + "k"] = mat(H * dk, d, 1.5), mat(H * dk, d, 1.5)
            W[q + "v"], W[q + "g"] = mat(H * dv, d, 1.5), mat(H * dv, d, 2.0)
            W[q + "i"], W[q + "f"] = mat(H, d, 3.0), mat(H, d, 3.0)
            W[q + "i.b"], W[q + "f.b"] = uni((H,), -2.0, 1.0), uni((H,), 0.5, 5.0)
            W[q + "norm"], W[q + "o"] = uni((H * dv,), 0.8, 1.2), mat(d, H * dv)
        else:
            a, r = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            W[q + "q"], W[q + "k"], W[q + "v"] = mat(H * dk, d, 2.0), mat(G * dk, d, 2.0), mat(G * dv, d, 1.5)
            W[q + "q.b"], W[q + "k.b"], W[q + "v.b"] = uni((H * dk,), -0.3, 0.3), uni((G * dk,), -0.3, 0.3), uni((G * dv,), -0.3, 0.3)
            W[q + "q.norm"], W[q + "k.norm"] = uni((dk,), 0.7, 1.4), uni((dk,), 0.7, 1.4)
            W[q + "sink"] = uni((H,), -1.0, 2.0)
            W[q + "g"], W[q + "o"], W[q + "o.b"] = mat(H * dv, d, 2.0), mat(d, H * dv), uni((d,), -0.3, 0.3)
            C, taps, nb = r["width"], r["conv"], r["blocks"]
            sz = C // nb
            q = p + "mix.right."
            W[q + "y"], W[q + "x"] = mat(C, d, 1.5), mat(C, d, 1.5)
            W[q + "y.b"], W[q + "x.b"] = uni((C,), -0.3, 0.3), uni((C,), -0.3, 0.3)
            W[q + "conv"], W[q + "conv.b"] = uni((C, taps), -0.6, 0.6), uni((C,), -0.2, 0.2)
            W[q + "ra"], W[q + "ri"] = torch.randn(nb, sz, sz, generator=g) * (2.0 / math.sqrt(sz)), torch.randn(nb, sz, sz, generator=g) * (2.0 / math.sqrt(sz))
            W[q + "ra.b"], W[q + "ri.b"] = uni((nb, sz), -1.0, 1.0), uni((nb, sz), -1.0, 1.0)
            W[q + "lam"], W[q + "o"] = uni((C,), -5.0, 1.0), mat(d, C)
            W[p + "mix.left.out"], W[p + "mix.right.out"] = uni((d,), 0.6, 1.4), uni((d,), 0.6, 1.4)
        mlp = L.get("mlp")
        if not mlp:
            continue
        W[p + "norm2"] = uni((d,), 0.8, 1.2)
        E = mlp["router"]["experts"]
        W[p + "mlp.router"] = mat(E, d, 3.0)
        W[p + "mlp.correction"] = uni((E,), -0.4, 0.4)
        for e in range(E):
            W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(mlp["expert"]["ff"], d, 2.0), mat(d, mlp["expert"]["ff"])
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}
