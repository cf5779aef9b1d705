"""The Mevulix design in the engine against the plain float64 implementation, on the GPU, in 32 bit and in bfloat16:
each mechanism alone (one-mechanism models, single kernels, and the stream after every layer), each request whole,
prefill against token-by-token decoding, portions down to two tokens, mixed batches with pages and slots that are used
again, keys far away, at page borders and at the edges of the distance buckets, long decoding, and greedy generation
through ``LMBackend``, the command line and the replay command."""
import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
import mevulix_helpers as mh
import plain_mevulix as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# 32 bit: the largest difference of a logit (or a stream entry) as a fraction of the largest value of its request's
# reference.  bfloat16: the root mean square of a position's differences as a fraction of that of the request's
# reference logits, and at most three times what rounding alone causes.
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
LENGTHS = {"wide": [250, 5, 199, 64], "mix": [3, 37, 60, 121], "odd": [1, 7, 26, 45], "one": [2, 25, 33, 58], "sharp": [1, 40, 97, 150],
           "only_attention": [1, 9, 40, 75], "only_latent": [2, 30, 47], "only_dense": [1, 6, 21], "only_experts": [1, 6, 21, 50],
           "only_shared_kv": [1, 2, 19, 44]}
_cache = {}


def model(tmp_path_factory, which):
    if which not in _cache:
        cfg, W = mh.build(which, 31 + len(which))
        folder = mh.write_folder(tmp_path_factory.mktemp("mevulix"), which, cfg, W)
        _cache[which] = (cfg, W, folder)
    return _cache[which]


def make_runner(folder, which, dtype, num_pages=None, max_batch=4, max_seq_len=256, **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    ps = mh.PAGE_SIZE[which] if isinstance(which, str) else int(which)
    cfg = EngineConfig(max_batch=max_batch, max_seq_len=max_seq_len, page_size=ps, dtype=dtype,
                       num_pages=num_pages if num_pages is not None else max_batch * (max_seq_len // ps), **kw)
    return ModelRunner(folder, engine_config=cfg)


CLOSE_CALL = 0.05      # a router's choice decided by less than this (in logits) may fall either way once the input is rounded to bfloat16


class Noise(list):
    """Per request and position the error that bfloat16 rounding alone causes: the plain implementation with rounding against
    itself without, and at least twice the median of that over the positions.  ``margins``: per request and position the smallest
    margin by which any router decided; ``compare`` leaves a position with a close call out (attention carries nothing of one
    position's feed-forward to another position of the same layer, but later layers do: the rest of that request is left out too)."""
    margins = None


def routed(cfg, W, t):
    plain.MARGINS, plain.CHOICES = [], []
    logits = plain.forward(cfg, W, t)[0]
    m = plain.MARGINS
    plain.MARGINS, plain.CHOICES = None, []
    return logits, (torch.stack(m).min(dim=0).values if m else torch.full((len(t),), 9.0))


def rounding_noise(cfg, W, toks, refs):
    out = Noise()
    out.margins = []
    for t, ref in zip(toks, refs):
        _, margins = routed(cfg, W, t)
        with plain.rounding("bfloat16"):
            em, _ = routed(cfg, W, t)
        out.margins.append(margins)
        err = (em - ref).pow(2).mean(dim=1).sqrt()
        calm = err[margins >= CLOSE_CALL]
        out.append(torch.clamp(err, min=2.0 * (calm.median().item() if calm.numel() else err.median().item())))
    return out


def compare(results, refs, lengths, dtype, what, noise=None):
    worst = 0.0
    for i, n in enumerate(lengths):
        got = helpers.stack_positions(results, i, n).double()
        if dtype == "float32":
            err = (got - refs[i]).abs().max(dim=1).values
            scale = refs[i].abs().max().item()
        else:
            err = (got - refs[i]).pow(2).mean(dim=1).sqrt()
            scale = refs[i].pow(2).mean().sqrt().item()
        allowed = torch.full_like(err, TOL[dtype] * scale)
        if noise is not None:
            allowed = torch.maximum(allowed, 3.0 * noise[i % len(noise)])
        bad = (err > allowed).nonzero()[:, 0].tolist()
        if noise is not None:
            # bfloat16: a close call of a router ends the comparison of the request; otherwise one position in fifty may be over
            # the bound (an estimate from one rounded run), by less than three times.
            outliers = []
            for p in bad:
                if noise.margins[i % len(noise)][:p + 1].min() < CLOSE_CALL:
                    err, bad = err[:p], [q for q in bad if q < p]
                    break
                if err[p] <= 3.0 * allowed[p]:
                    outliers.append(p)
            if len(outliers) <= max(1, len(err) // 50):
                bad = [q for q in bad if q not in outliers]
            if not err.numel():
                continue
        if bad:
            p = bad[0]
            raise AssertionError(f"{what}: request {i} first differs at position {p} (of {n}): error {err[p].item():.3e}, "
                                 f"allowed {allowed[p].item():.3e}")
        worst = max(worst, err.max().item() / scale)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(LENGTHS))
def test_every_way_of_cutting(tmp_path_factory, which, dtype):
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = LENGTHS[which]
    toks = [helpers.random_tokens(n, cfg["vocab"], 200 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    ps = mh.PAGE_SIZE[which]
    runner = make_runner(folder, which, dtype)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    worst = {}
    worst["whole"] = compare(helpers.run_schedule(runner, toks, helpers.whole(lengths)), refs, lengths, dtype, "whole", noise)
    worst["one by one"] = compare(helpers.run_schedule(runner, toks, helpers.last_one_by_one(lengths)), refs, lengths, dtype,
                                  "last 32 one by one", noise)
    for seed, sizes in ((1, (7, 2, 13, 2, 5, 3, 16, 2, 9)), (2, (2, 2, 3, 31, 2, 17, 33, 40))):
        res = helpers.run_schedule(runner, toks, helpers.changing_portions(lengths, seed=seed, sizes=sizes))
        worst[f"portions {seed}"] = compare(res, refs, lengths, dtype, "changing portions", noise)
    # mixed: more requests than slots, and a pool so small that pages of finished requests are used again
    prompt_lens = [max(1, n // 2) for n in lengths]
    steps, ends = helpers.mixed(lengths * 3, prompt_lens * 3, seed=3, max_live=3)
    tight = make_runner(folder, which, dtype, num_pages=helpers.peak_pages(steps, ends, ps), max_batch=3)
    res = helpers.run_schedule(tight, toks * 3, steps, ends)
    worst["mixed"] = compare(res, refs * 3, lengths * 3, dtype, "mixed with pages and slots used again", noise)
    print(f"\nworst logit error {which} {dtype}: " + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_larger_sizes(tmp_path_factory, dtype):
    """Width 512, 8 experts, heads of 64: a 700-token prompt whole (about 175 rows an expert: the tcgen05 products; the warp-MMA
    attention; the library's batched product for the latent's heads), in portions of 256 beside a second request, and its last
    tokens one by one."""
    cfg, W, folder = model(tmp_path_factory, "larger")
    lengths = [700, 130]
    toks = [helpers.random_tokens(n, cfg["vocab"], 900 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    runner = make_runner(folder, "larger", dtype, max_batch=2, max_seq_len=704, max_tokens_per_step=1024)
    compare(helpers.run_schedule(runner, toks, helpers.whole(lengths)), refs, lengths, dtype, "whole", noise)
    steps = [[(0, 0, 256), (1, 0, 100)], [(0, 256, 256), (1, 100, 1)], [(0, 512, 180), (1, 101, 29)]] + [[(0, p, 1)] for p in range(692, 700)]
    compare(helpers.run_schedule(runner, toks, steps), refs, lengths, dtype, "portions of 256 beside a second request", noise)


@pytest.mark.parametrize("which", ["mix", "odd", "one", "only_attention", "only_latent", "only_dense", "only_experts", "only_shared_kv"])
def test_stream_after_every_layer(tmp_path_factory, which):
    """32 bit: the residual stream after every layer, for a prompt in one step and for the same prompt cut in two."""
    from delta_b200.engine.step import RowInput
    cfg, W, folder = model(tmp_path_factory, which)
    toks = helpers.random_tokens(29, cfg["vocab"], 5)
    _, after = plain.forward(cfg, W, toks)
    runner = make_runner(folder, which, "float32")
    for cut in (29, 11):
        slot = runner.cache.acquire_slot()
        got = []
        for a, b in ((0, cut), (cut, 29)):
            if a == b:
                continue
            runner.capture = {"layer_totals": []}
            runner.run_rows([RowInput(slot, toks[a:b], a, [])])
            got.append(torch.stack(runner.capture["layer_totals"]).cpu())
        runner.capture = None
        runner.cache.release_slot(slot)
        got = torch.cat(got, dim=1).double()
        assert got.shape == after.shape
        for r in range(after.shape[0]):
            err = (got[r] - after[r]).abs().max().item()
            assert err <= TOL["float32"] * after[r].abs().max().item(), f"{which}: layer {r} differs by {err:.3e} (cut at {cut})"


@pytest.mark.parametrize("which,dtype", [("mix", "float32"), ("odd", "float32"), ("mix", "bfloat16")])
def test_long_decoding(tmp_path_factory, which, dtype):
    """A short prompt, then 180 tokens one by one: pages fill one after the other, the query temperature steps up many times and
    the distances pass through every bucket of the bias tables."""
    cfg, W, folder = model(tmp_path_factory, which)
    n = 185
    toks = [helpers.random_tokens(n, cfg["vocab"], 9)]
    refs = [plain.forward(cfg, W, toks[0])[0]]
    runner = make_runner(folder, which, dtype, max_batch=1)
    steps = [[(0, 0, 5)]] + [[(0, p, 1)] for p in range(5, n)]
    res = helpers.run_schedule(runner, toks, steps)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    print("\nlong decoding worst", compare(res, refs, [n], dtype, "long decoding", noise))
    assert all(g.pool.held_pages == 0 for g in runner.cache.groups.values())


def test_a_slot_used_again_starts_clean(tmp_path_factory):
    """Request B after request A in the same slot and pages equals B alone: the cache of A is gone."""
    from delta_b200.engine.step import RowInput
    cfg, W, folder = model(tmp_path_factory, "mix")
    runner = make_runner(folder, "mix", "float32", max_batch=1, num_pages=8, max_seq_len=128)
    a, b = helpers.random_tokens(100, cfg["vocab"], 1), helpers.random_tokens(50, cfg["vocab"], 2)
    ref = plain.forward(cfg, W, b)[0]
    for toks in (a, b):
        slot = runner.cache.acquire_slot()
        assert slot == 0
        logits = runner.run_rows([RowInput(slot, toks, 0, list(range(len(toks))))])
        runner.cache.release_slot(slot)
    err = (logits.cpu().double() - ref).abs().max().item()
    assert err <= TOL["float32"] * ref.abs().max().item()


# ---- weights made so that one key or the bias table decides ------------------------------------------------------

def crafted_needle(seed=77):
    """One attention layer whose key projection is its query projection with the columns permuted (same bias, same norm), and
    token 1's embedding is token 0's under that permutation: a query of token 1 meets a key of token 0 with the largest score there
    is, and no other key comes close.  Token 0 stands once, far back; token 1 is the last token: what the last position gives is
    the value of the far one."""
    full = dict(architecture="Mevulix", norm=dict(eps=1e-5), vocab=800, width=64, logit_scale=0.9, layers=[
        mh.bare(mh.attention(2, 2, 16, 16, 0.6, rows=8, far=300, softcap=50.0))])
    W = mh.make_weights(full, seed, mh.bias_rows(full))
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(seed))
    W["l0.mix.k"] = W["l0.mix.q"][:, perm].clone()      # k(e) = W_q e' with e'[perm[j]] = e[j]
    for s in (".b", ".norm"):
        W["l0.mix.k" + s] = W["l0.mix.q" + s].clone()
    W["embed"][1, perm] = W["embed"][0]
    W["l0.mix.rel"] = W["l0.mix.rel"] * 0.1
    W["l0.mix.sink"] = W["l0.mix.sink"] * 0.0 - 2.0
    return mh.strip(full), W


def needle_prompt(vocab, n, a_at, seed):
    g = torch.Generator().manual_seed(seed)
    toks = (torch.randperm(vocab - 2, generator=g)[:n] + 2).tolist()
    toks[a_at], toks[-1] = 0, 1
    return toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("distance", [15, 16, 17, 33, 250, 561])
def test_a_far_key_carries_the_weight(tmp_path_factory, dtype, distance):
    """The crafted key is read ``distance`` tokens later (next door, on both sides of a page's border, hundreds of tokens back): in a
    whole prompt, with the reader decoded alone, with the reader opening a portion, and with the key ending one."""
    cfg, W = crafted_needle()
    n = distance + 30
    a_at = n - 1 - distance
    toks = needle_prompt(cfg["vocab"], n, a_at, distance)
    ref = plain.forward(cfg, W, toks)[0]
    without = list(toks)
    without[a_at] = [t for t in range(2, cfg["vocab"]) if t not in toks][0]
    assert (plain.forward(cfg, W, without)[0][-1] - ref[-1]).abs().max().item() > 0.2 * ref.abs().max().item(), "the crafted key does not carry the weight"
    folder = mh.write_folder(tmp_path_factory.mktemp("needle"), f"needle{distance}", cfg, W)
    runner = make_runner(folder, 16, dtype, max_batch=2, max_seq_len=640, max_tokens_per_step=640)
    noise = rounding_noise(cfg, W, [toks], [ref]) if dtype == "bfloat16" else None
    b_at = n - 1
    for what, steps in (("whole", [[(0, 0, n)]]), ("the reader decoded alone", [[(0, 0, b_at - 3)]] + [[(0, p, 1)] for p in range(b_at - 3, n)]),
                        ("the reader opens a portion", [[(0, 0, 2)], [(0, 2, b_at - 4)], [(0, b_at - 2, 2)], [(0, b_at, 1)]]),
                        ("the key ends a portion", [[(0, 0, a_at + 1)], [(0, a_at + 1, n - a_at - 1)]] if a_at > 0 else [[(0, 0, 1)], [(0, 1, n - 1)]])):
        compare(helpers.run_schedule(runner, [toks], steps), [ref], [n], dtype, what, noise)


def crafted_bias_only(rows, far, seed=5):
    """Two attention layers whose queries are zero (no query weights, no query bias): every score is the bias of its distance,
    so a distance that falls into the wrong bucket, at any edge, moves the softmax weights of all positions behind it.  The
    second layer reads the first one's keys and values with a table of another size."""
    full = dict(architecture="Mevulix", norm=dict(eps=1e-5), vocab=97, width=32, layers=[
        mh.bare(mh.attention(2, 1, 8, 8, 0.5, rows=rows, far=far)), mh.bare(mh.attention(2, 1, 8, 8, 0.5, rows=rows + 3, far=far * 1.5, kv_from=0))])
    W = mh.make_weights(full, seed, mh.bias_rows(full))
    for i in (0, 1):
        W[f"l{i}.mix.q"] *= 0.0
        W[f"l{i}.mix.q.b"] *= 0.0
        W[f"l{i}.mix.rel"] *= 2.5
    return mh.strip(full), W


@pytest.mark.parametrize("rows,far", [(10, 23), (7, 9.5), (2, 2), (16, 128)])
def test_the_distance_buckets_decide(tmp_path_factory, rows, far):
    """32 bit, prompts longer than the tables reach: whole, every token alone, and portions whose starts walk over the buckets' edges."""
    cfg, W = crafted_bias_only(rows, far)
    n = int(far * 1.5) + 20
    toks = helpers.random_tokens(n, cfg["vocab"], rows)
    ref = plain.forward(cfg, W, toks)[0]
    folder = mh.write_folder(tmp_path_factory.mktemp("bias"), f"bias{rows}", cfg, W)
    runner = make_runner(folder, 4, "float32", max_batch=1, max_seq_len=256)
    for what, steps in (("whole", [[(0, 0, n)]]), ("every token alone", [[(0, p, 1)] for p in range(n)]),
                        ("portions of three", [[(0, p, min(3, n - p))] for p in range(0, n, 3)]),
                        ("portions of seven behind one token", [[(0, 0, 1)]] + [[(0, p, min(7, n - p))] for p in range(1, n, 7)])):
        compare(helpers.run_schedule(runner, [toks], steps), [ref], [n], "float32", what)
    from delta_b200.parts.row_attention import distance_buckets
    table = distance_buckets(rows, far)
    assert table == [plain.distance_bucket(k, rows, far) for k in range(len(table))]
    assert all(plain.distance_bucket(k, rows, far) == table[-1] == rows - 1 for k in range(len(table) - 1, len(table) + 300))


# ---- single kernels against their equations ---------------------------------------------------------------------

DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [50, 256, 1030, 2048, 9000])
@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_sublayer_norm_add_kernel(dtype, d, kind):
    from delta_b200.kernels import ops
    g = torch.Generator().manual_seed(d)
    T = 13
    x, y = torch.randn(T, d, generator=g), (torch.randn(T, d, generator=g) * 3 + 0.7).to(dtype)
    w, b = torch.rand(d, generator=g) + 0.5, torch.randn(d, generator=g) * 0.3
    X = x.to(DEV).clone()
    out = torch.empty(T, d, dtype=dtype, device=DEV)
    ops.sublayer_norm_add(X, y.to(DEV), out, weight=w.to(DEV), bias=b.to(DEV), eps=1e-5, kind=kind)
    yy = y.double()
    if kind == "layer":
        yy = yy - yy.mean(-1, keepdim=True)
    want = x.double() + yy / torch.sqrt((yy * yy).mean(-1, keepdim=True) + 1e-5) * w.double() + b.double()
    assert (X.cpu().double() - want).abs().max().item() <= 2e-6 * want.abs().max().item()
    assert torch.equal(out.cpu(), X.cpu().to(dtype))
    X2 = x.to(DEV).clone()       # no bias, no rounded copy
    ops.sublayer_norm_add(X2, y.to(DEV), None, weight=w.to(DEV), eps=1e-5, kind=kind)
    assert (X2.cpu().double() - (want - b.double())).abs().max().item() <= 2e-6 * want.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(3, 1, 10, 6), (4, 2, 16, 8), (8, 8, 64, 64), (2, 0, 24, 8)])
def test_append_with_a_norm_over_all_heads_and_a_query_temperature(dtype, sizes):
    """``rows_append_unit``: biases, one RMS norm over all of q's columns and one over all of k's, the query temperature by position;
    keys and values land in their pages; without keys (KV 0) only the queries are made."""
    from delta_b200.kernels import ops
    H, KV, dk, dv = sizes
    g = torch.Generator().manual_seed(H * 10 + dk)
    T, ps, pages = 9, 4, 6
    n = (H + KV) * dk + KV * dv
    src = (torch.randn(T, n + 3, generator=g) * 2).to(dtype)
    bias = torch.randn(n, generator=g) * 0.5
    qw, kw = torch.rand(H * dk, generator=g) + 0.5, torch.rand(max(KV, 1) * dk, generator=g) + 0.5
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 30, 31, 62], dtype=torch.int32)
    row = torch.zeros(T, dtype=torch.int32)
    table = torch.tensor([[3, 1, 4, 0, 5, 2, 0, 1, 3, 4, 5, 2, 1, 0, 3, 4]], dtype=torch.int32)      # logical page -> page
    cache = torch.zeros(pages, max(KV, 1), ps, dk + dv, dtype=dtype) if KV else None
    s_dev = src.to(DEV).clone()
    c_dev = cache.to(DEV) if KV else None
    coef, every = 0.7, 3
    ops.rows_append_unit(s_dev, pos.to(DEV), row.to(DEV), table.to(DEV), c_dev, H=H, KV=KV, dk=dk, dv=dv, ps=ps, row_width=dk + dv, k_off=0,
                         v_off=dk, bias=bias.to(DEV), q_norm=qw.to(DEV), k_norm=kw.to(DEV) if KV else None, pre_eps=1e-5, norm_whole=True,
                         q_temp=(coef, every))
    x = src[:, :n].double() + bias.double()
    q = x[:, :H * dk]
    q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + 1e-5) * qw.double()
    q = q * (1.0 + coef * torch.log(torch.floor((pos.double() + 1) / every) + 1.0))[:, None]
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert (s_dev[:, :H * dk].cpu().double() - q).abs().max().item() <= tol * q.abs().max().item()
    if not KV:
        return
    k = x[:, H * dk:(H + KV) * dk]
    k = (k / torch.sqrt((k * k).mean(-1, keepdim=True) + 1e-5) * kw.double()).view(T, KV, dk)
    v = x[:, (H + KV) * dk:].view(T, KV, dv)
    got = c_dev.cpu().double()
    for t in range(T):
        page, off = int(table[0, int(pos[t]) // ps]), int(pos[t]) % ps
        assert (got[page, :, off, :dk] - k[t]).abs().max().item() <= tol * k.abs().max().item()
        assert (got[page, :, off, dk:] - v[t]).abs().max().item() <= tol * v.abs().max().item()


@pytest.mark.parametrize("case", [("float32", 4, 2, 16, 8, None), ("float32", 3, 1, 10, 6, None), ("bfloat16", 4, 2, 16, 16, False),
                                  ("bfloat16", 8, 2, 64, 32, False), ("bfloat16", 8, 2, 64, 32, True), ("bfloat16", 16, 1, 96, 64, False)])
def test_attention_kernels_with_a_cap_and_biases_by_distance(case):
    """The plain kernel (32 bit) and the tensor-core kernel (bfloat16; ``True``: single tokens with the keys split over blocks)
    against the softmax written out: capped scores, a bias by distance whose last row stands for everything farther, a sink."""
    from delta_b200.kernels import ops
    name, H, KV, dk, dv, singles = case
    dtype = torch.float32 if name == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(H + dk)
    ps, n_ctx, D = 8, 150, 37
    lens = [1, 1, 1] if singles else [40, 1, 17]
    starts = [n_ctx - n for n in lens]
    rows = len(lens)
    max_pages = -(-n_ctx // ps)
    perm = torch.randperm(rows * max_pages, generator=g).view(rows, max_pages).to(torch.int32)
    cache = (torch.randn(rows * max_pages, KV, ps, dk + dv, generator=g)).to(dtype)
    T = sum(lens)
    q = (torch.randn(T, H * dk, generator=g) * 1.5).to(dtype)
    sink = torch.randn(H, generator=g)
    dist = torch.randn(D + 1, H, generator=g) * 2
    cap, scale = 4.0, 0.3
    tok_row = torch.tensor([r for r, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    tok_pos = torch.tensor([starts[r] + j for r, n in enumerate(lens) for j in range(n)], dtype=torch.int32)
    q_start = torch.tensor([sum(lens[:r]) for r in range(rows)], dtype=torch.int32)
    out = torch.full((T, H * dv), float("nan"), dtype=dtype, device=DEV)
    # the struct holds raw addresses: the device tensors stay bound to ``on`` until the kernels have run
    on = {k: v.to(DEV) for k, v in dict(q=q, cache=cache, block_table=perm, tok_row=tok_row, tok_pos=tok_pos, row_q_start=q_start,
                                        row_q_len=torch.tensor(lens, dtype=torch.int32), row_pos_start=torch.tensor(starts, dtype=torch.int32),
                                        sink=sink, dist_bias=dist.t().contiguous()).items()}
    params = ops.row_attn_params(q_stride=H * dk, q_head_stride=dk, out=out, H=H, KV=KV, dk=dk, dv=dv, ps=ps, row_width=dk + dv, k_off=0, v_off=dk,
                                 scale=scale, softcap=cap, **on)
    if name == "float32":
        ops.attention_rows_plain(params)
    else:
        assert ops.attention_rows_mma_supported(params)
        if singles:
            splits = 4
            scratch = torch.empty(ops.attention_rows_mma_scratch_floats(T, H, dv, splits), dtype=torch.float32, device=DEV)
            ops.attention_rows_mma(params, H // KV, splits, scratch)
        else:
            params.row_filter = 1
            ops.attention_rows_mma(params, H // KV, 1, None)
            params.row_filter = 2
            ops.attention_rows_mma(params, max(lens) * (H // KV), 1, None)
    torch.cuda.synchronize()
    got = out.cpu().double().view(T, H, dv)
    worst = 0.0
    for t in range(T):
        r, p = int(tok_row[t]), int(tok_pos[t])
        rows_kv = torch.stack([cache[int(perm[r, j // ps]), :, j % ps] for j in range(p + 1)]).double()      # [keys, KV, dk + dv]
        for h in range(H):
            kv = h // (H // KV)
            s = (rows_kv[:, kv, :dk] @ q[t, h * dk:(h + 1) * dk].double()) * scale
            s = cap * torch.tanh(s / cap) + dist[torch.clamp(p - torch.arange(p + 1), max=D), h].double()
            m = max(s.max().item(), sink[h].item())
            e = torch.exp(s - m)
            want = (e[:, None] * rows_kv[:, kv, dk:]).sum(0) / (e.sum() + math.exp(sink[h].item() - m))
            worst = max(worst, (got[t, h] - want).abs().max().item())
    assert worst <= (1e-5 if name == "float32" else 2e-2), worst
    del on


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_of_the_feed_forwards_and_the_latent(dtype):
    """The gated activation with a cubic term (the tanh form of gelu), the norm of a slice of wider rows, the router's raw sigmoid
    weights, and the experts' first product (and gathered rows) when a choice's weight multiplies what the expert reads."""
    from delta_b200.kernels import ops
    from delta_b200.parts.feed_forward import GELU_TANH_GATE, SILU_GATE
    g = torch.Generator().manual_seed(3)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for F_ in (24, 50):
        gu = (torch.randn(11, 2 * F_, generator=g) * 3).to(dtype)
        for consts, fn in ((GELU_TANH_GATE, plain.gelu_tanh), (SILU_GATE, plain.silu)):
            out = torch.empty(11, F_, dtype=dtype, device=DEV)
            ops.glu_clamped(gu.to(DEV), out, -1.0, consts["alpha"], consts["shift"], consts["cubic"])
            want = fn(gu[:, :F_].double()) * gu[:, F_:].double()
            assert (out.cpu().double() - want).abs().max().item() <= tol * want.abs().max().item()
    for d, ld in ((10, 27), (96, 240)):
        x = (torch.randn(7, ld, generator=g) * 2).to(dtype)
        w = (torch.rand(d, generator=g) + 0.5).to(dtype)
        out = torch.empty(7, d, dtype=dtype, device=DEV)
        ops.rms_norm_strided(x.to(DEV), ld, w.to(DEV), 1e-6, out)
        want = plain.rms_norm(x[:, :d].double(), w, 1e-6)
        assert (out.cpu().double() - want).abs().max().item() <= tol * want.abs().max().item()
    T, d, E, top = 9, 40, 7, 3
    x, wr = torch.randn(T, d, generator=g).to(dtype), (torch.randn(E, d, generator=g) * 0.5).to(dtype)
    z = torch.empty(T, E, device=DEV)
    choice, weight = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    ops.router(x.to(DEV), wr.to(DEV), E, top, z, choice, weight, scoring="sigmoid", normalize=False)
    zz = x.double() @ wr.double().T
    order = torch.sort(zz, dim=-1, descending=True).indices[:, :top]
    assert torch.equal(torch.sort(choice.cpu().long(), dim=-1).values, torch.sort(order, dim=-1).values)
    assert (weight.cpu().double() - torch.sigmoid(torch.gather(zz, 1, choice.cpu().long()))).abs().max().item() <= 1e-5
    # the experts' first product with a weight per slot: expert(w x) = act(w (x W^T)), the rows sorted by expert into tiles
    F_ = 16
    w1 = (torch.randn(E, 2 * F_, d, generator=g) * 0.3).to(dtype)
    tile = ops.experts_tile_rows()
    slots = T * top
    capacity = -(-(slots + (tile - 1) * min(E, slots)) // tile) * tile
    sorted_slots = torch.empty(capacity, dtype=torch.int32, device=DEV)
    tile_expert = torch.empty(capacity // tile, dtype=torch.int32, device=DEV)
    ops.experts_align(choice, E, sorted_slots, tile_expert, tile)
    y = torch.zeros(capacity, F_, dtype=dtype, device=DEV)
    ops.experts_gemm(x.to(DEV), w1.to(DEV), y, sorted_slots, tile_expert, top=top, n=F_, k=d, act="gated", limit=-1.0, alpha=1.0, shift=0.0,
                     row_scale=weight.view(-1))
    at = sorted_slots.cpu().tolist()
    for p_, s_ in enumerate(at):
        if s_ < 0:
            continue
        t_, e_ = s_ // top, int(choice.view(-1)[s_])
        gu = (weight.view(-1)[s_].item() * x[t_].double()) @ w1[e_].double().T
        want = plain.silu(gu[:F_]) * gu[F_:]
        assert (y[p_].cpu().double() - want).abs().max().item() <= 3 * tol * max(1.0, want.abs().max().item())
    if dtype == torch.bfloat16:      # the rows gathered side by side for the tcgen05 product carry the weight themselves
        rows = ops.experts_gather(x.to(DEV), sorted_slots, top, torch.empty(capacity, d, dtype=dtype, device=DEV), row_scale=weight.view(-1))
        for p_, s_ in enumerate(at):
            want = weight.view(-1)[s_].item() * x[s_ // top].double() if s_ >= 0 else torch.zeros(d, dtype=torch.float64)
            assert (rows[p_].cpu().double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())


def test_ramp_scaled_rotary_table():
    """The engine's table of cos and sin against the plain frequencies and magnitude, with and without the scaling rule."""
    from delta_b200.parts.rope import RotaryPositions
    for dims, base, scaling in ((8, 1000.0, (4.0, 64, 8.0, 1.0)), (6, 300.0, (3.0, 40, 2.0, 0.5)), (32, 5e5, (6.0, 1024, 16.0, 0.75)), (16, 50.0, None)):
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        f, mag = plain.yarn_frequencies(dims, base, sc)
        t = RotaryPositions(dims, base, 300, interleaved=True, scaling=sc).table_cpu().double()
        ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
        assert (t[..., 0] - torch.cos(ang) * mag).abs().max().item() <= 1e-6 and (t[..., 1] - torch.sin(ang) * mag).abs().max().item() <= 1e-6


# ---- through the engine's own entry points -----------------------------------------------------------------------

def greedy_plain(cfg, W, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        logits, _ = plain.forward(cfg, W, toks)
        toks.append(int(torch.argmax(logits[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_backend(tmp_path_factory, graph):
    """``LMBackend``: more prompts than slots, a token budget that cuts prompts, decode steps (recorded or not)."""
    from delta_b200.engine import LMBackend
    cfg, W, folder = model(tmp_path_factory, "mix")
    prompts = [helpers.random_tokens(n, cfg["vocab"], 50 + n) for n in (4, 23, 9, 31, 2)]
    want = [greedy_plain(cfg, W, p, 10) for p in prompts]
    e = LMBackend(dtype="float32", device="cuda:0", cuda_graph_decode=graph)
    e.load_model(str(folder))
    e.setup_caches(max_batch_size=3, max_seq_length=64, page_size=16, max_tokens_per_step=16)
    got = e.generate(prompts, 10)
    assert got == want
    assert e.scheduler.stats["prefill_steps"] > 2
    if graph:
        assert e.runner.graph_replays > 0 and not e.runner.graph_fallbacks


def test_generation_survives_preemption(tmp_path_factory):
    """A pool too small for all running requests: the youngest is preempted and computed again from a fresh slot; the tokens are
    those of the plain implementation all the same."""
    from delta_b200.engine import LMBackend
    cfg, W, folder = model(tmp_path_factory, "mix")
    prompts = [helpers.random_tokens(n, cfg["vocab"], 80 + n) for n in (14, 15, 13)]
    want = [greedy_plain(cfg, W, p, 12) for p in prompts]
    e = LMBackend(dtype="float32", device="cuda:0")
    e.load_model(str(folder))
    e.setup_caches(max_batch_size=3, max_seq_length=32, page_size=4, max_tokens_per_step=16, num_pages=15)
    assert e.generate(prompts, 12) == want
    assert e.scheduler.stats["preemptions"] >= 1


def test_trace_replay_command(tmp_path_factory, tmp_path):
    """``bin/trace_run`` on a Mevulix folder: a prompt in portions beside another request's single tokens."""
    import numpy as np
    cfg, W, folder = model(tmp_path_factory, "odd")
    a, b = helpers.random_tokens(21, cfg["vocab"], 3), helpers.random_tokens(12, cfg["vocab"], 4)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:7], want=[6])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[7:9], want=[0, 1]), dict(id="b", tokens=b[:11], want=[10])], end=[]),
             dict(step=2, entries=[dict(id="b", tokens=b[11:], want=[0]), dict(id="a", tokens=a[9:], want=[11])], end=["a", "b"])]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128", "--page-size", "4"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ra, rb = plain.forward(cfg, W, a)[0], plain.forward(cfg, W, b)[0]
    V = cfg["vocab"]
    got = {k: torch.from_numpy(np.fromfile(out / f"{k}.f32", dtype="<f4").reshape(-1, V)).double() for k in range(3)}
    want = {0: ra[[6]], 1: torch.cat([ra[[7, 8]], rb[[10]]]), 2: torch.cat([rb[[11]], ra[[20]]])}
    for k in range(3):
        assert got[k].shape == want[k].shape
        assert (got[k] - want[k]).abs().max().item() <= TOL["float32"] * want[k].abs().max().item()


def test_command_line_generates(tmp_path_factory, tmp_path):
    """``python -m delta_b200.cli`` on a Mevulix folder: the model class comes from config.json, prompts are scheduled and sampled."""
    import random
    from delta_b200 import cli
    cfg, W, folder = model(tmp_path_factory, "one")
    out = tmp_path / "result.json"
    rc = cli.main(["--model", str(folder), "--B", "3", "--max_len", "128", "--dataset", "random", "--prompt_len", "19", "--num_samples", "5",
                   "--max_new_tokens", "6", "--dtype", "float32", "--max_tokens_per_step", "32", "--out", str(out)])
    assert rc == 0
    res = json.loads(out.read_text())
    assert res["summary"]["requests"] == 5 and res["summary"]["generated_tokens"] == 30
    rng = random.Random(123)       # the command line's default seed draws the prompts
    prompt = [rng.randrange(cfg["vocab"]) for _ in range(19)]
    first = [r for r in res["results"] if r["request_id"] == 0][0]
    assert first["output_ids"] == greedy_plain(cfg, W, prompt, 6)
