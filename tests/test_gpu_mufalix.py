"""The Mufalix design in the engine against the plain float64 implementation, on the GPU, in 32 bit and in bfloat16:
each mechanism alone (one-mechanism models, single kernels, and the stream after every layer run), each request whole,
prefill against token-by-token decoding, portions down to two tokens, mixed batches with pages, slots and states that
are used again, keys at a window's edges and states carried across many tiny pages, long decoding, and greedy
generation through ``LMBackend``, the command line and the replay command."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
import mufalix_helpers as mh
import plain_mufalix as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# 32 bit: the largest difference of a logit (or a stream entry) as a fraction of the largest value of its request's
# reference.  bfloat16: the root mean square of a position's differences as a fraction of that of the request's
# reference logits, and at most three times what rounding alone causes.
TOL = {"float32": 2e-5, "bfloat16": 6e-2}
LENGTHS = {"wide": [250, 5, 199, 64], "mix": [3, 37, 60, 121], "odd": [1, 7, 26, 45], "one": [2, 25, 33, 58], "sharp": [1, 40, 97, 150],
           "only_memory": [1, 9, 40, 75], "only_pair": [2, 30, 47], "only_experts": [1, 6, 21, 50], "only_loop": [1, 2, 19]}
_cache = {}


def model(tmp_path_factory, which):
    if which not in _cache:
        cfg = mh.config(which)
        W = mh.make_weights(cfg, 23 + len(which))
        folder = mh.write_folder(tmp_path_factory.mktemp("mufalix"), which, cfg, W)
        _cache[which] = (cfg, W, folder)
    return _cache[which]


def make_runner(folder, which, dtype, num_pages=None, max_batch=4, max_seq_len=256, **kw):
    from delta_b200.config import EngineConfig
    from delta_b200.engine.step import ModelRunner
    ps = mh.PAGE_SIZE[which] if isinstance(which, str) else int(which)
    cfg = EngineConfig(max_batch=max_batch, max_seq_len=max_seq_len, page_size=ps, dtype=dtype,
                       num_pages=num_pages if num_pages is not None else max_batch * (max_seq_len // ps), **kw)
    return ModelRunner(folder, engine_config=cfg)


CLOSE_CALL = 0.02      # a router's choice decided by less than this (in score) may fall either way once the input is rounded to bfloat16


class Noise(list):
    """Per request and position the error that bfloat16 rounding alone causes: the plain implementation with rounding against itself
    without, and at least twice the median of that over the positions before the rounded run chooses other experts than the exact
    one (if it does).  Single positions can be far above the median, where a matrix memory's denominator |z . q| nearly cancels.  ``margins``: per request and
    position the smallest margin by which any router decided.  A choice that falls the other way changes that position and, through
    the states, the ones behind it: ``compare`` accepts a first difference at a position with a close call and leaves the rest of
    that request out."""
    margins = None


def routed(cfg, W, t):
    plain.MARGINS, plain.CHOICES = [], []
    logits = plain.forward(cfg, W, t)[0]
    m, c = plain.MARGINS, plain.CHOICES
    plain.MARGINS, plain.CHOICES = None, []
    return logits, (torch.stack(m).min(dim=0).values if m else torch.full((len(t),), 9.0)), c


def rounding_noise(cfg, W, toks, refs):
    out = Noise()
    out.margins = []
    for t, ref in zip(toks, refs):
        _, margins, exact = routed(cfg, W, t)
        with plain.rounding("bfloat16"):
            em, _, rounded = routed(cfg, W, t)
        same = len(t)
        for a, b in zip(exact, rounded):
            other = (a != b).any(dim=-1).nonzero()
            if other.numel():
                same = min(same, int(other[0, 0]))
        out.margins.append(margins)
        err = (em - ref).pow(2).mean(dim=1).sqrt()
        out.append(torch.clamp(err, min=2.0 * err[:max(same, 1)].median().item()))
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
            # bfloat16: the bound is an estimate from one rounded run, and where a matrix memory's denominator nearly cancels one
            # run says little about another.  A close call of a router ends the comparison of the request; otherwise one
            # position in fifty may be over the bound, by less than three times.
            outliers = []
            for p in bad:
                if noise.margins[i % len(noise)][p] < CLOSE_CALL:
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
    worst["mixed"] = compare(res, refs * 3, lengths * 3, dtype, "mixed with pages, slots and states used again", noise)
    print(f"\nworst logit error {which} {dtype}: " + ", ".join(f"{k} {v:.2e}" for k, v in worst.items()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_larger_sizes(tmp_path_factory, dtype):
    """Width 512, 8 experts, heads of 64 and 128: a 700-token prompt whole (about 175 rows an expert: the tcgen05 products; the
    memory's chunks and the recurrence's segments in parallel; the library's batched product for the gates), in portions of 256
    beside a second request, and its last tokens one by one."""
    cfg, W, folder = model(tmp_path_factory, "larger")
    lengths = [700, 130]
    toks = [helpers.random_tokens(n, cfg["vocab"], 900 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    runner = make_runner(folder, "larger", dtype, max_batch=2, max_seq_len=704, max_tokens_per_step=1024)
    compare(helpers.run_schedule(runner, toks, helpers.whole(lengths)), refs, lengths, dtype, "whole", noise)
    steps = [[(0, 0, 256), (1, 0, 100)], [(0, 256, 256), (1, 100, 1)], [(0, 512, 180), (1, 101, 29)]] + [[(0, p, 1)] for p in range(692, 700)]
    compare(helpers.run_schedule(runner, toks, steps), refs, lengths, dtype, "portions of 256 beside a second request", noise)


@pytest.mark.parametrize("which", ["mix", "odd", "one", "only_memory", "only_pair", "only_experts", "only_loop"])
def test_stream_after_every_layer_run(tmp_path_factory, which):
    """32 bit: the residual stream after every run of a layer, for a prompt in one step and for the same prompt cut in two."""
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
            assert err <= TOL["float32"] * after[r].abs().max().item(), f"{which}: layer run {r} differs by {err:.3e} (cut at {cut})"


@pytest.mark.parametrize("which,dtype", [("mix", "float32"), ("odd", "float32"), ("mix", "bfloat16")])
def test_long_decoding(tmp_path_factory, which, dtype):
    """A short prompt, then 180 tokens one by one: pages fill one after the other and leave the window, the memories, the
    recurrence and the convolution's inputs are carried 180 times."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["only_pair", "mix", "odd"])
def test_long_portions_run_their_segments_in_parallel(tmp_path_factory, which, dtype):
    """Portions long enough for the recurrence's segments to run in parallel: several segments, one that ends in the middle of
    a segment, rows of unequal length in one batch (some a single token), and a state carried on into single tokens."""
    cfg, W, folder = model(tmp_path_factory, which)
    lengths = [150, 9, 117, 33]
    toks = [helpers.random_tokens(n, cfg["vocab"], 300 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    runner = make_runner(folder, which, dtype)
    steps = [[(0, 0, 100), (1, 0, 8), (2, 0, 17)], [(0, 100, 41), (1, 8, 1), (2, 17, 97), (3, 0, 32)], [(0, 141, 1), (3, 32, 1), (2, 114, 3)]]
    steps += [[(0, p, 1)] for p in range(142, 150)]
    res = helpers.run_schedule(runner, toks, steps)
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    print("\nsegments in parallel worst", compare(res, refs, lengths, dtype, "long portions", noise))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_the_edges_of_segments(tmp_path_factory, dtype):
    """Portions of exactly one and two segments, one token more and one less, on both sides of the length from which the
    segments run in parallel; every request goes on with a portion that starts in the middle of a segment and ends on an edge."""
    from delta_b200.parts import gated_recurrence
    c = gated_recurrence.SEGMENT
    cfg, W, folder = model(tmp_path_factory, "only_pair")
    first = [c, c + 1, 2 * c, 2 * c + 1, 3 * c - 1, 1, c - 1]
    lengths = [4 * c for _ in first]           # every request ends at 4 segments
    toks = [helpers.random_tokens(n, cfg["vocab"], 500 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    for together in (True, False):      # the rows in one batch (the longest decides the path), and each alone (its own path)
        runner = make_runner(folder, "only_pair", dtype, max_batch=len(first), max_seq_len=4 * c)
        if together:
            steps = [[(i, 0, n) for i, n in enumerate(first)], [(i, n, lengths[i] - n) for i, n in enumerate(first)]]
        else:
            steps = [[(i, 0, n)] for i, n in enumerate(first)] + [[(i, n, lengths[i] - n)] for i, n in enumerate(first)]
        res = helpers.run_schedule(runner, toks, steps)
        compare(res, refs, lengths, dtype, f"segment edges, together={together}", noise)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_the_edges_of_the_memorys_chunks(tmp_path_factory, dtype):
    """The matrix memory alone: portions of two, three and four chunks, one token more and one less, on both sides of the length
    from which the chunks run in parallel; every request goes on with a portion that starts inside a chunk."""
    from delta_b200.kernels import ops
    from delta_b200.parts import matrix_memory
    c, start = ops.matrix_memory_chunk(), matrix_memory.PARALLEL_FROM
    cfg, W, folder = model(tmp_path_factory, "only_memory")
    first = [start - 1, start, 2 * c, 2 * c + 1, 3 * c - 1, 4 * c, 1, c + 1]
    lengths = [6 * c + 3 for _ in first]
    toks = [helpers.random_tokens(n, cfg["vocab"], 700 + i) for i, n in enumerate(lengths)]
    refs = [plain.forward(cfg, W, t)[0] for t in toks]
    noise = rounding_noise(cfg, W, toks, refs) if dtype == "bfloat16" else None
    for together in (True, False):
        runner = make_runner(folder, "only_memory", dtype, max_batch=len(first), max_seq_len=8 * c)
        if together:
            steps = [[(i, 0, n) for i, n in enumerate(first)], [(i, n, lengths[i] - n) for i, n in enumerate(first)]]
        else:
            steps = [[(i, 0, n)] for i, n in enumerate(first)] + [[(i, n, lengths[i] - n)] for i, n in enumerate(first)]
        res = helpers.run_schedule(runner, toks, steps)
        compare(res, refs, lengths, dtype, f"chunk edges of the memory, together={together}", noise)


@pytest.mark.parametrize("sizes", [(2, 16, 8), (3, 7, 5), (1, 64, 96), (2, 24, 72)])
@pytest.mark.parametrize("gates", ["usual", "closing", "wide open", "late burst"])
def test_the_memorys_chunks_in_parallel_against_the_tokens_in_turn(sizes, gates):
    """The two kernels of the matrix memory and the plain recurrence, 32 bit, on rows of unequal lengths that continue from a state
    left by an earlier call; with forget gates that nearly close (the sum of their logarithms inside a chunk is large), input
    gates at the cap, and a burst of large input gates late in a row (the running maximum jumps inside a chunk)."""
    from delta_b200.kernels import ops
    H, dk, dv = sizes
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(H * 100 + dk)
    cap = 12.0
    lens1, lens2 = [70, 33, 1, 128], [95, 64, 140, 31]
    rows = len(lens1)
    stride = 2 * H * dk + H * dv + 5

    def draw(T):
        src = torch.randn(T, stride, generator=gen)
        gi, gf = torch.randn(T, H, generator=gen) * 2, torch.randn(T, H, generator=gen) * 2 + 3
        if gates == "closing":
            gf = gf - 6.0
        if gates == "wide open":
            gi, gf = gi + 20.0, gf + 20.0
        if gates == "late burst":
            gi[T // 2 + 3:T // 2 + 6] += 14.0
            gi[:T // 2] -= 8.0
        return src, torch.cat([gi, gf], dim=1)

    def plain_rows(parts):       # parts: per row [(src, g), ...] in order; the plain recurrence over the row's whole history
        outs = []
        for pieces in parts:
            src = torch.cat([p[0] for p in pieces]).double()
            g = torch.cat([p[1] for p in pieces]).double()
            T = src.shape[0]
            q = src[:, :H * dk].view(T, H, dk) * dk ** -0.5
            k = src[:, H * dk:2 * H * dk].view(T, H, dk)
            v = src[:, 2 * H * dk:2 * H * dk + H * dv].view(T, H, dv)
            li = plain.capped(g[:, :H], cap)
            lf = torch.nn.functional.logsigmoid(plain.capped(g[:, H:], cap))
            o, cond = plain.matrix_memory(q, k, v, li, lf, with_condition=True)
            outs.append((o.reshape(T, H * dv), cond.max(dim=1).values))
        return outs

    pieces = [[draw(n)] for n in lens1]
    for i, n in enumerate(lens2):
        pieces[i].append(draw(n))
    want = plain_rows(pieces)
    bias = torch.zeros(2 * H, device=dev)
    results = {}
    for how in ("in turn", "in turn, sliced", "in parallel", "parallel then turn"):
        S = torch.zeros(rows, H, dk, dv, device=dev)
        z = torch.zeros(rows, H, dk, device=dev)
        m = torch.zeros(rows, H, device=dev)
        got = [[] for _ in range(rows)]
        for call, lens in enumerate((lens1, lens2)):
            src = torch.cat([pieces[i][call][0] for i in range(rows)]).to(dev)
            g = torch.cat([pieces[i][call][1] for i in range(rows)]).to(dev).contiguous()
            T = src.shape[0]
            starts = [sum(lens[:i]) for i in range(rows)]
            meta = dict(row_slot=torch.arange(rows, dtype=torch.int32, device=dev).flip(0).contiguous(),
                        row_q_start=torch.tensor(starts, dtype=torch.int32, device=dev), row_q_len=torch.tensor(lens, dtype=torch.int32, device=dev))
            out = torch.full((T, H * dv), float("nan"), device=dev)
            parallel = how == "in parallel" or (how == "parallel then turn" and call == 0)
            if parallel:
                c = ops.matrix_memory_chunk()
                counts = [-(-n // c) for n in lens]
                base = torch.tensor([sum(counts[:i]) for i in range(rows)], dtype=torch.int32, device=dev)
                work = torch.full((ops.matrix_memory_chunked_work(sum(counts), H, dk, dv),), float("nan"), device=dev)
                ops.matrix_memory_chunked(src, 0, H * dk, 2 * H * dk, dk ** -0.5, g, bias, cap, 1e-6, S, z, m, out, work, base, sum(counts),
                                          max(counts), H=H, dk=dk, dv=dv, **meta)
            else:
                ops.matrix_memory(src, 0, H * dk, 2 * H * dk, dk ** -0.5, g, bias, cap, 1e-6, S, z, m, out, H=H, dk=dk, dv=dv,
                                  slice_=max(1, dv // 3) if how.endswith("sliced") else None, **meta)
            for i in range(rows):
                got[i].append(out[starts[i]:starts[i] + lens[i]].cpu().double())
        results[how] = (S.cpu(), z.cpu(), m.cpu())
        for i in range(rows):
            o = torch.cat(got[i])
            assert torch.isfinite(o).all(), f"{how}: row {i} has entries that are not finite"
            ref, cond = want[i]       # where |z . q| nearly cancels, 32-bit rounding of the denominator is that much larger in the output
            err = (o - ref).abs().max(dim=1).values
            bad = (err > 2e-5 * ref.abs().max().item() + 1e-6 + 2e-6 * cond * ref.abs().max(dim=1).values).nonzero()
            assert not bad.numel(), f"{how}: row {i} first differs at token {int(bad[0, 0])}: {err[int(bad[0, 0])].item():.3e}"
    for how in ("in turn, sliced", "in parallel", "parallel then turn"):      # the states the two kernels leave are the same up to rounding
        for a, b, name in zip(results["in turn"], results[how], ("memory", "keys' sum", "maximum")):
            assert (a - b).abs().max().item() <= 2e-5 * a.abs().max().item() + 1e-6, f"{how}: the {name} left behind differs"


@pytest.mark.parametrize("sizes", [(2, 16, 8), (3, 7, 12), (1, 64, 96), (2, 24, 200)])
def test_the_memorys_single_tokens(sizes):
    """The kernel for steps of single tokens against the plain recurrence, 32 bit: 40 steps of four rows whose slots are not in
    order, one of them with input gates at the cap from its 20th token on."""
    from delta_b200.kernels import ops
    H, dk, dv = sizes
    assert ops.matrix_memory_step_supported(dk, dv)
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(dk * 7 + dv)
    cap, rows, steps = 10.0, 4, 40
    stride = 2 * H * dk + H * dv + 3
    src = torch.randn(steps, rows, stride, generator=gen)
    g = torch.cat([torch.randn(steps, rows, H, generator=gen) * 2, torch.randn(steps, rows, H, generator=gen) * 2 + 3], dim=2)
    g[20:, 1, :H] += 25.0
    S = torch.zeros(rows + 2, H, dk, dv, device=dev)
    z = torch.zeros(rows + 2, H, dk, device=dev)
    m = torch.zeros(rows + 2, H, device=dev)
    slots = torch.tensor([4, 0, 5, 2], dtype=torch.int32, device=dev)
    starts = torch.arange(rows, dtype=torch.int32, device=dev)
    bias = torch.zeros(2 * H, device=dev)
    got = []
    for t in range(steps):
        out = torch.full((rows, H * dv), float("nan"), device=dev)
        ops.matrix_memory_step(src[t].to(dev), 0, H * dk, 2 * H * dk, dk ** -0.5, g[t].to(dev).contiguous(), bias, cap, 1e-6, S, z, m, out,
                               H=H, dk=dk, dv=dv, row_slot=slots, row_q_start=starts)
        got.append(out.cpu().double())
    got = torch.stack(got)       # [steps, rows, H * dv]
    assert S[1].abs().max().item() == 0 and S[3].abs().max().item() == 0, "a slot of no row was written"
    for r in range(rows):
        x, gr = src[:, r].double(), g[:, r].double()
        q = x[:, :H * dk].view(steps, H, dk) * dk ** -0.5
        k = x[:, H * dk:2 * H * dk].view(steps, H, dk)
        v = x[:, 2 * H * dk:2 * H * dk + H * dv].view(steps, H, dv)
        ref, cond = plain.matrix_memory(q, k, v, plain.capped(gr[:, :H], cap), torch.nn.functional.logsigmoid(plain.capped(gr[:, H:], cap)),
                                        with_condition=True)
        ref = ref.reshape(steps, H * dv)
        err = (got[:, r] - ref).abs().max(dim=1).values
        bad = (err > 2e-5 * ref.abs().max().item() + 1e-6 + 2e-6 * cond.max(dim=1).values * ref.abs().max(dim=1).values).nonzero()
        assert not bad.numel(), f"row {r} first differs at step {int(bad[0, 0])}: {err[int(bad[0, 0])].item():.3e}"


def test_a_slot_used_again_starts_clean(tmp_path_factory):
    """Request B after request A in the same slot and pages equals B alone: memories, maxima, recurrence, the convolution's
    inputs and the cache of A are gone."""
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


# ---- weights made so that one key, one gate or the sink decides ---------------------------------------------------

def crafted_window(window, sink, seed=77):
    """One pair of mixers whose left half has a single head without rotation; its key matrix is a permutation P and token 1's
    embedding is P times token 0's, so a query of token 1 meets a key of token 0 with the largest score there is (the head
    size), and no other key comes close.  Token 0 stands at A; token 1 at A + window - 1 (the last place that still sees A)
    and at A + window (the first that does not)."""
    d = 32
    cfg = dict(architecture="Mufalix", norm=dict(eps=1e-5), vocab=64, width=d,
               layers=[mh.bare(mh.parallel(mh.left(1, 1, d, d, 1.0, window=window), 8, 2, 1))])
    g = torch.Generator().manual_seed(seed)
    W = mh.make_weights(cfg, 9)
    P = torch.eye(d)[torch.randperm(d, generator=g)]
    W["embed"][1] = P @ W["embed"][0]
    p = "l0.mix.left."
    W[p + "q"], W[p + "k"] = torch.eye(d), P.clone()
    W[p + "q.b"], W[p + "k.b"] = torch.zeros(d), torch.zeros(d)
    W[p + "q.norm"], W[p + "k.norm"], W["l0.norm1"] = torch.ones(d), torch.ones(d), torch.ones(d)
    W[p + "sink"] = torch.full((1,), float(sink))
    n, a_at = 80, 30
    toks = [2 + t % 62 for t in helpers.random_tokens(n, 62, 8)]
    toks[a_at] = 0
    toks[a_at + window - 1] = toks[a_at + window] = 1
    return cfg, W, toks, a_at


def with_left(cfg, **changes):
    import copy
    c = copy.deepcopy(cfg)
    for k, v in changes.items():
        if k == "window":
            c["layers"][0]["mixer"]["left"]["mask"]["size"] = v
    return c


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sink", [0.0, 30.0])
def test_a_key_at_the_windows_edge_and_the_sink(tmp_path_factory, dtype, sink):
    """The last query that sees the crafted key and the first that does not, in a whole prompt, decoded alone, ending a portion
    and opening one, over pages of four tokens (the window starts and ends inside pages).  A window one token longer or
    shorter, or a softmax without the sink, changes the plain implementation's logits there beyond any tolerance."""
    window = 21
    cfg, W, toks, a_at = crafted_window(window, sink)
    n, b_in, b_out = len(toks), a_at + window - 1, a_at + window
    ref = plain.forward(cfg, W, toks)[0]
    size = ref.abs().max().item()
    longer, shorter = plain.forward(with_left(cfg, window=window + 1), W, toks)[0], plain.forward(with_left(cfg, window=window - 1), W, toks)[0]
    assert (longer[b_out] - ref[b_out]).abs().max().item() > 0.1 * size, "a window one token longer would not show"
    assert (shorter[b_in] - ref[b_in]).abs().max().item() > 0.1 * size, "a window one token shorter would not show"
    no_sink = dict(W)
    no_sink["l0.mix.left.sink"] = torch.full((1,), -30.0)
    diff = (plain.forward(cfg, no_sink, toks)[0] - ref).abs().max(dim=1).values
    assert diff[0].item() > 0.2 * size, "a softmax without the sink would not show at the first token"
    if sink > 0:        # a sink this large takes most of the weight wherever the crafted key is not seen
        assert diff.median().item() > 0.2 * size
    folder = mh.write_folder(tmp_path_factory.mktemp("edge"), f"edge{int(sink)}", cfg, W)
    runner = make_runner(folder, 4, dtype, max_batch=2, max_seq_len=96)
    noise = rounding_noise(cfg, W, [toks], [ref]) if dtype == "bfloat16" else None
    for what, steps in (("whole", [[(0, 0, n)]]),
                        ("both decoded alone", [[(0, 0, b_in - 3)]] + [[(0, p, 1)] for p in range(b_in - 3, n)]),
                        ("one ends a portion, the other opens the next", [[(0, 0, 2)], [(0, 2, b_in - 1)], [(0, b_out, n - b_out)]]),
                        ("portions of two", [[(0, 0, a_at + 1)]] + [[(0, p, 2)] for p in range(a_at + 1, n - 1, 2)] + [[(0, n - 1, 1)]])):
        compare(helpers.run_schedule(runner, [toks], steps), [ref], [n], dtype, what, noise)


def crafted_memory(seed=78):
    """One matrix memory of one head whose key matrix is a permutation P, token 1's embedding P times token 0's, and an input
    gate that opens wide for token 0 alone while the forget gate stays next to 1: what token 0 wrote near the start is most
    of the memory 140 tokens later, when token 1 asks for it."""
    d = 32
    cfg = dict(architecture="Mufalix", norm=dict(eps=1e-5), vocab=64, width=d, layers=[mh.bare(mh.mlstm(1, d, d, 12.0))])
    g = torch.Generator().manual_seed(seed)
    W = mh.make_weights(cfg, 10)
    P = torch.eye(d)[torch.randperm(d, generator=g)]
    W["embed"][1] = P @ W["embed"][0]
    p = "l0.mix."
    W[p + "q"], W[p + "k"], W["l0.norm1"] = torch.eye(d), P.clone(), torch.ones(d)
    h0 = W["embed"][0] / W["embed"][0].pow(2).mean().sqrt()
    W[p + "i"], W[p + "i.b"] = (h0 * (10.0 / d)).view(1, d).to(torch.bfloat16).float(), torch.full((1,), -4.0)
    W[p + "f"], W[p + "f.b"] = torch.zeros(1, d), torch.full((1,), 8.0)
    n, a_at, b_at = 150, 3, 140
    toks = [2 + t % 62 for t in helpers.random_tokens(n, 62, 11)]
    toks[a_at], toks[b_at] = 0, 1
    return cfg, W, toks, a_at, b_at


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_stays_in_the_memory(tmp_path_factory, dtype):
    """The crafted write is read 137 tokens later: in a whole prompt, with the reader decoded alone, and with the prompt cut so
    that the write ends a portion and the reader opens one.  Before the write the input gates are negative, so the running
    maximum is the one the memory starts with (zero): a maximum that started at minus infinity changes those logits."""
    cfg, W, toks, a_at, b_at = crafted_memory()
    n = len(toks)
    ref = plain.forward(cfg, W, toks)[0]
    size = ref.abs().max().item()
    without = list(toks)
    without[a_at] = 5
    assert (plain.forward(cfg, W, without)[0][b_at] - ref[b_at]).abs().max().item() > 0.2 * size, "the crafted write does not carry the weight"
    folder = mh.write_folder(tmp_path_factory.mktemp("memory"), "memory", cfg, W)
    runner = make_runner(folder, 8, dtype, max_batch=2, max_seq_len=160)
    noise = rounding_noise(cfg, W, [toks], [ref]) if dtype == "bfloat16" else None
    for what, steps in (("whole", [[(0, 0, n)]]), ("the reader decoded alone", [[(0, 0, b_at)]] + [[(0, p, 1)] for p in range(b_at, n)]),
                        ("the reader opens a portion", [[(0, 0, 2)], [(0, 2, b_at - 2)], [(0, b_at, n - b_at)]]),
                        ("the write ends a portion", [[(0, 0, a_at)], [(0, a_at, 1)], [(0, a_at + 1, b_at - a_at)], [(0, b_at + 1, n - b_at - 1)]]),
                        ("token by token from the start", [[(0, p, 1)] for p in range(n)])):
        compare(helpers.run_schedule(runner, [toks], steps), [ref], [n], dtype, what, noise)


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
    """A pool too small for all running requests: the youngest is preempted and computed again from a fresh slot, whose
    memories, recurrence and convolution inputs start over; the tokens are those of the plain implementation all the same."""
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
    """``bin/trace_run`` on a Mufalix folder: a prompt in portions beside another request's single tokens."""
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
    """``python -m delta_b200.cli`` on a Mufalix folder: the model class comes from config.json, prompts are scheduled and sampled."""
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
