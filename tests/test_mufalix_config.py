"""Mufalix on the CPU: the configuration reader, the run order, the specification's tensor list against the names the
tests write out on their own, and properties of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import mufalix_helpers as mh
import plain_mufalix as plain

ALL = ["larger", "wide", "mix", "odd", "one", "sharp", "only_memory", "only_pair", "only_experts", "only_loop"]
F = torch.float64


def build(which):
    import delta_b200.models  # noqa: F401
    from delta_b200.config.registry import architecture_of
    from delta_b200.models import Model
    cfg = mh.config(which)
    arch = architecture_of(cfg)
    typed = arch.config_from_dict(cfg)
    return cfg, typed, Model(arch.build_spec(typed, None))


@pytest.mark.parametrize("which", ALL)
def test_tensor_list(which):
    cfg, typed, model = build(which)
    want = {k: tuple(v.shape) for k, v in mh.make_weights(cfg, 1).items()}
    got = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert got == want


def test_run_order_and_passes():
    cfg, typed, model = build("mix")
    assert typed.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert [(i, p is not None) for i, p in typed.run_order()] == plain.run_order(cfg)
    assert [e.enters_pass for e in model.order] == [None, 0, None, 1, None, None]
    assert len({e.cache for e in model.order}) == 6        # every run has a cache or state of its own
    cfg, typed, model = build("odd")
    assert [e.enters_pass for e in model.order] == [0, None, 1, None, 2, None, None]
    cfg, typed, model = build("one")                       # a span that runs once still enters its pass through the projection
    assert [e.enters_pass for e in model.order] == [None, 0, None]
    cfg, typed, model = build("sharp")                     # no span: no projection, and no tensor for it
    assert [e.enters_pass for e in model.order] == [None, None]
    assert "loop.in" not in {s.name for s in model.tensor_specs()}


def test_state_and_cache_declared_per_run():
    cfg, typed, model = build("mix")
    states = model.state_specs()
    by_run = {}
    for k, s in states.items():
        if k.startswith("run"):
            by_run.setdefault(k.split(".")[0], {})[k.split(".", 1)[1]] = s
    # runs 0, 2, 4 are matrix memories; runs 1, 3, 5 pairs whose right half keeps a convolution's inputs and a recurrence
    assert sorted(by_run) == [f"run{r}" for r in range(6)]
    assert {k: tuple(v.shape) for k, v in by_run["run0"].items()} == {"memory": (3, 16, 24), "normalizer": (3, 16), "maximum": (3,)}
    assert {k: tuple(v.shape) for k, v in by_run["run2"].items()} == {"memory": (2, 24, 16), "normalizer": (2, 24), "maximum": (2,)}
    assert {k: tuple(v.shape) for k, v in by_run["run3"].items()} == {"conv": (3, 64), "recurrence": (64,)}
    assert {k: tuple(v.shape) for k, v in by_run["run5"].items()} == {"conv": (1, 48), "recurrence": (48,)}
    assert all(s.dtype == torch.float32 and s.fill == 0.0 for d in by_run.values() for s in d.values())
    assert sorted(model.cache_specs()) == [1, 3, 5]          # the pairs' left halves keep pages; one cache per run
    assert model.has_run_state()


def test_config_errors():
    from delta_b200.config.model_config import ConfigError
    from delta_b200.config.mufalix_config import MufalixConfig
    good = mh.config("mix")
    MufalixConfig.from_dict(good)
    for path, value, text in ((("layers", 1, "mixer", "left", "kv_heads"), 3, "multiple"), (("loop", "stop"), 9, "loop"),
                              (("loop", "times"), 0, "loop"), (("layers", 1, "mlp", "router", "top"), 7, "top"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 15, "rot.dims"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 26, "rot.dims"),
                              (("layers", 1, "mixer", "left", "mask", "size"), 0, "window"),
                              (("layers", 1, "mixer", "right", "blocks"), 3, "equal parts"),
                              (("layers", 1, "mixer", "right", "conv"), 0, "tap"),
                              (("layers", 0, "mixer", "gate_cap"), 0.0, "gate_cap"),
                              (("layers", 0, "type"), "mamba", "unknown mixer"), (("layers", 0, "mlp", "kind"), "glu", "feed-forward kind")):
        bad = copy.deepcopy(good)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            MufalixConfig.from_dict(bad)
    for key in ("vocab", "width", "norm", "layers"):
        bad = {k: v for k, v in good.items() if k != key}
        with pytest.raises(ConfigError, match=key):
            MufalixConfig.from_dict(bad)
    for path in (("layers", 0, "mixer", "gate_cap"), ("layers", 1, "mixer", "left", "scale"), ("layers", 1, "mixer", "right", "conv"),
                 ("layers", 1, "mixer", "left", "rot", "scaling", "high"), ("layers", 1, "mlp", "expert", "ff")):
        bad = copy.deepcopy(good)
        at = bad
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=path[-1]):
            MufalixConfig.from_dict(bad)


def test_engine_frequencies_match_the_plain_ones():
    """The engine's table of scaled frequencies against the plain implementation's, in all three ranges of wavelength."""
    from delta_b200.parts import rope
    for base, dims, scaling in ((1000.0, 16, (8.0, 1.0, 4.0, 64)), (300.0, 6, (3.0, 0.5, 2.0, 40)), (20000.0, 32, (4.0, 1.0, 4.0, 32)),
                                (50.0, 2, None), (5000.0, 32, (2.0, 1.0, 2.0, 128))):
        sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
        want = plain.scaled_frequencies(base, dims, sc)
        got = rope.RotaryPositions(dims, base, 8, scaling=sc).frequencies()
        assert torch.allclose(torch.as_tensor(got, dtype=F), want, rtol=1e-12, atol=0)
    kept = plain.scaled_frequencies(1000.0, 16, dict(factor=8.0, low=1.0, high=4.0, original=64))
    plainf = plain.scaled_frequencies(1000.0, 16, None)
    ratio = (plainf / kept)
    assert ratio[0] == 1.0 and abs(ratio[-1].item() - 8.0) < 1e-12 and ((ratio > 1.0 + 1e-9) & (ratio < 8.0 - 1e-9)).any()


def test_plain_sink_window_and_rotation():
    """A lone first token attends to itself with weight e^s / (e^s + e^sink), not 1; a window of one token sees itself only;
    rotation pairs entry i with entry i + dims/2 and leaves the rest."""
    q = torch.randn(3, 2, 4, dtype=F)
    k = torch.randn(3, 1, 4, dtype=F)
    v = torch.randn(3, 1, 5, dtype=F)
    sink = torch.tensor([0.3, -1.1], dtype=F)
    out = plain.sink_window_attention(q, k, v, 0.7, 1, sink)
    for t in range(3):
        for h in range(2):
            s = (q[t, h] @ k[t, 0]) * 0.7
            assert torch.allclose(out[t, h], torch.exp(s) / (torch.exp(s) + torch.exp(sink[h])) * v[t, 0])
    out = plain.sink_window_attention(q, k, v, 0.7, 2, sink)
    s0, s1 = (q[2, 1] @ k[1, 0]) * 0.7, (q[2, 1] @ k[2, 0]) * 0.7
    den = torch.exp(s0) + torch.exp(s1) + torch.exp(sink[1])
    assert torch.allclose(out[2, 1], (torch.exp(s0) * v[1, 0] + torch.exp(s1) * v[2, 0]) / den)
    x = torch.arange(6, dtype=F).view(1, 1, 6) + 1.0
    f = torch.tensor([0.5, 0.25], dtype=F)
    y = plain.rotate_half(x, torch.tensor([3]), f)[0, 0]
    a0, a1 = 1.5, 0.75
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5.0, 6.0]
    assert torch.allclose(y, torch.tensor(want, dtype=F))


def test_plain_memory_first_token_and_recurrence():
    """The matrix memory's running maximum starts at 0: with a negative input gate the first token's maximum is
    max(log_f, log_i), not log_i.  The recurrence treats the first token like every other (the state before it is 0)."""
    q, k = torch.randn(1, 1, 4, dtype=F), torch.randn(1, 1, 4, dtype=F)
    v = torch.randn(1, 1, 3, dtype=F)
    li, lf = torch.tensor([[-3.0]], dtype=F), torch.tensor([[-0.2]], dtype=F)
    out = plain.matrix_memory(q, k, v, li, lf)[0, 0]
    mx = max(-0.2, -3.0)
    take = math.exp(-3.0 - mx)
    dot = (k[0, 0] @ q[0, 0]).item()
    want = take * dot * v[0, 0] / (max(abs(take * dot), math.exp(-mx)) + 1e-6)
    assert torch.allclose(out, want)
    u = torch.randn(2, 3, dtype=F)
    r, i = torch.rand(2, 3, dtype=F), torch.rand(2, 3, dtype=F)
    lam = torch.tensor([-2.0, 0.0, 1.5], dtype=F)
    S = plain.gated_linear_recurrence(u, r, i, lam)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam))
    s0 = torch.sqrt(1 - a[0] ** 2) * i[0] * u[0]
    assert torch.allclose(S[0], s0)
    assert torch.allclose(S[1], a[1] * s0 + torch.sqrt(1 - a[1] ** 2) * i[1] * u[1])


def test_plain_router_correction_enters_the_choice_only():
    h = torch.randn(5, 8, dtype=F)
    w = torch.randn(4, 8, dtype=F)
    corr = torch.tensor([0.0, 5.0, 0.0, -5.0], dtype=F)         # expert 1 is always chosen, expert 3 never
    choice, weight = plain.route(h, w, corr, 2, 2.5)
    s = torch.sigmoid(h @ w.T)
    assert (choice[:, 0] == 1).all() and not (choice == 3).any()
    picked = torch.gather(s, 1, choice)
    assert torch.allclose(weight, picked / picked.sum(-1, keepdim=True) * 2.5)
    assert torch.allclose(weight.sum(-1), torch.full((5,), 2.5, dtype=F))


def test_a_feed_forward_without_a_kind_is_a_mixture():
    from delta_b200.config.mufalix_config import MufalixConfig
    cfg = mh.config("only_experts")
    for L in cfg["layers"]:
        L["mlp"].pop("kind")
    got = MufalixConfig.from_dict(cfg)
    assert got.layers[0].mlp["router"]["experts"] == 7
