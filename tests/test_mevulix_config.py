"""Mevulix on the CPU: the configuration reader (sizes that only the tensors' shapes give among them), which cache every layer
reads, the specification's tensor list against the names the tests write out on their own, and properties of the plain
implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

import mevulix_helpers as mh
import plain_mevulix as plain

ALL = list(mh.PAGE_SIZE)
F = torch.float64


def build(which):
    import delta_b200.models  # noqa: F401
    from delta_b200.config.registry import architecture_of
    from delta_b200.models import Model
    cfg, W = mh.build(which, 1)
    arch = architecture_of(cfg)
    assert arch.name == "Mevulix"
    typed = arch.config_from_dict(arch.sizes_from_shapes(cfg, {k: tuple(v.shape) for k, v in W.items()}))
    return cfg, W, typed, Model(arch.build_spec(typed, None))


@pytest.mark.parametrize("which", ALL)
def test_tensor_list(which):
    cfg, W, typed, model = build(which)
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == {k: tuple(v.shape) for k, v in W.items()}


def test_which_cache_a_layer_reads():
    cfg, W, typed, model = build("mix")
    assert [(e.layer, e.cache, e.writes_cache) for e in model.order] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False), (4, 4, True)]
    assert sorted(model.cache_specs()) == [0, 1, 2, 4]
    assert not model.has_run_state()
    cfg, W, typed, model = build("only_shared_kv")
    assert [e.cache for e in model.order] == [0, 0, 0, 0] and sorted(model.cache_specs()) == [0]
    names = {s.name for s in model.tensor_specs()}
    assert "l1.mix.q" in names and not names & {"l1.mix.k", "l1.mix.v", "l1.mix.k.b", "l1.mix.v.b", "l1.mix.k.norm"}


def test_the_model_folder_gives_the_rows_of_the_bias_tables(tmp_path):
    from delta_b200.config.registry import read_config
    from delta_b200.config.model_config import ConfigError
    cfg, W = mh.build("mix", 2)
    folder = mh.write_folder(tmp_path, "m", cfg, W)
    arch, typed = read_config(folder)
    assert [L.mixer.get("bias_rows") for L in typed.layers] == [None, 12, None, 8, 20]
    with pytest.raises(ConfigError, match="bias_rows"):      # without a folder the configuration has to say it
        arch.config_from_dict(cfg)
    named = copy.deepcopy(cfg)
    named["layers"][1]["mixer"]["bias_rows"] = 12
    named["layers"][3]["mixer"]["bias_rows"] = 8
    named["layers"][4]["mixer"]["bias_rows"] = 20
    assert arch.config_from_dict(named) == typed


def test_config_errors():
    from delta_b200.config.model_config import ConfigError
    from delta_b200.config.mevulix_config import MevulixConfig, sizes_from_shapes
    cfg, W = mh.build("mix", 1)
    good = sizes_from_shapes(cfg, {k: tuple(v.shape) for k, v in W.items()})
    MevulixConfig.from_dict(good)
    for path, value, text in ((("layers", 1, "mixer", "kv_heads"), 3, "multiple"), (("layers", 1, "mlp", "router", "top"), 7, "top"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 10, "rot.dims"),
                              (("layers", 3, "mixer", "kv_from"), 0, "attention"), (("layers", 3, "mixer", "kv_from"), 3, "earlier"),
                              (("layers", 3, "mixer", "dim"), 16, "differ"), (("layers", 1, "mixer", "softcap"), 0.0, "cap"),
                              (("layers", 1, "mixer", "q_temp", "every"), 0, "every"), (("layers", 1, "mixer", "bias_max"), 5, "logarithmic"),
                              (("layers", 0, "type"), "mamba", "unknown mixer"), (("layers", 0, "mlp", "kind"), "glu", "feed-forward kind"),
                              (("layers", 0, "mixer", "q_rank"), None, "q_rank"), (("norm",), None, "norm"), (("vocab",), 0, "positive")):
        bad = copy.deepcopy(good)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            MevulixConfig.from_dict(bad)
    chain = copy.deepcopy(good)      # a layer cannot read the keys of a layer that has none of its own
    chain["layers"][4] = copy.deepcopy(chain["layers"][3])
    chain["layers"][4]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError, match="own"):
        MevulixConfig.from_dict(chain)


def test_optional_keys():
    """A model without cap, temperature, bias table, scaling, shared expert and logit scale is read and builds its parts without them."""
    from delta_b200.config.mevulix_config import MevulixConfig
    from delta_b200.models import Model
    from delta_b200.models.mevulix import mevulix_spec
    cfg = dict(architecture="Mevulix", norm=dict(eps=1e-5), vocab=50, width=32, layers=[
        dict(type="attention", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.3), mlp=dict(kind="moe", router=dict(experts=3, top=1), expert=dict(ff=8))),
        dict(type="latent_attention", mixer=dict(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=12, q_rank=8, scale=0.3, rot=dict(base=100.0, dims=4)), mlp=None)])
    typed = MevulixConfig.from_dict(cfg)
    model = Model(mevulix_spec(typed))
    names = {s.name for s in model.tensor_specs()}
    assert "l0.mix.rel" not in names and "l0.mlp.shared.gate" not in names and "l1.norm2" not in names and "l0.mix.o.b" not in names
    assert model.spec.logit_scale == 1.0
    att = model.blocks[0].mixer
    assert att.softcap is None and att.q_temp is None and att.distance_bias is None


def test_plain_pieces():
    """What the GPU tests lean on: the bucket rule's ends, the gelu form, the sink's share of the softmax, and the rotation's length."""
    assert [plain.distance_bucket(n, 8, 20) for n in (0, 3, 4, 5, 19, 20, 400)] == [0, 3, 4, 4, 7, 7, 7]
    assert plain.distance_bucket(4, 9, 20) == 4 and plain.distance_bucket(3, 9, 20) == 3      # an odd table: rows // 2 exact rows
    z = torch.linspace(-6, 6, 101, dtype=F)
    assert (plain.gelu_tanh(z) - z * torch.sigmoid(2.0 * math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))).abs().max().item() < 1e-12
    s = torch.zeros(1, 1, 3, dtype=F)
    w = plain.softmax_with_sink(s, torch.ones(1, 1, 3, dtype=torch.bool), torch.tensor([math.log(3.0)], dtype=F))
    assert (w - 1.0 / 6.0).abs().max().item() < 1e-12      # three keys of weight 1 and a sink of weight 3
    x = torch.randn(5, 2, 12, dtype=F)
    rot = dict(base=100.0, dims=8, scaling=dict(factor=4.0, original=16, fast=4.0, slow=1.0))
    y = plain.rotate_pairs(x, torch.arange(5), rot)
    mag = 0.1 * math.log(4.0) + 1.0
    assert torch.allclose(y[..., :8].pow(2).sum(-1), x[..., :8].pow(2).sum(-1) * mag * mag) and torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[0, :, :8], x[0, :, :8] * mag)      # position 0 turns nothing


def test_rounded_plain_run_stays_close():
    cfg, W = mh.build("mix", 3)
    toks = list(range(40))
    ref = plain.forward(cfg, W, toks)[0]
    with plain.rounding("bfloat16"):
        r = plain.forward(cfg, W, toks)[0]
    err = (r - ref).pow(2).mean().sqrt().item() / ref.pow(2).mean().sqrt().item()
    assert 1e-4 < err < 0.1
