"""Mevulix as a ``ModelSpec``: a decoder whose config.json lists its layers.  The norms sit on the sublayers' outputs and the
sublayers read the 32-bit residual stream itself,

    x <- x + s1 * layer_norm1(mixer(x)),    x <- x + s2 * layer_norm2(feed_forward(x))        (the second half may be absent)

with layer norms that have a weight and a bias and a scale per column s behind them.  The mixers:

  * ``attention``: grouped-query attention with biases on q, k and v, an RMS norm over all of q's columns at once (and over all of
    k's), no rotation, a query temperature that grows with the position, capped scores, a learned bias by distance in logarithmic
    buckets and a learned sink in the softmax (``parts/row_attention.py``); a layer may read the keys and values that an earlier
    attention layer cached (``kv_from``) instead of making its own;
  * ``latent_attention``: queries, keys and values through small latents, a short rotated key part that all heads share, rotary
    positions with the ramp rule for long contexts (``parts/latent_attention.py``, ``parts/rope.py``).

The feed-forward is a dense gated one with the tanh form of gelu, or a mixture of silu-gated experts with sigmoid scores whose
weights multiply what an expert reads, beside a shared expert.  The logits are scaled.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``); layer i: ``l<i>.norm1|norm2`` (+ ``.b``), ``l<i>.ls1|ls2``,
``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from typing import Optional

from ..config.engine_config import EngineConfig
from ..config.mevulix_config import MevulixConfig
from ..parts.base import PartSpec, TensorSpec
from ..parts.feed_forward import GELU_TANH_GATE, SILU_GATE
from .spec import LayerSpec, ModelSpec, RunEntry


def _mixer(cfg: MevulixConfig, i: int, max_pos: int) -> PartSpec:
    L = cfg.layers[i]
    m, pre, d = L.mixer, f"l{i}.mix.", cfg.width
    if L.type == "attention":
        bias = dict(rows=m["bias_rows"], far=m["bias_max"]) if m.get("bias_max") is not None else None
        return PartSpec("sink_attention", dict(
            prefix=pre, width=d, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"], scale=m["scale"],
            sink=True, bias=True, out_bias=False, qk_norm_eps=cfg.eps, qk_norm_whole=True, q_temp=m.get("q_temp") or None,
            softcap=m.get("softcap"), distance_bias=bias, shared_kv=m.get("kv_from") is not None), "mixer")
    position = None
    if m["rot_dim"]:
        rot = m["rot"]
        position = PartSpec("rotary", dict(head_dim=rot["dims"], theta=rot["base"], max_positions=max_pos, interleaved=True,
                                           scaling=rot.get("scaling") or None), "position")
    return PartSpec("latent_attention", dict(prefix=pre, width=d, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                                             value_dim=m["vdim"], kv_rank=m["kv_rank"], q_rank=m["q_rank"], eps=cfg.eps, scale=m["scale"],
                                             position=position, rot_dims=m["rot"]["dims"] if m["rot_dim"] else None), "mixer")


def _feed_forward(cfg: MevulixConfig, i: int) -> Optional[PartSpec]:
    mlp, pre, d = cfg.layers[i].mlp, f"l{i}.mlp.", cfg.width
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("clamped_glu", dict(prefix=pre, width=d, intermediate=mlp["ff"], limit=None, **GELU_TANH_GATE), "feed_forward")
    r = mlp["router"]
    shared = dict(intermediate=mlp["shared"]["ff"], limit=None, gate=False, alpha=SILU_GATE["alpha"], shift=SILU_GATE["shift"]) if mlp.get("shared") else None
    return PartSpec("experts", dict(prefix=pre, width=d, experts=r["experts"], top=r["top"], intermediate=mlp["expert"]["ff"],
                                    limit=None, alpha=SILU_GATE["alpha"], shift=SILU_GATE["shift"], shared=shared, scoring="sigmoid",
                                    normalize=False, weight_input=True), "feed_forward")


def mevulix_spec(cfg: MevulixConfig, engine: Optional[EngineConfig] = None) -> ModelSpec:
    engine = engine or EngineConfig()
    d = cfg.width

    def norm(name, scale=None):
        return PartSpec("layer_norm", dict(name=name, width=d, eps=cfg.eps, bias=True, scale=scale), "norm")

    layers = []
    for i in range(len(cfg.layers)):
        parts = dict(norm1=norm(f"l{i}.norm1", f"l{i}.ls1"), mixer=_mixer(cfg, i, engine.max_seq_len))
        ff = _feed_forward(cfg, i)
        if ff is not None:
            parts["norm2"] = norm(f"l{i}.norm2", f"l{i}.ls2")
            parts["feed_forward"] = ff
        layers.append(LayerSpec(parts, block="sublayer_norm"))
    order = tuple(RunEntry(i, cache=cfg.cache_of(i), writes_cache=cfg.cache_of(i) == i) for i in range(len(cfg.layers)))
    return ModelSpec(
        vocab_size=cfg.vocab, width=d, layers=tuple(layers), order=order, final_norm=norm("final.norm"),
        embedding=TensorSpec("embed", (cfg.vocab, d), kind="table"), lm_head=TensorSpec("head", (cfg.vocab, d), kind="matrix"),
        max_positions=engine.max_seq_len, stream=PartSpec("residual_f32", dict(width=d, rounded_start=True), "stream"), logit_scale=cfg.logit_scale)
