"""Mufalix as a ``ModelSpec``: a decoder whose config.json lists its layers.  Every layer is a pre-norm block on a 32-bit
residual stream, x <- x + mixer(rms_norm(x)), x <- x + experts(rms_norm(x)) (the second half may be absent), with one of two
mixers:

  * ``mlstm``: a matrix memory per head with exponential gates (``parts/matrix_memory.py``);
  * ``parallel``: two mixers side by side (``parts/side_by_side.py``), each output RMS-normed over the width, half their sum:
    grouped-query attention over a sliding window with biases, a weighted RMS norm of query and key heads, partly rotated
    heads with scaled frequencies, a learned sink in the softmax and an output gate (``parts/row_attention.py``); and a
    recurrent block with a gated diagonal linear recurrence behind a short convolution (``parts/gated_recurrence.py``).

The feed-forward is a mixture of experts with sigmoid scores, a correction that enters the choice only, and experts of one
branch through relu(.)^2.  The token embedding is scaled; a span of layers may run several times with the same weights,
every run with a cache and state of its own, and before every pass (the first too) the stream and the embedding output go
through one projection together.

Tensor names: ``embed``, ``loop.in``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from typing import Optional

from ..config.engine_config import EngineConfig
from ..config.mufalix_config import MufalixConfig
from ..parts.base import PartSpec, TensorSpec
from .spec import LayerSpec, ModelSpec, RunEntry

DECAY_SCALE = 8.0       # the recurrence's decay is exp(-8 r softplus(lam))
MEMORY_GUARD = 1e-6     # added to the matrix memory's denominator
MIX_FACTOR = 0.5        # the two mixers side by side are averaged


def _mixer(cfg: MufalixConfig, i: int, max_pos: int) -> PartSpec:
    L = cfg.layers[i]
    m, pre, d = L.mixer, f"l{i}.mix.", cfg.width
    if L.type == "mlstm":
        return PartSpec("matrix_memory", dict(prefix=pre, width=d, heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"],
                                              gate_cap=m["gate_cap"], eps=cfg.eps, guard=MEMORY_GUARD, wide_output=True), "mixer")
    a, r = m["left"], m["right"]
    rot = a.get("rot") or None
    position = None
    if rot and rot["dims"]:
        position = PartSpec("rotary", dict(head_dim=rot["dims"], theta=rot["base"], max_positions=max_pos, interleaved=False,
                                           scaling=rot.get("scaling") or None), "position")
    left = PartSpec("sink_attention", dict(prefix=pre + "left.", width=d, heads=a["heads"], kv_heads=a["kv_heads"], head_dim=a["dim"],
                                           value_dim=a["vdim"], scale=a["scale"], window=(a.get("mask") or {}).get("size"),
                                           sink=True, position=position, rot_dims=rot["dims"] if position is not None else None,
                                           bias=True, qk_norm_eps=cfg.eps, gate=True), "mixer")
    right = PartSpec("gated_recurrence", dict(prefix=pre + "right.", width=d, channels=r["width"], conv=r["conv"], blocks=r["blocks"],
                                              decay_scale=DECAY_SCALE), "mixer")
    return PartSpec("side_by_side", dict(prefix=pre, width=d, left=left, right=right, eps=cfg.eps, factor=MIX_FACTOR), "mixer")


def _feed_forward(cfg: MufalixConfig, i: int) -> Optional[PartSpec]:
    mlp, pre, d = cfg.layers[i].mlp, f"l{i}.mlp.", cfg.width
    if mlp is None:
        return None
    r = mlp["router"]
    return PartSpec("experts", dict(prefix=pre, width=d, experts=r["experts"], top=r["top"], intermediate=mlp["expert"]["ff"],
                                    scoring="sigmoid", correction=True, route_scale=float(r.get("scale", 1.0)),
                                    activation="relu_squared", wide_output=True), "feed_forward")


def mufalix_spec(cfg: MufalixConfig, engine: Optional[EngineConfig] = None) -> ModelSpec:
    engine = engine or EngineConfig()
    d = cfg.width
    norm = lambda name: PartSpec("rms_norm", dict(name=name, width=d, eps=cfg.eps), "norm")     # noqa: E731
    layers = []
    for i in range(len(cfg.layers)):
        parts = dict(norm1=norm(f"l{i}.norm1"), mixer=_mixer(cfg, i, engine.max_seq_len))
        ff = _feed_forward(cfg, i)
        if ff is not None:
            parts["norm2"] = norm(f"l{i}.norm2")
            parts["feed_forward"] = ff
        layers.append(LayerSpec(parts, block="residual_pre_norm"))
    reentry = dict(project="loop.in", passes=cfg.loop["times"]) if cfg.loop else None
    return ModelSpec(
        vocab_size=cfg.vocab, width=d, layers=tuple(layers),
        order=tuple(RunEntry(i, enters_pass=t) for i, t in cfg.run_order()),
        final_norm=norm("final.norm"),
        embedding=TensorSpec("embed", (cfg.vocab, d), kind="table"), lm_head=TensorSpec("head", (cfg.vocab, d), kind="matrix"),
        max_positions=engine.max_seq_len,
        stream=PartSpec("residual_f32", dict(width=d, scale=cfg.embed_scale, reentry=reentry), "stream"))
