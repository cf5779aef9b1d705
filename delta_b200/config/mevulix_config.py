"""Typed configuration of the Mevulix design, read from its config.json.

The file names the design in ``architecture`` and gives every size and every constant that may differ between
models of the design:

    vocab, width                         token interface and stream width
    norm.eps                             eps of every norm (layer norms, query/key norms, latent norms)
    logit_scale                          factor on the logits (absent: 1)
    layers[i] {type, mixer, mlp}         the mixer's kind and sizes; mlp or null

Mixer kinds and their keys:
    attention          heads, kv_heads, dim, vdim, scale, softcap (absent: none), q_temp {coef, every} (absent: none),
                       bias_max (absent: no bias by distance), bias_rows (the rows of the bias table ``rel``; absent: taken from the
                       tensor's shape in the model folder), kv_from (absent: the layer has keys and values of its own)
    latent_attention   heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                       rot {base, dims, scaling {factor, original, fast, slow} (absent: unscaled)} (needed when rot_dim > 0)
Feed-forward kinds (``kind``):
    dense       ff
    moe         router {experts, top}, expert {ff}, shared {ff} (absent: no shared expert)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"),
}
SCALING_KEYS = ("factor", "original", "fast", "slow")


@dataclass(frozen=True)
class MevulixLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


def bias_table_name(layer: int) -> str:
    return f"l{layer}.mix.rel"


def sizes_from_shapes(c: dict, shapes: dict) -> dict:
    """config.json with the sizes that only the tensors give filled in: the rows of every attention layer's bias table."""
    out = dict(c)
    layers = []
    for i, L in enumerate(c.get("layers") or []):
        m = L.get("mixer") if isinstance(L, dict) else None
        if isinstance(m, dict) and L.get("type") == "attention" and m.get("bias_max") is not None and m.get("bias_rows") is None:
            shape = shapes.get(bias_table_name(i))
            if shape is not None and len(shape) == 2:
                L = dict(L, mixer=dict(m, bias_rows=int(shape[0])))
        layers.append(L)
    out["layers"] = layers
    return out


@dataclass(frozen=True)
class MevulixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple
    logit_scale: float = 1.0

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(c: dict) -> "MevulixConfig":
        def need(d, key, where):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                raise ConfigError(f"config.json has no '{key}' in {where}")
            return d[key]

        raw_layers = need(c, "layers", "the model")
        if not raw_layers:
            raise ConfigError("config.json lists no layers")
        layers = []
        for i, L in enumerate(raw_layers):
            kind = need(L, "type", f"layer {i}")
            if kind not in MIXER_KEYS:
                raise ConfigError(f"layer {i}: unknown mixer type '{kind}'; known: {', '.join(MIXER_KEYS)}")
            m = dict(need(L, "mixer", f"layer {i}"))
            for k in MIXER_KEYS[kind]:
                need(m, k, f"the mixer of layer {i}")
            if kind == "attention":
                if m.get("q_temp"):
                    need(m["q_temp"], "coef", f"q_temp of layer {i}")
                    need(m["q_temp"], "every", f"q_temp of layer {i}")
                if m.get("bias_max") is not None:
                    need(m, "bias_rows", f"the mixer of layer {i} (nor is there a tensor '{bias_table_name(i)}' to take it from)")
            else:
                if m["rot_dim"]:
                    rot = need(m, "rot", f"the mixer of layer {i}")
                    need(rot, "base", f"rot of layer {i}")
                    need(rot, "dims", f"rot of layer {i}")
                    if rot.get("scaling"):
                        for k in SCALING_KEYS:
                            need(rot["scaling"], k, f"rot.scaling of layer {i}")
            mlp = L.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                mk = need(mlp, "kind", f"mlp of layer {i}")
                if mk == "dense":
                    need(mlp, "ff", f"mlp of layer {i}")
                elif mk == "moe":
                    r = need(mlp, "router", f"mlp of layer {i}")
                    need(r, "experts", f"router of layer {i}")
                    need(r, "top", f"router of layer {i}")
                    need(need(mlp, "expert", f"mlp of layer {i}"), "ff", f"expert of layer {i}")
                    if mlp.get("shared"):
                        need(mlp["shared"], "ff", f"shared expert of layer {i}")
                else:
                    raise ConfigError(f"layer {i}: unknown feed-forward kind '{mk}' (dense, moe)")
            layers.append(MevulixLayer(kind, m, mlp))
        cfg = MevulixConfig(
            architecture=str(c.get("architecture") or (c.get("architectures") or ["Mevulix"])[0]),
            vocab=int(need(c, "vocab", "the model")), width=int(need(c, "width", "the model")),
            eps=float(need(need(c, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
            logit_scale=float(c["logit_scale"]) if c.get("logit_scale") is not None else 1.0)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type == "attention":
                if min(m["heads"], m["kv_heads"], m["dim"], m["vdim"]) < 1:
                    raise ConfigError(f"layer {i}: heads, kv_heads, dim and vdim must be positive")
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"layer {i}: {m['heads']} heads are no multiple of {m['kv_heads']} key-value heads")
                if m.get("softcap") is not None and float(m["softcap"]) <= 0:
                    raise ConfigError(f"layer {i}: a score cap of {m['softcap']}")
                if m.get("q_temp") and int(m["q_temp"]["every"]) < 1:
                    raise ConfigError(f"layer {i}: q_temp.every {m['q_temp']['every']} must be at least 1")
                if m.get("bias_max") is not None:
                    rows = int(m["bias_rows"])
                    if rows < 2 or float(m["bias_max"]) <= rows // 2:
                        raise ConfigError(f"layer {i}: a bias table of {rows} rows up to distance {m['bias_max']} has no logarithmic half")
                src = m.get("kv_from")
                if src is not None:
                    if not (0 <= int(src) < i) or self.layers[int(src)].type != "attention":
                        raise ConfigError(f"layer {i}: kv_from {src} names no earlier attention layer")
                    o = self.layers[int(src)].mixer
                    if o.get("kv_from") is not None:
                        raise ConfigError(f"layer {i}: kv_from {src} names a layer that has no keys and values of its own")
                    if any(o[k] != m[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"layer {i}: kv_heads, dim and vdim differ from layer {src}'s, whose keys and values it reads")
            else:
                if min(m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]) < 1 or m["rot_dim"] < 0:
                    raise ConfigError(f"layer {i}: heads, dim, vdim, kv_rank and q_rank must be positive")
                if m["rot_dim"]:
                    dims = int(m["rot"]["dims"])
                    if dims % 2 or dims > m["rot_dim"] or dims < 2:
                        raise ConfigError(f"layer {i}: rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
            if L.mlp and L.mlp["kind"] == "moe" and not (1 <= L.mlp["router"]["top"] <= L.mlp["router"]["experts"]):
                raise ConfigError(f"layer {i}: top {L.mlp['router']['top']} of {L.mlp['router']['experts']} experts")

    def cache_of(self, layer: int) -> int:
        """The layer whose run fills the cache that ``layer`` reads: itself, or the one ``kv_from`` names."""
        src = self.layers[layer].mixer.get("kv_from") if self.layers[layer].type == "attention" else None
        return layer if src is None else int(src)
