"""Typed configuration of the Mufalix design, read from its config.json.

The file names the design in ``architecture`` and gives every size and every constant that may differ between
models of the design:

    vocab, width                         token interface and stream width
    norm.eps                             eps of every RMS norm (layer norms, query/key norms, head norms, the side-by-side outputs)
    embedding.scale                      factor on the token embedding (absent: 1)
    loop {start, stop, times}            layers start..stop-1 run ``times`` times in a row with the same weights; before every pass
                                         the stream is projected together with the embedding output (absent: no such span)
    layers[i] {type, mixer, mlp}         the mixer's kind and sizes; mlp or null

Mixer kinds and their keys:
    mlstm       heads, dim, vdim, gate_cap
    parallel    left  {heads, kv_heads, dim, vdim, scale, mask {size} (absent: every earlier token is seen),
                       rot {base, dims, scaling {factor, low, high, original} (absent: unscaled)} (absent: no rotation)}
                right {width, conv, blocks}
Feed-forward kinds (``kind``; absent: moe):
    moe         router {experts, top, scale (absent: 1)}, expert {ff}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

MIXER_KEYS = {
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
    "parallel": ("left", "right"),
}
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
RIGHT_KEYS = ("width", "conv", "blocks")
SCALING_KEYS = ("factor", "low", "high", "original")


@dataclass(frozen=True)
class MufalixLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class MufalixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: tuple
    embed_scale: float = 1.0
    loop: Optional[dict] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @staticmethod
    def from_dict(c: dict) -> "MufalixConfig":
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
            if kind == "parallel":
                for k in LEFT_KEYS:
                    need(m["left"], k, f"the left mixer of layer {i}")
                for k in RIGHT_KEYS:
                    need(m["right"], k, f"the right mixer of layer {i}")
                rot = m["left"].get("rot")
                if rot:
                    need(rot, "base", f"rot of layer {i}")
                    need(rot, "dims", f"rot of layer {i}")
                    if rot.get("scaling"):
                        for k in SCALING_KEYS:
                            need(rot["scaling"], k, f"rot.scaling of layer {i}")
                if m["left"].get("mask"):
                    need(m["left"]["mask"], "size", f"mask of layer {i}")
            mlp = L.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                mk = mlp.get("kind") or "moe"      # the design has one kind of feed-forward
                if mk != "moe":
                    raise ConfigError(f"layer {i}: unknown feed-forward kind '{mk}' (moe)")
                r = need(mlp, "router", f"mlp of layer {i}")
                need(r, "experts", f"router of layer {i}")
                need(r, "top", f"router of layer {i}")
                need(need(mlp, "expert", f"mlp of layer {i}"), "ff", f"expert of layer {i}")
            layers.append(MufalixLayer(kind, m, mlp))
        emb = c.get("embedding") or {}
        loop = c.get("loop")
        if loop:
            loop = dict(start=int(need(loop, "start", "loop")), stop=int(need(loop, "stop", "loop")), times=int(need(loop, "times", "loop")))
        cfg = MufalixConfig(
            architecture=str(c.get("architecture") or (c.get("architectures") or ["Mufalix"])[0]),
            vocab=int(need(c, "vocab", "the model")), width=int(need(c, "width", "the model")),
            eps=float(need(need(c, "norm", "the model"), "eps", "norm")), layers=tuple(layers),
            embed_scale=float(emb.get("scale", 1.0)), loop=loop or None)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        n = len(self.layers)
        if self.loop:
            a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= n) or t < 1:
                raise ConfigError(f"loop {a}..{b} x {t} does not fit {n} layers")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type == "mlstm":
                if min(m["heads"], m["dim"], m["vdim"]) < 1 or float(m["gate_cap"]) <= 0:
                    raise ConfigError(f"layer {i}: heads, dim, vdim and gate_cap must be positive")
            else:
                a, r = m["left"], m["right"]
                if a["heads"] % a["kv_heads"]:
                    raise ConfigError(f"layer {i}: {a['heads']} heads are no multiple of {a['kv_heads']} key-value heads")
                rot = a.get("rot")
                if rot and (rot["dims"] % 2 or rot["dims"] > a["dim"]):
                    raise ConfigError(f"layer {i}: rot.dims {rot['dims']} must be even and at most dim {a['dim']}")
                if a.get("mask") and int(a["mask"]["size"]) < 1:
                    raise ConfigError(f"layer {i}: a window of {a['mask']['size']} tokens sees nothing")
                if r["blocks"] < 1 or r["width"] % r["blocks"]:
                    raise ConfigError(f"layer {i}: {r['width']} channels do not split into {r['blocks']} equal parts")
                if r["conv"] < 1:
                    raise ConfigError(f"layer {i}: the convolution needs at least one tap")
            if L.mlp and not (1 <= L.mlp["router"]["top"] <= L.mlp["router"]["experts"]):
                raise ConfigError(f"layer {i}: top {L.mlp['router']['top']} of {L.mlp['router']['experts']} experts")

    def run_order(self) -> list:
        """[(layer, number of the pass this run starts, or None)] in the order the layers run."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, None) for i in range(a)]
        for t in range(times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]
