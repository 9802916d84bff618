"""Roritar: a decoder whose layers are listed one by one in config.json and of which a stretch
may run several times in a row with the same weights (every pass with a cache entry or state
of its own).  A layer normalises before AND after each sublayer,

    x += norm1b(mixer(norm1(x)));   x += norm2b(feed_forward(norm2(x)))

with layer norms that have a weight and no bias.  The mixer is softmax attention over a
sliding window plus one mean key and value for every block of positions wholly behind the
window (per-head RMS norms of queries and keys, rotary positions on part of each head, values
rotated by their position and the output turned back), or a recurrent block around a
real-gated linear recurrent unit (two branches, a short causal convolution, block-diagonal
gates, a float32 state per request).  The feed-forward is dense with the xIELU activation, or
absent.  The head is the token table; its logits are scaled and capped by a tanh.

config.json::

    {"architecture": "Roritar", "vocab": V, "width": W, "norm": {"eps": e},
     "logit_scale": s, "logit_softcap": c,
     "loop": {"start": a, "stop": b, "times": n}   (optional: layers a .. b-1 run n times),
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                           "mask": {"size", "pool"}, "rot": {"base", "dims"}},
                 "mlp": {"kind": "dense", "ff"} | null},
                {"type": "rglru", "mixer": {"width", "blocks", "conv"}, "mlp": ...}, ...]}

Tensors: ``embed``; per layer ``l<i>.norm1``, ``norm1b`` (and ``norm2``, ``norm2b`` with a
feed-forward), ``l<i>.mix.{q, k, v, q.norm, k.norm, o}`` or ``l<i>.mix.{y, y.b, x, x.b, conv,
conv.b, ra, ra.b, ri, ri.b, lam, o}``, ``l<i>.mlp.{up, down, act}``; ``final.norm``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Any, Mapping

import torch

from ..config.model_config import (Architecture, ConfigError, need, positive_int,
                                   register_architecture)
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

LAYER_TYPES = ("attention", "rglru")
# log a = -DECAY_SCALE * r * softplus(lam): fixed by the design
DECAY_SCALE = 8.0


def _number(name: str, v: Any, positive: bool = False) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{name} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _section(raw: Mapping, key: str, where: str) -> Mapping:
    v = raw.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where} needs an object {key!r}")
    return v


def _check_layer(i: int, layer) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, Mapping) or layer.get("type") not in LAYER_TYPES:
        raise ConfigError(f"{where}.type must be one of {LAYER_TYPES}")
    m = _section(layer, "mixer", where)
    wm = where + ".mixer"
    if layer["type"] == "attention":
        for key in ("heads", "kv_heads", "dim", "vdim"):
            positive_int(f"{wm}.{key}", need(m, key))
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{wm}.heads is not a multiple of kv_heads")
        if m["vdim"] % 2:
            raise ConfigError(f"{wm}.vdim must be even: the values are rotated in pairs")
        _number(f"{wm}.scale", need(m, "scale"))
        mask = _section(m, "mask", wm)
        positive_int(f"{wm}.mask.size", need(mask, "size"))
        positive_int(f"{wm}.mask.pool", need(mask, "pool"))
        rot = _section(m, "rot", wm)
        _number(f"{wm}.rot.base", need(rot, "base"), positive=True)
        dims = need(rot, "dims")
        if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 \
                or dims > m["dim"]:
            raise ConfigError(f"{wm}.rot.dims must be an even number up to dim, got {dims!r}")
    else:
        for key in ("width", "blocks", "conv"):
            positive_int(f"{wm}.{key}", need(m, key))
        if m["width"] % m["blocks"]:
            raise ConfigError(f"{wm}.width is not a multiple of blocks")
    mlp = layer.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
            raise ConfigError(f"{where}.mlp must be null or an object of kind 'dense'")
        positive_int(f"{where}.mlp.ff", need(mlp, "ff"))


@dataclass(frozen=True)
class RoritarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    logit_softcap: float            # 0: the logits are not capped
    loop: tuple | None              # (start, stop, times)
    layers: tuple                   # the layer entries of config.json, as they stand
    architectures: tuple[str, ...] = ("Roritar",)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RoritarConfig":
        vocab = positive_int("vocab", need(raw, "vocab"))
        width = positive_int("width", need(raw, "width"))
        eps = _number("norm.eps", need(_section(raw, "norm", "config.json"), "eps"), positive=True)
        scale = _number("logit_scale", raw.get("logit_scale", 1.0))
        cap = raw.get("logit_softcap")
        cap = 0.0 if cap is None else _number("logit_softcap", cap)
        if cap < 0:
            raise ConfigError("logit_softcap is not negative")
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("'loop' must be an object with start, stop and times")
            a, b, n = (need(loop, "start"), need(loop, "stop"),
                       positive_int("loop.times", need(loop, "times")))
            if not all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b)) \
                    or not 0 <= a <= b <= len(layers):
                raise ConfigError(f"loop: start..stop must lie inside the {len(layers)} layers")
            loop = (a, b, n)
        return cls(vocab, width, eps, scale, cap, loop, tuple(copy.deepcopy(list(layers))))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": "Roritar", "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
               "logit_softcap": self.logit_softcap or None,
               "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return out

    def layer_runs(self) -> list[int]:
        """The layers in the order they run: the looped stretch is repeated."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def num_parameters(self) -> int:
        return sum(math.prod(t.shape) for t in init_weights(self, 0, shapes_only=True).values())


def _norm_spec(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec("layernorm", dict(width=width, eps=eps, weight=name, bias=None))


def build_spec(cfg: RoritarConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            mixer = PartSpec("pooled_window_attention", dict(
                width=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                value_dim=m["vdim"], scale=m["scale"], window=m["mask"]["size"],
                pool=m["mask"]["pool"], rot_base=m["rot"]["base"], rot_dims=m["rot"]["dims"],
                rotate_values=True, qk_norm=True, eps=eps, prefix=p + "mix."))
        else:
            mixer = PartSpec("rglru", dict(
                width=W, channels=m["width"], blocks=m["blocks"], taps=m["conv"],
                decay_scale=DECAY_SCALE, prefix=p + "mix."))
        parts = dict(norm1=_norm_spec(p + "norm1", W, eps), mixer=mixer,
                     norm1b=_norm_spec(p + "norm1b", W, eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            parts.update(
                norm2=_norm_spec(p + "norm2", W, eps), norm2b=_norm_spec(p + "norm2b", W, eps),
                feed_forward=PartSpec("dense", dict(
                    width=W, inner=mlp["ff"], activation="xielu", act_params=p + "mlp.act",
                    in_weight=p + "mlp.up", in_bias=None, out_weight=p + "mlp.down",
                    out_bias=None, stored_in_out=False)))
        layers.append(LayerSpec("sandwich_norm", parts))
    # every run of a layer has a cache entry (or state) of its own: the schedule names the
    # layers of the looped stretch once per pass
    schedule = tuple(LayerCall(i) for i in cfg.layer_runs())
    return ModelSpec(
        name="Roritar", vocab_size=cfg.vocab, width=W, max_positions=None,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=W, table="embed")),
        position=PartSpec("none", {}),
        layers=tuple(layers), schedule=schedule,
        final_norm=_norm_spec("final.norm", W, eps),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=W, weight="embed",
                                     scale=cfg.logit_scale, softcap=cfg.logit_softcap)),
        eos_token_id=None)


def init_weights(cfg: RoritarConfig, seed: int, shapes_only: bool = False):
    """Seeded random float32 weights under the checkpoint's names, drawn from one CPU generator
    in the order the names are listed here.  Matrices ~ N(0, 1/sqrt(in)); norm weights near 1;
    biases and the recurrence's parameters spread enough that leaving one out changes the
    logits."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    w: dict[str, torch.Tensor] = {}

    def put(name, shape, std=None, mean=0.0):
        if shapes_only:
            w[name] = torch.empty(shape, device="meta")
            return
        if std is None:
            std = 1.0 / math.sqrt(shape[-1])
        w[name] = torch.randn(shape, generator=gen, dtype=torch.float32) * std + mean

    W = cfg.width
    put("embed", (cfg.vocab, W), 0.5)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        put(p + "norm1", (W,), 0.1, 1.0)
        put(p + "norm1b", (W,), 0.1, 1.0)
        a = p + "mix."
        if layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            put(a + "q", (H * D, W), 2.0 / math.sqrt(W)); put(a + "k", (G * D, W), 2.0 / math.sqrt(W))
            put(a + "v", (G * V, W))
            put(a + "q.norm", (D,), 0.2, 1.5); put(a + "k.norm", (D,), 0.2, 1.5)
            put(a + "o", (W, H * V))
        else:
            C, B, taps = m["width"], m["blocks"], m["conv"]
            put(a + "y", (C, W)); put(a + "y.b", (C,), 0.3)
            put(a + "x", (C, W)); put(a + "x.b", (C,), 0.3)
            put(a + "conv", (C, taps), 0.5); put(a + "conv.b", (C,), 0.2)
            put(a + "ra", (B, C // B, C // B)); put(a + "ra.b", (B, C // B), 0.5)
            put(a + "ri", (B, C // B, C // B)); put(a + "ri.b", (B, C // B), 0.5)
            put(a + "lam", (C,), 1.0, -2.5)
            put(a + "o", (W, C))
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        put(p + "norm2", (W,), 0.1, 1.0)
        put(p + "norm2b", (W,), 0.1, 1.0)
        put(p + "mlp.up", (mlp["ff"], W), 1.5 / math.sqrt(W))
        put(p + "mlp.down", (W, mlp["ff"]))
        put(p + "mlp.act", (2,), 0.5, 0.3)
    put("final.norm", (W,), 0.1, 1.0)
    return w


def _attention(heads, kv_heads, dim, vdim, window, pool, rot_dims=None, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
            "mask": {"size": window, "pool": pool},
            "rot": {"base": base, "dims": dim // 2 if rot_dims is None else rot_dims}}


def _layers(n, attention, recurrent, ff):
    """n layers: two recurrent ones after every attention layer."""
    out = []
    for i in range(n):
        kind = "attention" if i % 3 == 0 else "rglru"
        out.append({"type": kind, "mixer": copy.deepcopy(attention if kind == "attention"
                                                         else recurrent),
                    "mlp": {"kind": "dense", "ff": ff}})
    return out


def _preset(vocab, width, layers, loop=None, eps=1e-6, logit_scale=1.0, softcap=30.0):
    out = {"architecture": "Roritar", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "logit_scale": logit_scale, "logit_softcap": softcap, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


PRESETS: dict[str, dict] = {
    # a few hundred thousand parameters: for demonstrations and smoke runs
    "roritar-tiny": _preset(384, 96, [
        {"type": "attention", "mixer": _attention(4, 2, 24, 16, 40, 4), "mlp": {"kind": "dense", "ff": 160}},
        {"type": "rglru", "mixer": {"width": 64, "blocks": 2, "conv": 4}, "mlp": {"kind": "dense", "ff": 160}},
        {"type": "attention", "mixer": _attention(4, 2, 24, 16, 40, 4), "mlp": None},
    ], loop=(1, 3, 2), logit_scale=0.5),
    # layer sizes of a small and a mid-sized production model, few layers: for measurements
    "roritar-1k": _preset(32768, 1024, _layers(
        6, _attention(16, 4, 64, 64, 256, 16), {"width": 1024, "blocks": 16, "conv": 4}, 4096)),
    "roritar-2k": _preset(32768, 2048, _layers(
        6, _attention(32, 8, 64, 64, 256, 16), {"width": 2048, "blocks": 16, "conv": 4}, 8192)),
}

RORITAR = Architecture(name="Roritar", config_cls=RoritarConfig, build_spec=build_spec,
                       init_weights=init_weights, model_types=("roritar",), presets=PRESETS,
                       preset_aliases={})
register_architecture(RORITAR, replace=True)
