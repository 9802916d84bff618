"""Mafuzen: a decoder whose layers are listed one by one in config.json.  The token table is
scaled at the input and is also the head.  Every layer normalises before AND behind each
sublayer with layer norms that have a weight and a bias,

    x += norm1b(mixer(norm1(x)));   x += norm2b(feed_forward(norm2(x)));   x += side(x)

and ends with a per-layer token input (``token_side``): a narrow second embedding of the token
id gates a projection of the stream, whose RMS norm is added.  The mixer is one of

``retention``  linear attention with a fixed decay per head on a float32 state per request,
               rotary positions on q and k (number i pairs with i + dims/2), keys scaled by
               dim^(-1/2), a unit-RMS norm per head and a silu gate;
``attention``  grouped softmax attention whose scores lose slope_h * distance, with slope_h =
               2^(-8 (h+1) / heads); ``kv_from: j`` makes a layer read layer j's keys and values
               with queries of its own;
``parallel``   softmax attention over a window that keeps the first tokens (unit-RMS queries and
               keys, the keys as projected are the values, a sigmoid gate on the output) beside
               time mixing with a decay per token and key channel (a float32 state per request
               and the previous token's input); ``left_scale * left + right_scale * right``.

The feed-forward is dense (``W_down (silu(W_gate h) * W_up h)``), a mixture of squared-ReLU
experts chosen by a table of the token id (each of ``top`` weighing 1/top) with an optional
shared expert of the same form, or absent.  The model's layer norm and the token table follow.

config.json::

    {"architecture": "Mafuzen", "vocab": V, "width": W, "embedding": {"scale": s},
     "norm": {"eps": e}, "token_side": {"dim": d} (optional),
     "layers": [{"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [one per head],
                                                 "rot": {"base", "dims"}}, "mlp": ...},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                                                 "kv_from": j (optional)}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim",
                                                         "scale", "mask": {"size", "keep_first"}},
                                               "right": {"heads", "dim"},
                                               "left_scale", "right_scale"}, "mlp": ...}]}
    mlp: {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"},
                                    "shared": {"ff"} (optional)} | null

Tensors: ``embed``, ``side.embed`` [vocab, layers * d]; per layer ``l<i>.norm1|norm1b|norm2|
norm2b`` with ``.b``, ``l<i>.mix.{q, k, v, g, o}`` (retention), ``l<i>.mix.{q, k, v, o}``
(attention; without ``k`` and ``v`` under ``kv_from``), ``l<i>.mix.left.{q, k, g, o}`` and
``l<i>.mix.right.{mu.r, mu.k, mu.v, mu.g, mu.w, r, k, v, g, w1, w2, w0, u, norm, o}`` (parallel),
``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{table, e<k>.{up, down}, shared.{up, down}}``,
``l<i>.side.{gate, proj, norm}``; ``final.norm`` with ``.b``.  The inner size of the decay's two
matrices is read off ``w1``.
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

LAYER_TYPES = ("retention", "attention", "parallel")
SLOPE_RANGE = 8.0            # slope_h = 2^(-SLOPE_RANGE * (h + 1) / heads)


def distance_slopes(heads: int) -> tuple:
    return tuple(2.0 ** (-SLOPE_RANGE * (h + 1) / heads) for h in range(heads))


def _number(name: str, v: Any, positive: bool = False) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"{name} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _count(name: str, v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"{name} must be a whole number, not negative, got {v!r}")
    return v


def _section(raw: Mapping, key: str, where: str) -> Mapping:
    v = raw.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where} needs an object {key!r}")
    return v


def _decays(m: Mapping, where: str) -> list:
    decay = need(m, "decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        return [decay] * m["heads"]
    if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"]:
        raise ConfigError(f"{where}.decay must list one decay per head")
    return list(decay)


def _check_heads(m: Mapping, where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        positive_int(f"{where}.{key}", need(m, key))
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{where}.heads is not a multiple of kv_heads")
    _number(f"{where}.scale", need(m, "scale"))


def _check_mlp(i: int, mlp) -> None:
    if mlp is None:
        return
    where = f"layers[{i}].mlp"
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{where} must be null or an object of kind 'dense' or 'moe'")
    if mlp["kind"] == "dense":
        positive_int(f"{where}.ff", need(mlp, "ff"))
        return
    positive_int(f"{where}.expert.ff", need(_section(mlp, "expert", where), "ff"))
    ro = _section(mlp, "router", where)
    E = positive_int(f"{where}.router.experts", need(ro, "experts"))
    top = positive_int(f"{where}.router.top", need(ro, "top"))
    if top > E:
        raise ConfigError(f"{where}.router: {top} chosen experts do not fit into {E}")
    if mlp.get("shared") is not None:
        positive_int(f"{where}.shared.ff", need(_section(mlp, "shared", where), "ff"))


def _check_layer(i: int, layer, layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, Mapping) or layer.get("type") not in LAYER_TYPES:
        raise ConfigError(f"{where}.type must be one of {LAYER_TYPES}")
    m = _section(layer, "mixer", where)
    wm = where + ".mixer"
    if layer["type"] == "retention":
        for key in ("heads", "dim", "vdim"):
            positive_int(f"{wm}.{key}", need(m, key))
        for d in _decays(m, wm):
            _number(f"{wm}.decay[]", d)
        rot = m.get("rot")
        if rot is not None:
            rot = _section(m, "rot", wm)
            _number(f"{wm}.rot.base", need(rot, "base"), positive=True)
            dims = _count(f"{wm}.rot.dims", need(rot, "dims"))
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"{wm}.rot.dims must be an even number up to dim, got {dims}")
    elif layer["type"] == "attention":
        _check_heads(m, wm)
        src = m.get("kv_from")
        if src is not None:
            ok = (isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
                  and isinstance(layers[src], Mapping) and layers[src].get("type") == "attention"
                  and layers[src]["mixer"].get("kv_from") is None
                  and all(layers[src]["mixer"].get(k) == m[k]
                          for k in ("kv_heads", "dim", "vdim")))
            if not ok:
                raise ConfigError(f"{wm}.kv_from must name an earlier attention layer with keys "
                                  f"and values of its own and the same kv_heads, dim and vdim")
    else:
        left, right = _section(m, "left", wm), _section(m, "right", wm)
        _check_heads(left, wm + ".left")
        if left["vdim"] != left["dim"]:
            raise ConfigError(f"{wm}.left.vdim must equal dim: the values are the keys")
        mask = left.get("mask")
        if mask is not None:
            mask = _section(left, "mask", wm + ".left")
            positive_int(f"{wm}.left.mask.size", need(mask, "size"))
            _count(f"{wm}.left.mask.keep_first", mask.get("keep_first", 0))
        for key in ("heads", "dim"):
            positive_int(f"{wm}.right.{key}", need(right, key))
        _number(f"{wm}.left_scale", need(m, "left_scale"))
        _number(f"{wm}.right_scale", need(m, "right_scale"))
    _check_mlp(i, layer.get("mlp"))


@dataclass(frozen=True)
class MafuzenConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    side_dim: int                       # 0: no per-layer token input
    layers: tuple                       # the layer entries of config.json, as they stand
    architectures: tuple[str, ...] = ("Mafuzen",)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MafuzenConfig":
        vocab = positive_int("vocab", need(raw, "vocab"))
        width = positive_int("width", need(raw, "width"))
        emb = raw.get("embedding")
        scale = 1.0 if emb is None else _number(
            "embedding.scale", need(_section(raw, "embedding", "config.json"), "scale"))
        eps = _number("norm.eps", need(_section(raw, "norm", "config.json"), "eps"), positive=True)
        side = raw.get("token_side")
        side_dim = 0 if side is None else positive_int(
            "token_side.dim", need(_section(raw, "token_side", "config.json"), "dim"))
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        for i, layer in enumerate(layers):
            _check_layer(i, layer, layers)
        return cls(vocab, width, scale, eps, side_dim, tuple(copy.deepcopy(list(layers))))

    def to_dict(self) -> dict[str, Any]:
        out = {"architecture": "Mafuzen", "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        return out

    def num_parameters(self) -> int:
        return sum(math.prod(t.shape) for t in init_weights(self, 0, shapes_only=True).values())


def _norm_spec(name: str, width: int, eps: float) -> PartSpec:
    return PartSpec("layernorm", dict(width=width, eps=eps, weight=name, bias=name + ".b"))


def _relu2_ff(prefix: str, width: int, inner: int) -> PartSpec:
    return PartSpec("dense", dict(width=width, inner=inner, activation="relu2",
                                  in_weight=prefix + "up", in_bias=None,
                                  out_weight=prefix + "down", out_bias=None,
                                  stored_in_out=False))


def build_spec(cfg: MafuzenConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers, schedule = [], []
    entry_of: dict[int, int] = {}          # layer -> the cache entry (or state) it owns
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        reads = None
        if layer["type"] == "retention":
            rot = m.get("rot") or {"base": 10000.0, "dims": 0}
            mixer = PartSpec("retention", dict(
                width=W, n_heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                decay=tuple(_decays(m, p + "mixer")), rot_base=rot["base"], rot_dims=rot["dims"],
                eps=eps, prefix=p + "mix."))
        elif layer["type"] == "attention":
            reads = m.get("kv_from")
            mixer = PartSpec("span_attention", dict(
                width=W, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                value_dim=m["vdim"], scale=m["scale"], slopes=distance_slopes(m["heads"]),
                shares_cache=reads is not None, prefix=p + "mix."))
        else:
            left, right = m["left"], m["right"]
            mask = left.get("mask") or {"size": 0}
            mixer = PartSpec("summed_pair", dict(
                left=PartSpec("span_attention", dict(
                    width=W, n_heads=left["heads"], n_kv_heads=left["kv_heads"],
                    head_dim=left["dim"], value_dim=left["dim"], scale=left["scale"],
                    window=mask["size"], keep_first=mask.get("keep_first", 0), qk_norm=True,
                    eps=eps, values_are_keys=True, gate=True, out_scale=m["left_scale"],
                    prefix=p + "mix.left.")),
                right=PartSpec("time_mix", dict(
                    width=W, n_heads=right["heads"], dim=right["dim"], eps=eps,
                    out_scale=m["right_scale"], prefix=p + "mix.right."))))
        if reads is None:
            entry_of[i] = len(entry_of)
            schedule.append(LayerCall(i, entry_of[i], True))
        else:
            schedule.append(LayerCall(i, entry_of[reads], False))     # layer `reads` wrote them
        parts = dict(norm1=_norm_spec(p + "norm1", W, eps), mixer=mixer,
                     norm1b=_norm_spec(p + "norm1b", W, eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                ff = PartSpec("gated", dict(width=W, inner=mlp["ff"], activation="silu",
                                            gate_weight=p + "mlp.gate", up_weight=p + "mlp.up",
                                            down_weight=p + "mlp.down"))
            else:
                shared = mlp.get("shared")
                ff = PartSpec("routed_experts", dict(
                    width=W, ff=mlp["expert"]["ff"], experts=mlp["router"]["experts"],
                    top=mlp["router"]["top"], scoring="table", activation="relu2",
                    router=p + "mlp.table", table_rows=cfg.vocab, expert_prefix=p + "mlp.e",
                    shared=_relu2_ff(p + "mlp.shared.", W, shared["ff"]) if shared else None))
            parts.update(norm2=_norm_spec(p + "norm2", W, eps), feed_forward=ff,
                         norm2b=_norm_spec(p + "norm2b", W, eps))
        if cfg.side_dim:
            parts["side"] = PartSpec("token_side_input", dict(
                width=W, dim=cfg.side_dim, offset=i * cfg.side_dim, table="side.embed",
                table_shape=(cfg.vocab, len(cfg.layers) * cfg.side_dim),
                gate_weight=p + "side.gate", proj_weight=p + "side.proj",
                norm_weight=p + "side.norm", eps=eps))
        layers.append(LayerSpec("sandwich_norm", parts))
    return ModelSpec(
        name="Mafuzen", vocab_size=cfg.vocab, width=W, max_positions=None,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=W, table="embed",
                                               scale=cfg.embedding_scale)),
        position=PartSpec("none", {}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=_norm_spec("final.norm", W, eps),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=W, weight="embed")),
        eos_token_id=None)


def init_weights(cfg: MafuzenConfig, seed: int, shapes_only: bool = False):
    """Seeded random float32 weights (integer tables int32) under the checkpoint's names, drawn
    from one CPU generator in the order the names are listed here.  Matrices ~ N(0, 1/sqrt(in));
    norm weights near 1, norm biases, blends, decays and bonuses spread enough that leaving one
    out changes the logits."""
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

    def norm(name):
        put(name, (W,), 0.1, 1.0)
        put(name + ".b", (W,), 0.1)

    W, L = cfg.width, len(cfg.layers)
    put("embed", (cfg.vocab, W), 1.0 / max(cfg.embedding_scale, 1e-6))
    if cfg.side_dim:
        put("side.embed", (cfg.vocab, L * cfg.side_dim), 1.0)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b"):
            norm(p + n)
        a = p + "mix."
        if layer["type"] == "retention":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            put(a + "q", (H * D, W)); put(a + "k", (H * D, W)); put(a + "v", (H * V, W))
            put(a + "g", (H * V, W), 2.0 / math.sqrt(W)); put(a + "o", (W, H * V))
        elif layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            put(a + "q", (H * D, W), 2.0 / math.sqrt(W))
            if m.get("kv_from") is None:
                put(a + "k", (G * D, W), 2.0 / math.sqrt(W)); put(a + "v", (G * V, W))
            put(a + "o", (W, H * V))
        else:
            left, right = m["left"], m["right"]
            H, G, D = left["heads"], left["kv_heads"], left["dim"]
            b = a + "left."
            put(b + "q", (H * D, W)); put(b + "k", (G * D, W))
            put(b + "g", (H * D, W), 2.0 / math.sqrt(W)); put(b + "o", (W, H * D))
            HR, DR = right["heads"], right["dim"]
            c = a + "right."
            rank = max(2, min(32, W // 16))
            for s in ("r", "k", "v", "g", "w"):
                put(c + "mu." + s, (W,), 0.25, 0.5)
            for s in ("r", "k", "v"):
                put(c + s, (HR * DR, W))
            put(c + "g", (HR * DR, W), 2.0 / math.sqrt(W))
            put(c + "w1", (rank, W)); put(c + "w2", (HR * DR, rank), 1.0 / math.sqrt(rank))
            put(c + "w0", (HR * DR,), 1.0, -2.0)
            put(c + "u", (HR, DR), 0.5, 0.5)
            put(c + "norm", (HR * DR,), 0.1, 1.0)
            put(c + "o", (W, HR * DR))
        mlp = layer.get("mlp")
        if mlp is not None:
            for n in ("norm2", "norm2b"):
                norm(p + n)
            f = p + "mlp."
            if mlp["kind"] == "dense":
                put(f + "gate", (mlp["ff"], W), 2.0 / math.sqrt(W))
                put(f + "up", (mlp["ff"], W), 2.0 / math.sqrt(W))
                put(f + "down", (W, mlp["ff"]))
            else:
                ff, E, top = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
                for e in range(E):
                    put(f"{f}e{e}.up", (ff, W), 2.0 / math.sqrt(W))
                    put(f"{f}e{e}.down", (W, ff))
                if shapes_only:
                    w[f + "table"] = torch.empty((cfg.vocab, top), dtype=torch.int32, device="meta")
                else:       # every row names `top` different experts
                    w[f + "table"] = torch.rand((cfg.vocab, E), generator=gen).argsort(1)[
                        :, :top].to(torch.int32).contiguous()
                if mlp.get("shared") is not None:
                    put(f + "shared.up", (mlp["shared"]["ff"], W), 2.0 / math.sqrt(W))
                    put(f + "shared.down", (W, mlp["shared"]["ff"]))
        if cfg.side_dim:
            s = p + "side."
            put(s + "gate", (cfg.side_dim, W), 2.0 / math.sqrt(W))
            put(s + "proj", (W, cfg.side_dim))
            put(s + "norm", (W,), 0.1, 0.5)
    norm("final.norm")
    return w


def _retention(heads, dim, vdim, rot_dims=None, base=10000.0):
    decay = [1.0 - 2.0 ** (-4 - 5 * h / max(1, heads - 1)) for h in range(heads)]
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}


def _attention(heads, kv_heads, dim, vdim, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": 1.0 / math.sqrt(dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _parallel(heads, kv_heads, dim, window, keep_first, r_heads, r_dim, left_scale=0.5,
              right_scale=1.0):
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                     "scale": 1.0 / math.sqrt(dim) * 4.0,
                     "mask": {"size": window, "keep_first": keep_first}},
            "right": {"heads": r_heads, "dim": r_dim},
            "left_scale": left_scale, "right_scale": right_scale}


def _moe(ff, experts, top, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def _preset(vocab, width, side_dim, layers, eps=1e-6):
    out = {"architecture": "Mafuzen", "vocab": vocab, "width": width,
           "embedding": {"scale": math.sqrt(width)}, "norm": {"eps": eps}, "layers": layers}
    if side_dim:
        out["token_side"] = {"dim": side_dim}
    return out


def _stack(width, heads, kv_heads, dim, r_heads, ff, moe):
    """Four layers, one of each mixer and a reader of the second layer's keys and values;
    dense and routed feed-forwards in turn."""
    dense = {"kind": "dense", "ff": ff}
    return [
        {"type": "retention", "mixer": _retention(width // 128, 128, 128), "mlp": dense},
        {"type": "attention", "mixer": _attention(heads, kv_heads, dim, dim),
         "mlp": copy.deepcopy(moe)},
        {"type": "parallel", "mixer": _parallel(heads, kv_heads, dim, 256, 4, r_heads, 64),
         "mlp": dict(dense)},
        {"type": "attention", "mixer": _attention(heads, kv_heads, dim, dim, kv_from=1),
         "mlp": copy.deepcopy(moe)},
    ]


PRESETS: dict[str, dict] = {
    # a few hundred thousand parameters: for demonstrations and smoke runs
    "mafuzen-tiny": _preset(384, 96, 8, [
        {"type": "retention", "mixer": _retention(3, 16, 24, rot_dims=8, base=500.0),
         "mlp": {"kind": "dense", "ff": 160}},
        {"type": "attention", "mixer": _attention(4, 2, 16, 24), "mlp": _moe(48, 6, 2, 64)},
        {"type": "parallel", "mixer": _parallel(4, 1, 16, 40, 3, 2, 16), "mlp": None},
        {"type": "attention", "mixer": _attention(4, 2, 16, 24, kv_from=1),
         "mlp": _moe(48, 6, 1)},
    ]),
    # layer sizes of a small and a mid-sized production model, few layers: for measurements
    "mafuzen-1k": _preset(32768, 1024, 64, _stack(1024, 16, 4, 64, 16, 4096,
                                                  _moe(512, 32, 4, 1024))),
    "mafuzen-2k": _preset(32768, 2048, 64, _stack(2048, 32, 8, 64, 32, 8192,
                                                  _moe(1024, 64, 6, 2048))),
}

MAFUZEN = Architecture(name="Mafuzen", config_cls=MafuzenConfig, build_spec=build_spec,
                       init_weights=init_weights, model_types=("mafuzen",), presets=PRESETS,
                       preset_aliases={})
register_architecture(MAFUZEN, replace=True)
