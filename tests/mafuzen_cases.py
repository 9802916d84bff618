"""Small Mafuzen configurations for the tests, with random weights written to temporary
folders, and the plain implementation's view of the same weights."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

import plain_mafuzen


def _ret(heads, dim, vdim, decay, rot_dims=None, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot_dims is not None:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def _att(heads, kv_heads, dim, vdim, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _par(heads, kv_heads, dim, window, keep_first, r_heads, r_dim, scale=None, left_scale=0.7,
         right_scale=1.3):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
            "scale": scale if scale is not None else 3.0 / math.sqrt(dim)}
    if window:
        left["mask"] = {"size": window, "keep_first": keep_first}
    return {"left": left, "right": {"heads": r_heads, "dim": r_dim},
            "left_scale": left_scale, "right_scale": right_scale}


def _moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _model(vocab, width, eps, layers, scale=1.0, side=0):
    out = {"architecture": "Mafuzen", "vocab": vocab, "width": width,
           "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}
    if side:
        out["token_side"] = {"dim": side}
    return out


# sizes that are no multiple of a page (16), of 8 or of each other; grouped heads; values of
# another size than the keys; a partly rotated retention; a window and kept first tokens that end
# inside a page; two readers of one layer's keys; all three feed-forwards and none; a token input
CASE_A = _model(311, 44, 1e-5, [
    _layer("retention", _ret(3, 12, 20, [0.9, 0.97, 0.995], rot_dims=8, base=300.0),
           {"kind": "dense", "ff": 72}),
    _layer("attention", _att(6, 2, 12, 20, scale=0.4), _moe(28, 5, 2, shared=36)),
    _layer("parallel", _par(4, 2, 12, 21, 3, 3, 12), None),
    _layer("attention", _att(6, 2, 12, 20, kv_from=1), _moe(20, 4, 3)),
    _layer("retention", _ret(2, 16, 8, [0.9375, 0.75], rot_dims=16, base=5e5),
           {"kind": "dense", "ff": 40}),
    _layer("attention", _att(6, 2, 12, 20, scale=0.2, kv_from=1), None),
], scale=6.5, side=5)
# what the first case keeps apart is equal or 1 here, or absent: one head everywhere, key/value
# heads equal to the query heads, a decay of 1 (nothing fades), nothing rotated, a window of one
# token that keeps the first two, a pair without a window, one expert chosen of one, every expert
# chosen, scales of 1, no token input
CASE_B = _model(257, 40, 1e-6, [
    _layer("parallel", _par(1, 1, 8, 1, 2, 1, 8, scale=1.0, left_scale=1.0, right_scale=1.0),
           _moe(24, 1, 1)),
    _layer("retention", _ret(1, 8, 8, 1.0), None),
    _layer("attention", _att(2, 2, 8, 8), _moe(16, 3, 3, shared=16)),
    _layer("parallel", _par(2, 2, 16, 0, 0, 2, 4), {"kind": "dense", "ff": 48}),
    _layer("retention", _ret(2, 8, 24, [1.0, 0.5], rot_dims=0), {"kind": "dense", "ff": 48}),
])
# sizes the wide kernels take (multiples of 64), stored in bfloat16; a window longer than most
# portions of the tests beside layers that see everything
CASE_C = _model(512, 128, 1e-6, [
    _layer("retention", _ret(2, 64, 64, [0.97, 0.995], rot_dims=64), {"kind": "dense", "ff": 256}),
    _layer("attention", _att(4, 2, 64, 64), _moe(64, 8, 2, shared=128)),
    _layer("parallel", _par(4, 1, 64, 48, 16, 2, 64), _moe(64, 8, 2)),
    _layer("attention", _att(4, 2, 64, 64, kv_from=1), {"kind": "dense", "ff": 256}),
], scale=math.sqrt(128), side=16)

CASES = {"case_a": (CASE_A, 51), "case_b": (CASE_B, 52), "case_c": (CASE_C, 53)}


class Case:
    def __init__(self, name, folder, config, seed):
        from hetero_serve_b200.weights import read_safetensors
        self.name, self.dir, self.config, self.seed = name, str(folder), config, seed
        self.raw = read_safetensors(Path(folder) / "model.safetensors")
        self.plain = plain_mafuzen.prepare(self.raw)
        self.plain_bf16 = plain_mafuzen.prepare(self.raw, round_to=torch.bfloat16)
        self.vocab = config["vocab"]
        self._memo = {}

    def logits(self, tokens, dtype="float32"):
        key = (tuple(tokens), dtype)
        if key not in self._memo:
            w = self.plain_bf16 if dtype == "bfloat16" else self.plain
            self._memo[key] = plain_mafuzen.forward(self.config, w, tokens)
        return self._memo[key]

    def tokens(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.vocab, (n,), generator=g).tolist()


def make_cases(tmp_path_factory):
    from hetero_serve_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed) in CASES.items():
        folder = tmp_path_factory.mktemp("mafuzen_" + name)
        write_model_dir(folder, cfg, seed, "bfloat16" if name == "case_c" else "float32")
        stored = json.loads((folder / "config.json").read_text())
        out[name] = Case(name, folder, stored, seed)
    return out


# -- models in which ONE key stands out -------------------------------------------------------
# Token ASK's query and token MARK's key meet in one number of each head and nowhere else: every
# other pair of tokens scores 0 there, so an ASK query gives nearly all of its softmax to an
# earlier MARK it can see, and an edge that is one position off changes the logits by far more
# than any tolerance.  Each model is one layer whose other half (if any) is switched off, so a
# MARK that is not visible changes nothing at all.
MARK, ASK = 7, 11
PLANTED = {
    # a window of 13 that keeps the first 5 tokens
    "window": _model(97, 32, 1e-5, [
        _layer("parallel", _par(2, 1, 16, 13, 5, 1, 8, scale=1.0, left_scale=1.0,
                                right_scale=0.0), {"kind": "dense", "ff": 40})], side=3),
    # every key is seen, at a price that grows with the distance
    "slope": _model(97, 32, 1e-5, [
        _layer("attention", _att(2, 1, 16, 8, scale=0.5), {"kind": "dense", "ff": 40})]),
}


def planted_case(tmp_path_factory, which):
    from hetero_serve_b200.config.model_config import architecture_of
    from hetero_serve_b200.weights import write_safetensors
    raw = PLANTED[which]
    arch = architecture_of(raw)
    cfg = arch.config_cls.from_dict(raw)
    w = arch.init_weights(cfg, 61)
    W = raw["width"]
    w["embed"][:, :4] = 0.0
    w["embed"][MARK, 0], w["embed"][MARK, 1] = 3.0, -3.0
    w["embed"][ASK, 2], w["embed"][ASK, 3] = 3.0, -3.0
    w["l0.norm1"], w["l0.norm1.b"] = torch.ones(W), torch.zeros(W)
    probe = torch.zeros(2, W)                       # rows that sum to 0: the norm's mean drops out
    probe[0, 0], probe[0, 1] = 1.0, -1.0
    probe[1, 2], probe[1, 3] = 1.0, -1.0
    if which == "window":
        m, pre = raw["layers"][0]["mixer"]["left"], "l0.mix.left."
        strength = 40.0                             # unit-RMS rows: the planted number takes all
    else:
        m, pre = raw["layers"][0]["mixer"], "l0.mix."
        strength = 1.5
    D = m["dim"]
    w[pre + "q"][:, :4] = 0.0
    w[pre + "k"][:, :4] = 0.0
    for hd in range(m["heads"]):
        w[pre + "q"][hd * D + D - 1] = probe[1] * strength
    w[pre + "k"][D - 1] = probe[0] * strength
    folder = tmp_path_factory.mktemp("mafuzen_planted_" + which)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", w, {"format": "pt"})
    return Case("planted_" + which, folder, json.loads((folder / "config.json").read_text()), 61)


def planted_tokens(case, mark_at, length, seed):
    """Random tokens without MARK and ASK, then MARK at ``mark_at`` and ASK as the last token."""
    t = [x if x not in (MARK, ASK) else MARK + 1 for x in case.tokens(length, seed)]
    t[mark_at] = MARK
    t[-1] = ASK
    return t


def rms_error(got, want):
    """Root mean square of the difference with its mean taken off, over the root mean square
    of the wanted row."""
    d = got.double() - want.double()
    d = d - d.mean()
    return math.sqrt(float((d * d).mean())) / max(1e-12, math.sqrt(float((want.double() ** 2).mean())))
