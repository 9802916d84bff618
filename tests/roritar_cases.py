"""Small Roritar configurations for the tests, with random weights written to temporary
folders, and the plain implementation's view of the same weights."""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

import plain_roritar


def _att(heads, kv_heads, dim, vdim, window, pool, rot_dims, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
            "mask": {"size": window, "pool": pool}, "rot": {"base": base, "dims": rot_dims}}


def _rec(width, blocks, taps):
    return {"width": width, "blocks": blocks, "conv": taps}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _model(vocab, width, eps, layers, loop=None, logit_scale=1.0, softcap=None):
    out = {"architecture": "Roritar", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "logit_scale": logit_scale, "logit_softcap": softcap, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# windows and blocks that are no multiple of a page (16) nor of each other, grouped query
# heads, keys partly rotated, a looped stretch that starts with a recurrent layer, a layer
# without a feed-forward, two attention layers that differ in every size
CASE_A = _model(311, 48, 1e-5, [
    _layer("attention", _att(4, 2, 24, 16, 21, 5, 12, base=500.0, scale=0.3), 80),
    _layer("rglru", _rec(40, 2, 4), 64),
    _layer("attention", _att(6, 3, 16, 10, 34, 3, 16, base=10000.0), None),
    _layer("rglru", _rec(36, 3, 3), 56),
], loop=(1, 3, 3), logit_scale=0.5, softcap=12.0)
# what the first case keeps apart is equal or 1 here: one head, one block of gates, one tap
# (no history), a block of one position (every token behind the window is its own block), a
# window of one, nothing rotated in the keys, no loop, no cap on the logits
CASE_B = _model(257, 40, 1e-6, [
    _layer("rglru", _rec(40, 1, 1), 48),
    _layer("attention", _att(1, 1, 32, 32, 9, 1, 0), 48),
    _layer("attention", _att(2, 2, 8, 6, 1, 4, 8, base=50.0), None),
    _layer("rglru", _rec(24, 4, 2), None),
])
# sizes the wide kernels take (multiples of 32 and 64), stored in bfloat16; a window longer
# than most prompts of the tests beside a short one; a loop over everything
CASE_C = _model(512, 128, 1e-6, [
    _layer("attention", _att(4, 1, 64, 64, 48, 16, 32), 256),
    _layer("rglru", _rec(128, 4, 4), 256),
    _layer("attention", _att(8, 2, 32, 64, 200, 8, 32), 256),
], loop=(0, 3, 2), logit_scale=0.25, softcap=30.0)

CASES = {"case_a": (CASE_A, 31), "case_b": (CASE_B, 32), "case_c": (CASE_C, 33)}


class Case:
    def __init__(self, name, folder, config, seed):
        from hetero_serve_b200.weights import read_safetensors
        self.name, self.dir, self.config, self.seed = name, str(folder), config, seed
        self.raw = read_safetensors(Path(folder) / "model.safetensors")
        self.plain = plain_roritar.prepare(self.raw)
        self.plain_bf16 = plain_roritar.prepare(self.raw, round_to=torch.bfloat16)
        self.vocab = config["vocab"]
        self._memo = {}

    def logits(self, tokens, dtype="float32"):
        key = (tuple(tokens), dtype)
        if key not in self._memo:
            w = self.plain_bf16 if dtype == "bfloat16" else self.plain
            self._memo[key] = plain_roritar.forward(self.config, w, tokens)
        return self._memo[key]

    def tokens(self, n, seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randint(0, self.vocab, (n,), generator=g).tolist()


def make_cases(tmp_path_factory):
    from hetero_serve_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed) in CASES.items():
        folder = tmp_path_factory.mktemp("roritar_" + name)
        write_model_dir(folder, cfg, seed, "bfloat16" if name == "case_c" else "float32")
        stored = json.loads((folder / "config.json").read_text())
        out[name] = Case(name, folder, stored, seed)
    return out


# -- a model in which ONE key stands out ------------------------------------------------------
# Token ASK's query and token MARK's key meet in one unrotated number of each head and nowhere
# else: every other pair of tokens scores 0 there, so an ASK query gives nearly all of its softmax
# to an earlier MARK it can see (or to the block mean that holds it), and an edge that is one position
# off changes the logits by far more than any tolerance.  The model is this one layer, so a MARK
# that is not visible changes nothing at all.
MARK, ASK = 7, 11
PLANTED = _model(97, 32, 1e-5, [
    _layer("attention", _att(2, 1, 16, 8, 13, 4, 8, base=100.0, scale=1.0), 40),
], logit_scale=1.0, softcap=20.0)


def planted_case(tmp_path_factory, strength=14.0):
    from hetero_serve_b200.config.model_config import architecture_of
    from hetero_serve_b200.weights import write_safetensors
    arch = architecture_of(PLANTED)
    cfg = arch.config_cls.from_dict(PLANTED)
    w = arch.init_weights(cfg, 41)
    m = PLANTED["layers"][0]["mixer"]
    D, W = m["dim"], PLANTED["width"]
    w["embed"][:, :4] = 0.0
    w["embed"][MARK, 0], w["embed"][MARK, 1] = 3.0, -3.0
    w["embed"][ASK, 2], w["embed"][ASK, 3] = 3.0, -3.0
    w["l0.norm1"] = torch.ones(W)
    probe = torch.zeros(2, W)                       # rows that sum to 0: the norm's mean drops out
    probe[0, 0], probe[0, 1] = 1.0, -1.0
    probe[1, 2], probe[1, 3] = 1.0, -1.0
    for hd in range(m["heads"]):
        w["l0.mix.q"][hd * D + D - 1] = probe[1]
    w["l0.mix.k"][D - 1] = probe[0]
    w["l0.mix.q.norm"] = torch.zeros(D)
    w["l0.mix.q.norm"][D - 1] = strength
    w["l0.mix.k.norm"] = torch.ones(D)
    folder = tmp_path_factory.mktemp("roritar_planted")
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", w, {"format": "pt"})
    return Case("planted", folder, json.loads((folder / "config.json").read_text()), 41)


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
