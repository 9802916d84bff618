"""Mafuzen without a GPU: the configuration, the spec, the plain implementation's own sanity,
and the engine (step function, cache manager, state slots) driven with the plain twins of the
kernels against the plain model."""

import copy
import io
import math

import pytest
import torch

import mafuzen_cases as mc
import plain_mafuzen
import plain_ops
import traces
from hetero_serve_b200.config import ConfigError
from hetero_serve_b200.config.model_config import architecture_of
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import Model

TOL = 1e-4          # float32 rows between the twins; logits of these models reach 10 to 30
F64 = torch.float64


def _replay(case, steps, tmp_path, max_tokens, **kw):
    out = tmp_path / "out"
    out.mkdir(exist_ok=True)
    assert replay(model_dir=case.dir, dtype="float32", out_dir=out, max_tokens=max_tokens,
                  lines=traces.lines_of(steps), report=io.StringIO(), device="cpu",
                  ops=plain_ops.PlainOps(), **kw) == 0
    return out


def _worst(case, out, index, reqs):
    got = traces.collect(out, index, case.vocab)
    return traces.worst_error(got, {r: case.logits(t) for r, t in reqs.items()})


def _runner(case, pages, slots=1):
    model, _ = load_model(case.dir, "float32", "cpu")
    return Runner(model, num_pages=pages, page_size=16, max_requests=slots, dtype=torch.float32,
                  device="cpu", ops=plain_ops.PlainOps())


# -- configuration and spec -----------------------------------------------------------------
def test_config_is_read_and_written_back(mafuzen_case):
    arch = architecture_of(mafuzen_case.config)
    cfg = arch.config_cls.from_dict(mafuzen_case.config)
    assert arch.name == "Mafuzen"
    assert arch.config_cls.from_dict(cfg.to_dict()) == cfg
    assert cfg.width == mafuzen_case.config["width"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][5]["mixer"].update(vdim=8), "kv_from"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][2]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "do not fit"),
    (lambda c: c["layers"][1].update(type="lstm"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["token_side"].update(dim=0), "token_side"),
])
def test_config_errors(change, message):
    cfg = copy.deepcopy(mc.CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).config_cls.from_dict(cfg)


def test_cache_entries_and_states_of_the_spec(mafuzen_cases):
    case = mafuzen_cases["case_a"]
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    # rows [key | value]: one plane.  Layers 3 and 5 read layer 1's rows: one entry for three
    # layers; the window's group keeps its first tokens
    groups = {(g.kv_heads, g.head_dim, g.window, g.keep_first, g.planes): len(g.entries)
              for g in model.cache_groups}
    assert groups == {(2, 32, 0, 0, 1): 1, (2, 24, 21, 3, 1): 1}
    calls = model.schedule
    assert calls[3].cache == calls[1].cache == calls[5].cache
    assert not calls[3].writes_cache and not calls[5].writes_cache and calls[1].writes_cache
    assert model.state_shapes == {0: (3 * 12 * 20,), 2: (3 * 12 * 12 + 44,), 4: (2 * 16 * 8,)}
    names = set(model.tensor_requests())
    assert "l3.mix.k" not in names and "l3.mix.q" in names and "l2.norm2" not in names
    assert "l2.mix.left.v" not in names and "l1.mlp.e4.up" in names and "l1.mlp.e0.gate" not in names
    assert model.spec.max_positions is None


def test_the_inner_size_of_the_decay_is_read_off_its_tensor(mafuzen_cases, tmp_path):
    from hetero_serve_b200.weights import write_safetensors
    case = mafuzen_cases["case_b"]
    raw = dict(case.raw)
    g = torch.Generator().manual_seed(3)
    raw["l0.mix.right.w1"] = torch.randn(7, 40, generator=g) * 0.2
    raw["l0.mix.right.w2"] = torch.randn(8, 7, generator=g) * 0.4
    (tmp_path / "config.json").write_text((__import__("pathlib").Path(case.dir) / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", raw, {"format": "pt"})
    model, _ = load_model(tmp_path, "float32", "cpu")
    rn = Runner(model, num_pages=4, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(20, 4)
    got = rn.step([StepEntry("a", toks, want=[19])]).logits[0].double()
    want = plain_mafuzen.forward(case.config, plain_mafuzen.prepare(raw), toks)[19]
    assert (got - want).abs().max() < TOL


def test_a_checkpoint_that_does_not_fit(mafuzen_cases, tmp_path):
    from hetero_serve_b200.weights import WeightError, write_safetensors
    case = mafuzen_cases["case_a"]
    raw = {n: t for n, t in case.raw.items() if n != "l1.mlp.table"}
    raw["l3.mix.k"] = torch.zeros(24, 44)
    (tmp_path / "config.json").write_text((__import__("pathlib").Path(case.dir) / "config.json").read_text())
    write_safetensors(tmp_path / "model.safetensors", raw, {"format": "pt"})
    with pytest.raises(WeightError) as err:
        load_model(tmp_path, "float32", "cpu")
    assert "l1.mlp.table" in str(err.value) and "l3.mix.k" in str(err.value)


# -- the plain implementation's own sanity ----------------------------------------------------
def test_plain_prefix_property(mafuzen_case):
    toks = mafuzen_case.tokens(70, 5)
    full, part = mafuzen_case.logits(toks), mafuzen_case.logits(toks[:23])
    assert (full[:23] - part).abs().max() < 1e-9


def test_plain_visibility_rule():
    seen = [j for j in range(40) if plain_mafuzen.visible(30, j, 7, 3)]
    assert seen == [0, 1, 2, 24, 25, 26, 27, 28, 29, 30]
    assert [j for j in range(9) if plain_mafuzen.visible(5, j, 0, 0)] == [0, 1, 2, 3, 4, 5]
    assert [j for j in range(9) if plain_mafuzen.visible(4, j, 7, 3)] == [0, 1, 2, 3, 4]


def test_plain_visibility_of_one_key(mafuzen_planted):
    """The marked key counts inside the window and, as one of the kept first tokens, for ever;
    behind the window it is not seen at all."""
    case = mafuzen_planted["window"]
    mask = case.config["layers"][0]["mixer"]["left"]["mask"]
    size, keep = mask["size"], mask["keep_first"]
    for at in (keep - 1, keep, keep + 4):
        for i in range(at + 1, at + 30):
            t = mc.planted_tokens(case, at, i + 1, 3)
            blank = list(t)
            blank[at] = mc.MARK + 1
            change = float((case.logits(t)[-1] - case.logits(blank)[-1]).abs().max())
            if i - at < size or at < keep:
                assert change > 0.5, (at, i)
            else:
                assert change == 0.0, (at, i)


def test_plain_far_key_under_a_slope(mafuzen_planted):
    case = mafuzen_planted["slope"]
    t = mc.planted_tokens(case, 2, 400, 8)
    blank = list(t)
    blank[2] = mc.MARK + 1
    assert float((case.logits(t)[-1] - case.logits(blank)[-1]).abs().max()) > 0.5
    assert [round(plain_mafuzen.slope_of(h, 4), 6) for h in range(4)] == [0.25, 0.0625, 0.015625,
                                                                          0.003906]


def test_plain_retention_is_a_decaying_sum():
    """One head of one number, nothing rotated: o_t = q_t * sum_s decay^(t-s) k_s v_s."""
    T = 6
    w = {"m.q": torch.ones(1, 1), "m.k": torch.ones(1, 1), "m.v": torch.ones(1, 1),
         "m.g": torch.zeros(1, 1), "m.o": torch.ones(1, 1)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.arange(1, T + 1, dtype=F64)[:, None]
    S, want = 0.0, []
    for t in range(T):
        S = 0.5 * S + float(h[t, 0]) ** 2
        want.append(S * float(h[t, 0]))
    # the head norm of one number gives its sign, the gate silu(0) = 0: look at o before both
    m = {"heads": 1, "dim": 1, "vdim": 1, "decay": [0.5]}
    o = torch.zeros(T, dtype=F64)
    Sm = torch.zeros(1, 1, dtype=F64)
    for t in range(T):
        Sm = 0.5 * Sm + torch.outer(h[t] * 1.0, h[t])
        o[t] = (Sm.T @ h[t])[0]
    assert (o - torch.tensor(want, dtype=F64)).abs().max() < 1e-12
    assert plain_mafuzen.retention(m, w, "m.", h, 1e-6).abs().max() == 0.0      # gate closed


def test_plain_time_mix_bonus_and_decay():
    """One head of one number with all blends at 0 (every stream reads the token itself):
    o_t = r_t (S_(t-1) + u k_t v_t), S_t = w S_(t-1) + k_t v_t with w = exp(-exp(w0))."""
    T, W = 5, 1
    w = {f"m.mu.{s}": torch.zeros(W) for s in "rkvgw"}
    w.update({"m.r": torch.ones(1, 1), "m.k": torch.ones(1, 1), "m.v": torch.ones(1, 1),
              "m.g": torch.ones(1, 1) * 30.0, "m.w1": torch.zeros(2, 1), "m.w2": torch.zeros(1, 2),
              "m.w0": torch.tensor([-1.0]), "m.u": torch.tensor([[0.25]]),
              "m.norm": torch.ones(1), "m.o": torch.ones(1, 1)})
    w = {k: v.double() for k, v in w.items()}
    h = torch.tensor([[1.0], [2.0], [-1.0], [0.5], [3.0]], dtype=F64)
    dec = math.exp(-math.exp(-1.0))
    S, signs = 0.0, []
    for t in range(T):
        x = float(h[t, 0])
        signs.append(math.copysign(1.0, x * (S + 0.25 * x * x)))
        S = dec * S + x * x
    out = plain_mafuzen.time_mix({"heads": 1, "dim": 1}, w, "m.", h, 0.0)[:, 0]
    gate = 30.0 * h[:, 0] * torch.sigmoid(30.0 * h[:, 0])
    assert (out - torch.tensor(signs, dtype=F64) * gate).abs().max() < 1e-9


def test_plain_rotation_keeps_lengths_and_turns_by_the_difference():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(8, generator=g, dtype=F64), torch.randn(8, generator=g, dtype=F64)
    a = plain_mafuzen.rotate_halves(q, 9, 100.0, 6) @ plain_mafuzen.rotate_halves(k, 4, 100.0, 6)
    b = plain_mafuzen.rotate_halves(q, 25, 100.0, 6) @ plain_mafuzen.rotate_halves(k, 20, 100.0, 6)
    assert abs(float(a - b)) < 1e-12
    assert torch.equal(plain_mafuzen.rotate_halves(q, 9, 100.0, 6)[6:], q[6:])


# -- the engine with plain kernels -------------------------------------------------------------
@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(mafuzen_case, tmp_path, driver):
    reqs = {f"r{i}": mafuzen_case.tokens(n, 50 + i) for i, n in enumerate((1, 2, 19, 83))}
    if driver == "whole":
        steps, index = traces.whole(reqs)
    elif driver == "tail":
        steps, index = traces.tail_one_by_one(reqs, tail=45)
    else:
        steps, index = traces.portions(reqs, sizes=(7, 2, 16, 3, 2, 5, 21))
    out = _replay(mafuzen_case, steps, tmp_path, max_tokens=128)
    err, where = _worst(mafuzen_case, out, index, reqs)
    assert err < TOL, (err, where)


def test_mixed_batches_reuse_pages_and_slots(mafuzen_case, tmp_path):
    reqs = {f"r{i}": mafuzen_case.tokens(n, 70 + i) for i, n in
            enumerate((47, 5, 18, 66, 3, 26))}
    steps, index, peak = traces.mixed(reqs, seed=3, max_live=3, sizes=(1, 2, 5, 1, 17, 3, 1, 9))
    out = _replay(mafuzen_case, steps, tmp_path, max_tokens=peak, max_requests=3)
    err, where = _worst(mafuzen_case, out, index, reqs)
    assert sum(len(v) for v in index.values()) > 20 and err < TOL, (err, where)


def test_a_slot_is_cleared_for_its_next_owner(mafuzen_cases):
    case = mafuzen_cases["case_a"]
    rn = _runner(case, pages=8)
    a, b = case.tokens(50, 1), case.tokens(29, 2)
    rn.step([StepEntry("a", a)])
    rn.close("a")
    rn.step([StepEntry("b", b[:1])])               # the kept previous row must be zeros again
    rn.step([StepEntry("b", b[1:11])])
    res = rn.step([StepEntry("b", b[11:], want=[17])])
    assert (res.logits[0].double() - case.logits(b)[28]).abs().max() < TOL
    rn.manager.check()


def test_pages_behind_the_window_are_given_back_but_not_the_first(mafuzen_planted):
    """A request far longer than the pool holds runs in portions: the window's pages go back
    to the pool as it advances, the page of the kept first tokens stays and is still read."""
    case = mafuzen_planted["window"]               # window 13, the first 5 kept
    rn = _runner(case, pages=4)
    toks = mc.planted_tokens(case, 2, 200, 17)
    want, at = case.logits(toks), 0
    for n in (20, 13, 2, 19, 1, 1, 20, 7, 20, 20, 3, 20, 1, 20, 20, 2, 10, 1):
        res = rn.step([StepEntry("a", toks[at:at + n], want=[n - 1])])
        assert (res.logits[0].double() - want[at + n - 1]).abs().max() < TOL, at
        at += n
        assert rn.manager.pages_free(0) >= 1
    assert at == 200
    table = rn.manager.table("a", 0) if hasattr(rn.manager, "table") else None
    rn.manager.check()
    rn.close("a")
    assert rn.manager.pages_free(0) == rn.manager.pools[0].num_pages


@pytest.mark.parametrize("how", ["whole", "alone", "portions"])
def test_the_edges_of_the_window_and_of_the_first_tokens(mafuzen_planted, how):
    """One key that takes nearly all of the softmax when it is visible, asked for from every
    distance around the window's edge, from a first token that is kept and the next one that is
    not, and from far away: in a prompt, decoded alone, and at the end of a portion of two."""
    case = mafuzen_planted["window"]
    for at in (0, 4, 5, 15, 16):                   # kept / not kept; a page's last and first row
        for d in (1, 11, 12, 13, 14, 15, 16, 17, 31, 32, 33, 90):
            t = mc.planted_tokens(case, at, at + d + 1, 100 + d)
            rn = _runner(case, pages=12)
            n = len(t)
            if how == "whole":
                res = rn.step([StepEntry("a", t, want=[n - 1])])
            elif how == "alone":
                rn.step([StepEntry("a", t[:-1])])
                res = rn.step([StepEntry("a", t[-1:], want=[0])])
            else:
                cut = max(1, n - 2)
                head = t[:cut]
                for a in range(0, len(head), 7):
                    rn.step([StepEntry("a", head[a:a + 7])])
                res = rn.step([StepEntry("a", t[cut:], want=[n - cut - 1])])
            err = float((res.logits[-1].double() - case.logits(t)[-1]).abs().max())
            assert err < TOL, (at, d, err)


@pytest.mark.parametrize("how", ["whole", "alone"])
def test_a_far_key_under_the_slope(mafuzen_planted, how):
    case = mafuzen_planted["slope"]
    for at, n in ((0, 300), (15, 333), (16, 210), (100, 102)):
        t = mc.planted_tokens(case, at, n, 7 + at)
        rn = _runner(case, pages=24)
        if how == "whole":
            res = rn.step([StepEntry("a", t, want=[n - 1])])
        else:
            rn.step([StepEntry("a", t[:-1])])
            res = rn.step([StepEntry("a", t[-1:], want=[0])])
        err = float((res.logits[-1].double() - case.logits(t)[-1]).abs().max())
        assert err < TOL, (at, n, err)


def test_long_decoding(mafuzen_cases):
    case = mafuzen_cases["case_b"]
    t = case.tokens(120, 9)
    rn = _runner(case, pages=12)
    rn.step([StepEntry("d", t[:3])])
    want = case.logits(t)
    for i in range(3, 120):
        res = rn.step([StepEntry("d", [t[i]], want=[0])])
        assert (res.logits[0].double() - want[i]).abs().max() < TOL, i


def test_the_parts_in_another_arrangement(mafuzen_cases):
    """The new mixers and feed-forwards under norms BEFORE the sublayers only (x +=
    mixer(norm1(x)); x += ff(norm2(x))): they then add into the stream themselves."""
    import dataclasses
    from hetero_serve_b200.parts.spec import LayerCall, LayerSpec
    case = mafuzen_cases["case_a"]
    arch = architecture_of(case.config)
    spec = arch.build_spec(arch.config_cls.from_dict(case.config))
    layers = []
    for i in (0, 1, 2):
        parts = {k: v for k, v in spec.layers[i].parts.items()
                 if k not in ("norm1b", "norm2b", "side")}
        if i == 2:              # this layer has no feed-forward: borrow the first one's
            parts.update(norm2=spec.layers[0].parts["norm2"],
                         feed_forward=spec.layers[0].parts["feed_forward"])
        layers.append(LayerSpec("pre_norm", parts))
    spec = dataclasses.replace(spec, layers=tuple(layers),
                               schedule=(LayerCall(0), LayerCall(1), LayerCall(2)))
    model = Model(spec)
    model.bind({n: case.raw[n] for n in model.tensor_requests()}, torch.float32, "cpu")
    rn = Runner(model, num_pages=6, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(60, 3)
    rn.step([StepEntry("a", toks[:13])])
    got = rn.step([StepEntry("a", toks[13:], want=[0, 46])]).logits.double()
    w, cfg, P = case.plain, case.config, plain_mafuzen
    eps = cfg["norm"]["eps"]
    ln = lambda name, v: P.layer_norm(v, w[name], w[name + ".b"], eps)
    L = cfg["layers"]
    x = w["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
    x = x + P.retention(L[0]["mixer"], w, "l0.mix.", ln("l0.norm1", x), eps)
    x = x + P.dense_ff(w, "l0.mlp.", ln("l0.norm2", x))
    x = x + P.attention(L[1]["mixer"], w, "l1.mix.", ln("l1.norm1", x))[0]
    x = x + P.table_moe(L[1]["mlp"], w, "l1.mlp.", ln("l1.norm2", x), toks)
    x = x + P.parallel(L[2]["mixer"], w, "l2.mix.", ln("l2.norm1", x), eps)
    x = x + P.dense_ff(w, "l0.mlp.", ln("l0.norm2", x))
    want = ln("final.norm", x) @ w["embed"].T
    assert (got - want[[13, 59]]).abs().max() < TOL


@pytest.mark.parametrize("which", ["retention only", "pairs without a mask", "windows that differ",
                                   "a chain of readers", "one layer"])
def test_other_orders_of_layers(which, tmp_path):
    """Models of one kind of layer (no page group at all; no window), page groups that differ
    only in their window or kept tokens, several readers of two writers, a single layer: mixed
    batches with pages and slots used again against the plain model."""
    import json
    from hetero_serve_b200.weights import read_safetensors, write_model_dir
    moe = mc._moe(16, 3, 2)
    layers = {
        "retention only": [mc._layer("retention", mc._ret(2, 8, 12, [0.9, 0.99], rot_dims=4, base=100.0),
                                     {"kind": "dense", "ff": 64})] * 2,
        "pairs without a mask": [mc._layer("parallel", mc._par(2, 1, 8, 0, 0, 1, 8), None)] * 2,
        "windows that differ": [mc._layer("parallel", mc._par(2, 1, 8, 5, 0, 1, 8), None),
                                mc._layer("parallel", mc._par(2, 1, 8, 9, 30, 1, 8), None),
                                mc._layer("parallel", mc._par(2, 1, 8, 9, 0, 1, 8), moe)],
        "a chain of readers": [mc._layer("attention", mc._att(4, 2, 8, 4, scale=0.3), moe),
                               mc._layer("attention", mc._att(4, 2, 8, 4, kv_from=0), moe),
                               mc._layer("attention", mc._att(2, 2, 8, 4), None),
                               mc._layer("attention", mc._att(4, 2, 8, 4, kv_from=2), moe),
                               mc._layer("attention", mc._att(2, 2, 8, 4, kv_from=0), moe)],
        "one layer": [mc._layer("attention", mc._att(4, 2, 8, 4), None)],
    }[which]
    cfg = mc._model(90, 48, 1e-6, layers, scale=3.0, side=4 if which != "one layer" else 0)
    folder = tmp_path / "model"
    write_model_dir(folder, cfg, 1, "float32")
    case = mc.Case(which, folder, json.loads((folder / "config.json").read_text()), 1)
    reqs = {f"r{i}": case.tokens(n, 20 + i) for i, n in enumerate((70, 9, 33))}
    steps, index, peak = traces.mixed(reqs, seed=1, max_live=2, sizes=(1, 2, 5, 1, 17, 3))
    out = _replay(case, steps, tmp_path, max_tokens=peak, max_requests=2)
    err, where = _worst(case, out, index, reqs)
    assert err < TOL, (err, where)
