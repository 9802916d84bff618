"""Roritar without a GPU: configuration, spec and weights, and the engine's step function,
cache groups and state slots with the kernels replaced by their plain twins
(tests/plain_ops.py) — against the plain implementation of the whole model
(tests/plain_roritar.py)."""

import copy
import io

import pytest
import torch

import plain_ops
import plain_roritar
import roritar_cases as rc
import traces
from hetero_serve_b200.config import ConfigError
from hetero_serve_b200.config.model_config import architecture_of
from hetero_serve_b200.engine.loading import load_model
from hetero_serve_b200.engine.replay import replay
from hetero_serve_b200.engine.step import Runner, StepEntry
from hetero_serve_b200.parts import Model

TOL = 2e-5


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
def test_config_is_read_and_written_back(roritar_case):
    arch = architecture_of(roritar_case.config)
    cfg = arch.config_cls.from_dict(roritar_case.config)
    assert arch.name == "Roritar"
    assert arch.config_cls.from_dict(cfg.to_dict()) == cfg
    assert cfg.width == roritar_case.config["width"]


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mixer"].update(blocks=3), "multiple"),
    (lambda c: c["layers"][1].update(type="lstm"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors(change, message):
    cfg = copy.deepcopy(rc.CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).config_cls.from_dict(cfg)


def test_every_pass_of_a_looped_layer_has_its_own_cache_or_state(roritar_cases):
    case = roritar_cases["case_a"]                  # layers 1, 2 run three times
    arch = architecture_of(case.config)
    cfg = arch.config_cls.from_dict(case.config)
    assert cfg.layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3] == plain_roritar.layer_runs(case.config)
    model = Model(arch.build_spec(cfg))
    token_groups = {(g.kv_heads, g.head_dim, g.window, g.stride): len(g.entries)
                    for g in model.cache_groups}
    # rows [key | value]: one plane; per token for max(window, block) positions, and one row per
    # block for the whole sequence in a companion group
    assert token_groups == {(2, 40, 21, 1): 1, (3, 26, 34, 1): 3,
                            (2, 40, 0, 5): 1, (3, 26, 0, 3): 3}
    assert sorted(model.state_shapes.values()) == sorted([(40 * 4,)] * 3 + [(36 * 3,)])
    names = set(model.tensor_requests())
    assert "l2.norm2" not in names and "l2.norm1b" in names and "l1.mlp.act" in names
    assert model.spec.max_positions is None


def test_a_window_shorter_than_a_block_keeps_the_block(roritar_cases):
    case = roritar_cases["case_b"]                  # window 1 with blocks of 4
    arch = architecture_of(case.config)
    model = Model(arch.build_spec(arch.config_cls.from_dict(case.config)))
    assert sorted((g.window, g.stride) for g in model.cache_groups) == \
        [(0, 1), (0, 4), (4, 1), (9, 1)]


# -- the plain implementation's own sanity ----------------------------------------------------
def test_plain_prefix_property(roritar_case):
    toks = roritar_case.tokens(70, 5)
    full, part = roritar_case.logits(toks), roritar_case.logits(toks[:23])
    assert (full[:23] - part).abs().max() < 1e-9


def test_plain_visibility_of_one_key(roritar_planted):
    """The marked key counts inside the window and again once its block lies wholly behind
    the window; between the two it is not seen at all."""
    case = roritar_planted
    m = case.config["layers"][0]["mixer"]
    size, P = m["mask"]["size"], m["mask"]["pool"]
    at = 5
    seen_from = (at // P) * P + P - 1 + size        # first query position that sees the block
    for i in range(at + 1, at + 40):
        t = rc.planted_tokens(case, at, i + 1, 3)
        blank = list(t)
        blank[at] = rc.MARK + 1
        change = float((case.logits(t)[-1] - case.logits(blank)[-1]).abs().max())
        if i - at < size or i >= seen_from:
            assert change > 1.0, i
        else:
            assert change == 0.0, i


def test_plain_recurrence_is_a_decaying_sum():
    """One channel, gates forced open: S_t = a S_(t-1) + sqrt(1 - a^2) u_t with a fixed a."""
    T = 6
    w = {"m.y": torch.zeros(1, 1), "m.y.b": torch.tensor([50.0]),      # gelu(50) = 50
         "m.x": torch.ones(1, 1), "m.x.b": torch.zeros(1),
         "m.conv": torch.tensor([[0.0, 1.0]]), "m.conv.b": torch.zeros(1),
         "m.ra": torch.zeros(1, 1, 1), "m.ra.b": torch.tensor([[40.0]]),  # r = 1
         "m.ri": torch.zeros(1, 1, 1), "m.ri.b": torch.tensor([[40.0]]),  # i = 1
         "m.lam": torch.tensor([0.0]), "m.o": torch.ones(1, 1)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    out = plain_roritar.rglru(h, w, "m.", {"blocks": 1})[:, 0] / 50.0
    a = torch.exp(-8.0 * torch.log(torch.tensor(2.0, dtype=torch.float64)))
    S, want = 0.0, []
    for t in range(T):
        S = a * S + torch.sqrt(1 - a * a) * h[t, 0]
        want.append(float(S))
    assert (out - torch.tensor(want, dtype=torch.float64)).abs().max() < 1e-12


def test_plain_activation_and_norm():
    z = torch.tensor([-2.0, 0.0, 1.5], dtype=torch.float64)
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    sp = lambda v: float(torch.log1p(torch.exp(v)))
    got = plain_roritar.xielu(z, p, q)
    assert abs(float(got[2]) - (sp(p) * 2.25 + 0.75)) < 1e-12
    assert abs(float(got[0]) - ((0.5 + sp(q)) * (float(torch.exp(z[0])) - 1 + 2) - 1)) < 1e-12
    assert float(got[1]) == 0.0
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    n = plain_roritar.layer_norm(x, torch.ones(4, dtype=torch.float64), 0.0)
    assert abs(float(n.mean())) < 1e-12 and abs(float((n * n).mean()) - 1.0) < 1e-12


# -- the engine with plain kernels -------------------------------------------------------------
@pytest.mark.parametrize("driver", ["whole", "tail", "portions"])
def test_cuts_agree_with_the_plain_model(roritar_case, tmp_path, driver):
    reqs = {f"r{i}": roritar_case.tokens(n, 50 + i) for i, n in enumerate((1, 2, 19, 83))}
    if driver == "whole":
        steps, index = traces.whole(reqs)
    elif driver == "tail":
        steps, index = traces.tail_one_by_one(reqs, tail=45)
    else:
        steps, index = traces.portions(reqs, sizes=(7, 2, 16, 3, 2, 5, 21))
    out = _replay(roritar_case, steps, tmp_path, max_tokens=128)
    err, where = _worst(roritar_case, out, index, reqs)
    assert err < TOL, (err, where)


def test_mixed_batches_reuse_pages_and_slots(roritar_case, tmp_path):
    reqs = {f"r{i}": roritar_case.tokens(n, 70 + i) for i, n in
            enumerate((47, 5, 18, 66, 3, 26))}
    steps, index, peak = traces.mixed(reqs, seed=3, max_live=3, sizes=(1, 2, 5, 1, 17, 3, 1, 9))
    out = _replay(roritar_case, steps, tmp_path, max_tokens=peak, max_requests=3)
    err, where = _worst(roritar_case, out, index, reqs)
    assert sum(len(v) for v in index.values()) > 20 and err < TOL, (err, where)


def test_a_slot_is_cleared_for_its_next_owner(roritar_cases):
    case = roritar_cases["case_a"]
    rn = _runner(case, pages=8)
    a, b = case.tokens(50, 1), case.tokens(29, 2)
    rn.step([StepEntry("a", a)])
    rn.close("a")
    rn.step([StepEntry("b", b[:2])])               # shorter than the convolution's history
    rn.step([StepEntry("b", b[2:11])])
    res = rn.step([StepEntry("b", b[11:], want=[17])])
    assert (res.logits[0].double() - case.logits(b)[28]).abs().max() < TOL
    rn.manager.check()


def test_pages_behind_the_window_are_given_back(roritar_cases):
    """A request far longer than the token pool holds runs in portions: token rows behind the
    window go back to the pool as it advances, the rows of the blocks stay."""
    case = roritar_cases["case_a"]                  # windows 21 and 34, blocks of 5 and 3
    rn = _runner(case, pages=12)
    toks = case.tokens(230, 17)
    want, at = case.logits(toks), 0
    for n in (20, 13, 2, 19, 1, 1, 20, 7, 20, 20, 3, 20, 1, 20, 20, 20, 2, 20, 1):
        res = rn.step([StepEntry("a", toks[at:at + n], want=[n - 1])])
        assert (res.logits[0].double() - want[at + n - 1]).abs().max() < TOL, at
        at += n
        token_groups = [g for g, grp in enumerate(rn.model.cache_groups) if grp.stride == 1]
        assert all(12 - rn.manager.pages_free(g) <= 5 for g in token_groups)
    assert at == 230
    rn.manager.check()
    rn.close("a")
    assert all(rn.manager.pages_free(g) == rn.manager.pools[g].num_pages
               for g in range(len(rn.model.cache_groups)))


@pytest.mark.parametrize("how", ["whole", "alone", "portions"])
def test_the_edges_of_window_and_blocks(roritar_planted, how):
    """One key that takes nearly all of the softmax when it is visible, asked for from every
    distance around the window's edge and the block's first sight, and from far away: in a
    prompt, decoded alone, and at the start or end of a portion of two tokens."""
    case = roritar_planted
    for at in (0, 5, 15, 16):                       # also a page's last and first row
        for d in (1, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 31, 32, 33, 150):
            t = rc.planted_tokens(case, at, at + d + 1, 100 + d)
            rn = _runner(case, pages=12)
            n = len(t)
            if how == "whole":
                res = rn.step([StepEntry("a", t, want=[n - 1])])
            elif how == "alone":
                if n > 1:
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


def test_long_decoding(roritar_cases):
    case = roritar_cases["case_b"]
    t = case.tokens(150, 9)
    rn = _runner(case, pages=12)
    rn.step([StepEntry("d", t[:3])])
    want = case.logits(t)
    for i in range(3, 150):
        res = rn.step([StepEntry("d", [t[i]], want=[0])])
        assert (res.logits[0].double() - want[i]).abs().max() < TOL, i


def test_the_parts_in_another_arrangement(roritar_cases):
    """The new mixers under norms BEFORE the sublayers only (x += mixer(norm1(x)); x +=
    ff(norm2(x))): they then add into the stream themselves."""
    import dataclasses
    from hetero_serve_b200.parts.spec import LayerCall, LayerSpec
    case = roritar_cases["case_a"]
    arch = architecture_of(case.config)
    spec = arch.build_spec(arch.config_cls.from_dict(case.config))
    layers = []
    for i in (0, 1):
        parts = {k: v for k, v in spec.layers[i].parts.items() if k not in ("norm1b", "norm2b")}
        layers.append(LayerSpec("pre_norm", parts))
    spec = dataclasses.replace(spec, layers=tuple(layers), schedule=(LayerCall(0), LayerCall(1)))
    model = Model(spec)
    model.bind({n: case.raw[n] for n in model.tensor_requests()}, torch.float32, "cpu")
    rn = Runner(model, num_pages=6, page_size=16, max_requests=1, dtype=torch.float32,
                device="cpu", ops=plain_ops.PlainOps())
    toks = case.tokens(60, 3)
    rn.step([StepEntry("a", toks[:13])])
    got = rn.step([StepEntry("a", toks[13:], want=[0, 46])]).logits.double()
    w, cfg = case.plain, case.config
    eps = cfg["norm"]["eps"]
    P = plain_roritar
    x = w["embed"][torch.tensor(toks)]
    x = x + P.pooled_window_attention(P.layer_norm(x, w["l0.norm1"], eps), w, "l0.mix.",
                                      cfg["layers"][0]["mixer"], eps)
    x = x + P.dense_feed_forward(P.layer_norm(x, w["l0.norm2"], eps), w, "l0.mlp.")
    x = x + P.rglru(P.layer_norm(x, w["l1.norm1"], eps), w, "l1.mix.", cfg["layers"][1]["mixer"])
    x = x + P.dense_feed_forward(P.layer_norm(x, w["l1.norm2"], eps), w, "l1.mlp.")
    z = P.layer_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg["logit_scale"]
    want = cfg["logit_softcap"] * torch.tanh(z / cfg["logit_softcap"])
    assert (got - want[[13, 59]]).abs().max() < TOL
