"""The kernels of the Roritar parts, each mechanism alone, against the plain implementation's
function of the same mechanism (tests/plain_roritar.py, float64 on the CPU): layer norms
behind a sublayer, the learned activation, capped logits, the real-gated recurrence with its
short convolution and block-diagonal gates, and attention over a window and pooled blocks
over a paged cache whose pages are in no order."""

import math

import pytest
import torch

import plain_roritar as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, BF16, I32, F64 = torch.float32, torch.bfloat16, torch.int32, torch.float64


@pytest.fixture(scope="module")
def ops():
    from hetero_serve_b200.kernels import CudaOps
    return CudaOps(DEV)


def rnd(*shape, seed=0, std=1.0, dtype=F32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


def dev(*ts):
    out = tuple(t.to(DEV).contiguous() for t in ts)
    return out if len(out) > 1 else out[0]


def ints(v):
    return torch.tensor(list(v), dtype=I32, device=DEV)


def close(got, want, tol):
    want = want.double()
    err = ((got.detach().cpu().double() - want).abs() / (1.0 + want.abs())).max().item()
    assert err <= tol, err


# -- norms, activation, cap ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype, tol", [(F32, 1e-4), (BF16, 2e-2)])
@pytest.mark.parametrize("width", [1, 5, 100, 1030, 5000])
def test_layernorm_add(ops, dtype, tol, width):
    """A large eps so that it shows; rows whose mean is a hundred times their spread, where a
    variance formed as E[y^2] - E[y]^2 would be off by ten times the tolerance."""
    x, y = rnd(7, width, seed=1), rnd(9, width, seed=2, std=0.3) + 30.0
    g, g2 = rnd(width, seed=3) + 1.0, rnd(width, seed=4) + 1.0
    want = x.double() + P.layer_norm(y[:7].double(), g.double(), 1e-3)
    want2 = P.layer_norm(want, g2.double(), 2e-2)
    got = dev(x.clone())
    ops.layernorm_add(got, dev(y), dev(g), None, 1e-3)
    close(got, want, 1e-4)
    got, out = dev(x.clone()), torch.zeros(7, width, dtype=dtype, device=DEV)
    ops.layernorm_add(got, dev(y), dev(g), None, 1e-3, out=out, out_gamma=dev(g2), out_eps=2e-2)
    close(got, want, 1e-4)
    close(out, want2, tol)


@pytest.mark.parametrize("dtype, tol", [(F32, 2e-6), (BF16, 8e-3)])
def test_learned_activation(ops, dtype, tol):
    z = torch.cat([rnd(3, 333, seed=5, std=3.0), torch.tensor([[0.0, -0.0, 1e-8, -1e-8, -30.0, 30.0]
                                                                + [0.5] * 327])])
    for p, q in ((0.3, -0.2), (-4.0, 2.5), (0.0, 0.0)):
        want = P.xielu(z.double(), torch.tensor(p, dtype=F64), torch.tensor(q, dtype=F64))
        out = torch.zeros(4, 333, dtype=dtype, device=DEV)
        ops.learned_act(out, dev(z), "xielu", (p, q))
        close(out, want, tol)


@pytest.mark.parametrize("dtype, M, K, tol", [(F32, 5, 64, 2e-5), (F32, 40, 64, 2e-5), (F32, 300, 66, 2e-5),
                                              (BF16, 3, 64, 4e-2), (BF16, 40, 64, 4e-2),
                                              (BF16, 300, 64, 4e-2), (BF16, 700, 2048, 4e-2)])
def test_learned_activation_behind_a_product(ops, dtype, M, K, tol):
    """The activation as the last step of every linear kernel (few rows, tiles on the CUDA
    cores, tcgen05 with and without a split over the summed index): applied to the float32
    sums, before a residual, with numbers of either sign."""
    for values in ((0.8, -0.3), (-1.5, 2.0)):
        a, w = rnd(M, K, seed=1).to(dtype), rnd(96, K, seed=2, std=2.0 / math.sqrt(K)).to(dtype)
        bias, res = rnd(96, seed=3), rnd(M, 96, seed=4)
        p, q = (torch.tensor(v, dtype=F64) for v in values)
        z = a.double() @ w.double().T
        got = torch.zeros(M, 96, dtype=F32, device=DEV)
        ops.linear(got, dev(a), dev(w), dev(bias), act="xielu", residual=dev(res), act_values=values)
        close(got, P.xielu(z + bias.double(), p, q) + res.double(), tol)
        got2 = torch.zeros(M, 96, dtype=dtype, device=DEV)
        ops.linear(got2, dev(a), dev(w), None, act="xielu", act_values=values)
        close(got2, P.xielu(z, p, q), tol if dtype == F32 else 8e-2)
    with pytest.raises(Exception):
        ops.linear(got2, dev(a), dev(w), None, act="xielu", act_values=(1.0,))


def test_scaled_and_capped_logits(ops):
    z = rnd(5, 777, seed=6, std=40.0)
    for s, cap in ((0.25, 15.0), (1.0, 30.0), (3.0, 0.5)):
        got = dev(z.clone())
        ops.scale_softcap_(got, s, cap)
        close(got, cap * torch.tanh(z.double() * s / cap), 2e-6)


# -- the recurrence -------------------------------------------------------------------------------
def _recurrence_weights(C, B, taps, seed):
    n = C // B
    w = {"m.conv": rnd(C, taps, seed=seed, std=0.5), "m.conv.b": rnd(C, seed=seed + 1, std=0.2),
         "m.ra": rnd(B, n, n, seed=seed + 2, std=1 / math.sqrt(n)), "m.ra.b": rnd(B, n, seed=seed + 3),
         "m.ri": rnd(B, n, n, seed=seed + 4, std=1 / math.sqrt(n)), "m.ri.b": rnd(B, n, seed=seed + 5),
         "m.lam": rnd(C, seed=seed + 6) - 2.0}
    # the oracle's projections pick the two halves of a row [y | x] apart
    eye = torch.eye(C)
    w["m.y"], w["m.x"] = torch.cat([eye, 0 * eye], 1), torch.cat([0 * eye, eye], 1)
    w["m.y.b"] = w["m.x.b"] = torch.zeros(C)
    w["m.o"] = eye
    return w


@pytest.mark.parametrize("dtype, tol", [(F32, 5e-6), (BF16, 1e-2)])
@pytest.mark.parametrize("C, B, taps", [(40, 2, 4), (36, 3, 3), (24, 1, 1), (256, 4, 4), (70, 7, 2),
                                        (1056, 8, 2)])
def test_recurrence_in_portions_and_batches(ops, dtype, tol, C, B, taps):
    """Three requests side by side in slots that are in no order, cut into portions of unequal
    length (one shorter than the convolution's history, one long enough to be scanned in
    segments), one of them in a slot that another request left."""
    w = _recurrence_weights(C, B, taps, 10)
    w64 = {k: v.double() for k, v in w.items()}
    n = C // B
    w_gates = dev(torch.cat([w["m.ra"].transpose(1, 2), w["m.ri"].transpose(1, 2)], 2))
    b_gates = dev(torch.cat([w["m.ra.b"], w["m.ri.b"]], 1).reshape(-1))
    rate = dev(torch.nn.functional.softplus(w["m.lam"].double()).float())
    cw, cb = dev(w["m.conv"]), dev(w["m.conv.b"])
    rows = {"a": rnd(331, 2 * C, seed=20), "b": rnd(12, 2 * C, seed=21), "c": rnd(60, 2 * C, seed=22)}
    want = {r: P.rglru(h.double(), w64, "m.", {"blocks": B}) for r, h in rows.items()}
    slots = {"a": 3, "b": 0, "c": 2}
    state = torch.full((4, C * taps), 7.0, device=DEV)          # what a former owner left
    plan = [[("a", 2), ("b", 1)], [("a", 1), ("b", 5), ("c", 9)], [("a", 300), ("c", 1)],
            [("c", 50), ("b", 6), ("a", 28)]]
    fed = {r: 0 for r in rows}
    for step in plan:
        for r, _ in step:
            if fed[r] == 0:
                state[slots[r]] = 0.0                            # a slot is cleared when taken
        proj = torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step])
        T = proj.shape[0]
        starts, at = [], 0
        for r, k in step:
            starts.append(at)
            at += k
        tok_req = ints(i for i, (_, k) in enumerate(step) for _ in range(k))
        req_start, req_len = ints(starts), ints(k for _, k in step)
        req_slot = ints(slots[r] for r, _ in step)
        proj = dev(proj)
        u = torch.zeros(T, C, device=DEV)
        ops.rglru_conv(u, proj, cw, cb, state, tok_req, req_start, req_slot, x_off=C,
                       channels=C, taps=taps)
        z = torch.zeros(T, 2 * C, device=DEV)
        ops.grouped_linear(z, u, w_gates)
        out = torch.zeros(T, C, dtype=dtype, device=DEV)
        ops.rglru_scan(out, state, u, z, proj, b_gates, rate, req_start, req_len, req_slot,
                       channels=C, blocks=B, taps=taps, decay_scale=8.0, y_off=0, x_off=C)
        for (r, k), s in zip(step, starts):
            close(out[s:s + k], want[r][fed[r]:fed[r] + k], tol)
            fed[r] += k
    assert fed == {r: h.shape[0] for r, h in rows.items()}


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("C, B, taps", [(40, 2, 4), (36, 3, 3), (24, 1, 1), (256, 4, 4), (70, 7, 2),
                                        (512, 2, 4), (1024, 2, 4)])
def test_single_tokens_in_one_launch(ops, dtype, C, B, taps):
    """A step in which every request brings one token: convolution, gates and the state's step
    in one launch give the bits of the three launches (outputs, states and the convolution's
    history), step after step, in slots that are in no order and beside a row of padding."""
    w = _recurrence_weights(C, B, taps, 50)
    w_gates = dev(torch.cat([w["m.ra"].transpose(1, 2), w["m.ri"].transpose(1, 2)], 2))
    b_gates = dev(torch.cat([w["m.ra.b"], w["m.ri.b"]], 1).reshape(-1))
    rate = dev(torch.nn.functional.softplus(w["m.lam"].double()).float())
    cw, cb = dev(w["m.conv"]), dev(w["m.conv.b"])
    state_a = torch.zeros(12, C * taps, device=DEV)
    state_b = torch.zeros(12, C * taps, device=DEV)
    # eleven rows: ten requests (two tiles of tokens) and a row of padding
    tok_req, req_slot = ints(list(range(10)) + [-1]), ints([4, 0, 2, 9, 8, 7, 6, 5, 3, 10])
    req_start, req_len = ints(range(10)), ints([1] * 10)
    kw = dict(channels=C, blocks=B, taps=taps, decay_scale=8.0, y_off=0, x_off=C)
    for i in range(9):
        proj = dev(rnd(11, 2 * C, seed=60 + i))
        u = torch.zeros(11, C, device=DEV)
        ops.rglru_conv(u, proj, cw, cb, state_a, tok_req, req_start, req_slot, x_off=C,
                       channels=C, taps=taps)
        z = torch.zeros(11, 2 * C, device=DEV)
        ops.grouped_linear(z, u, w_gates)
        want = torch.zeros(11, C, dtype=dtype, device=DEV)
        ops.rglru_scan(want, state_a, u, z, proj, b_gates, rate, req_start, req_len, req_slot, **kw)
        got = torch.zeros(11, C, dtype=dtype, device=DEV)
        before = ops.launches
        took = ops.rglru_step(got, state_b, proj, cw, cb, w_gates, b_gates, rate, tok_req,
                              req_slot, **kw)
        if C // B > 256:
            assert not took and ops.launches == before       # a part too large: refused
            return
        assert took and ops.launches == before + 1
        assert torch.equal(got, want) and torch.equal(state_a, state_b), i
    assert float(state_b[4, :C].abs().max()) > 0 and float(state_b[1].abs().max()) == 0 \
        and float(state_b[11].abs().max()) == 0


def test_recurrence_keeps_a_long_memory(ops):
    """A decay close to 1: sqrt(1 - a^2) must keep its digits, and the state of the first token
    still counts after hundreds of steps taken one at a time."""
    C, B, taps = 8, 1, 2
    w = _recurrence_weights(C, B, taps, 30)
    w["m.lam"] = torch.full((C,), -9.0)                        # a = exp(-8 r softplus(-9)): 0.999..
    w64 = {k: v.double() for k, v in w.items()}
    h = rnd(400, 2 * C, seed=31)
    h[0, C:] += 50.0                                           # a large first input
    want = P.rglru(h.double(), w64, "m.", {"blocks": B})
    w_gates = dev(torch.cat([w["m.ra"].transpose(1, 2), w["m.ri"].transpose(1, 2)], 2))
    b_gates = dev(torch.cat([w["m.ra.b"], w["m.ri.b"]], 1).reshape(-1))
    rate = dev(torch.nn.functional.softplus(w["m.lam"].double()).float())
    state = torch.zeros(1, C * taps, device=DEV)
    one, zero = ints([1]), ints([0])
    for t in range(400):
        proj = dev(h[t:t + 1])
        u, z = torch.zeros(1, C, device=DEV), torch.zeros(1, 2 * C, device=DEV)
        ops.rglru_conv(u, proj, dev(w["m.conv"]), dev(w["m.conv.b"]), state, zero, zero, zero,
                       x_off=C, channels=C, taps=taps)
        ops.grouped_linear(z, u, w_gates)
        out = torch.zeros(1, C, device=DEV)
        ops.rglru_scan(out, state, u, z, proj, b_gates, rate, zero, one, zero, channels=C,
                       blocks=B, taps=taps, decay_scale=8.0, y_off=0, x_off=C)
        if t % 50 == 49 or t < 3:
            close(out[0], want[t], 2e-5)
    assert float(want[399].abs().max()) > 1.0                  # the first input is still there


@pytest.mark.parametrize("T, groups, k, n", [(64, 1, 32, 32), (200, 4, 64, 128), (1000, 3, 96, 40)])
def test_block_diagonal_product_in_three_terms(ops, T, groups, k, n):
    """With weights that are bfloat16 numbers, the tensor-core product of a float32 input that
    enters as three bfloat16 terms is the float32 product: it is compared with the float64
    product at float32's resolution, where the one-term product is a hundred times further
    off.  The inputs span six orders of magnitude."""
    a = rnd(T, groups * k, seed=71) * torch.logspace(-3, 3, groups * k)
    w = rnd(groups, k, n, seed=72).to(BF16).float()
    want = torch.einsum("tgk,gkn->tgn", a.double().view(T, groups, k), w.double()).reshape(T, -1)
    size = torch.einsum("tgk,gkn->tgn", a.double().abs().view(T, groups, k),
                        w.double().abs()).reshape(T, -1)
    w_nk = dev(w.transpose(1, 2).contiguous().to(BF16))
    got = torch.full((T, groups * n), float("nan"), device=DEV)
    before = ops.launches
    ops.grouped_linear(got, dev(a), dev(w), w_nk=w_nk, exact=True)
    assert ops.launches == before + 1
    err = ((got.cpu().double() - want).abs() / size).max().item()
    assert err < 3e-7, err
    rough = torch.zeros(T, groups * n, device=DEV)
    ops.grouped_linear(rough, dev(a), dev(w), w_nk=w_nk)
    assert ((rough.cpu().double() - want).abs() / size).max().item() > 30 * err
    plain = torch.zeros(T, groups * n, device=DEV)
    ops.grouped_linear(plain, dev(a), dev(w))                 # the CUDA-core kernel
    assert ((plain.cpu().double() - want).abs() / size).max().item() < 3e-7


# -- attention over a window and pooled blocks ------------------------------------------------------
def _attention_case(H, G, D, V, window, pool, rot, base, scale, seed):
    W = H * D + G * D + G * V
    eye = torch.eye(W)
    w = {"m.q": eye[:H * D], "m.k": eye[H * D:(H + G) * D], "m.v": eye[(H + G) * D:],
         "m.q.norm": rnd(D, seed=seed, std=0.3) + 1.0, "m.k.norm": rnd(D, seed=seed + 1, std=0.3) + 1.0,
         "m.o": torch.eye(H * V)}
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": scale,
         "mask": {"size": window, "pool": pool}, "rot": {"base": base, "dims": rot}}
    return W, w, m


def _frequencies(base, dims):
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64).float()


@pytest.mark.parametrize("dtype, tol", [(F32, 1e-5), (BF16, 3e-2)])
@pytest.mark.parametrize("H, G, D, V, window, pool, rot", [
    (4, 2, 24, 16, 21, 5, 12), (1, 1, 32, 32, 9, 1, 0), (2, 2, 8, 6, 1, 4, 8),
    (8, 2, 64, 64, 48, 16, 32), (4, 4, 128, 96, 40, 8, 128), (3, 1, 20, 258, 17, 3, 4),
    (4, 2, 128, 64, 70, 8, 32), (2, 1, 64, 128, 33, 7, 64), (2, 2, 128, 128, 20, 16, 0)])
@pytest.mark.parametrize("planned", [False, True])
def test_pooled_window_attention(ops, dtype, tol, H, G, D, V, window, pool, rot, planned):
    """Two requests whose pages are scattered over the pool (the second starts in the middle of
    the first's run), in portions that end inside pages, windows and blocks; then single tokens.
    Every position is compared.  With the step's work lists the portions of a bfloat16 cache run
    as tiles on the tensor cores where the sizes allow it.  The pages that neither a window nor
    an unfinished block of the step reaches are taken out of the table: nothing may look them
    up."""
    W, w, m = _attention_case(H, G, D, V, window, pool, rot, 300.0, 1.3 / math.sqrt(D), 40)
    w64 = {k: v.double() for k, v in w.items()}
    eps, page = 1e-5, 16
    rows = {"a": rnd(150, W, seed=41), "b": rnd(77, W, seed=42)}
    if dtype == BF16:
        rows = {r: h.to(BF16).float() for r, h in rows.items()}
    want = {r: P.pooled_window_attention(h.double(), w64, "m.", m, eps) for r, h in rows.items()}
    n_pages, max_pages = 24, 10
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(43)).tolist()
    cperm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(44)).tolist()
    table = torch.full((2, max_pages), -1, dtype=I32)
    ctable = torch.full((2, max_pages), -1, dtype=I32)
    table[0], table[1] = torch.tensor(perm[:10]), torch.tensor(perm[10:20])
    ctable[0], ctable[1] = torch.tensor(cperm[:10]), torch.tensor(cperm[10:20])
    table, ctable = dev(table, ctable)
    fine = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
    coarse = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    fq = dev(_frequencies(300.0, rot)) if rot else None
    fv = dev(_frequencies(300.0, V))
    wq, wk = dev(w["m.q.norm"], w["m.k.norm"])
    plan = [[("a", 37)], [("a", 2), ("b", 30)], [("b", 1), ("a", 58)], [("a", 1), ("b", 1)],
            [("b", 45), ("a", 1)], [("a", 1)]] + [[("a", 1)]] * 17 + [[("a", 33)]]
    fed = {"a": 0, "b": 0}
    idx = {"a": 0, "b": 1}
    for step in plan:
        proj = dev(torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step]))
        T = proj.shape[0]
        tok_pos = ints(p for r, k in step for p in range(fed[r], fed[r] + k))
        tok_req = ints(row for row, (r, k) in enumerate(step) for _ in range(k))
        order = [idx[r] for r, k in step]           # the tables' rows follow the batch
        tab, ctab = table[order].contiguous(), ctable[order].contiguous()
        q = torch.zeros(T, H * D, device=DEV)
        sizes = dict(n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, page_size=page, status=status)
        # single tokens only: the launch that appends also forms the mean of a block it completes
        folded = planned and all(k == 1 for _, k in step)
        extra = dict(coarse_pool=coarse, coarse_table=ctab, block=pool) if folded else {}
        ops.pooled_prepare(q, fine, proj, wq, wk, fq, fv, tab, tok_pos, tok_req, rot_dims=rot,
                           eps=eps, writes=True, **sizes, **extra)
        for row, (r, k) in enumerate(step):
            lo = max(0, min(fed[r] - window + 1, fed[r] // pool * pool))
            tab[row, :lo // page] = -1
        if not folded:
            ops.pooled_means(coarse, ctab, fine, tab, tok_pos, tok_req, n_kv_heads=G, row=D + V,
                             block=pool, page_size=page, status=status)
        out = torch.full((T, H * V), float("nan"), dtype=dtype, device=DEV)
        work = ops.make_plan([(row, row, fed[r], k) for row, (r, k) in enumerate(step)], T, page) \
            if planned else None
        before = ops.launches
        ops.pooled_attention(out, q, fine, tab, coarse, ctab, tok_pos, tok_req, fv,
                             window=window, block=pool, scale=m["scale"], plan=work, **sizes)
        if planned and work.tile_cap and work.decode_cap:      # tiles and single tokens apart?
            tiled = dtype == BF16 and D in (64, 128) and V in (64, 128)
            assert ops.launches - before == (2 if tiled else 1)
        at = 0
        for r, k in step:
            close(out[at:at + k], want[r][fed[r]:fed[r] + k], tol)
            fed[r] += k
            at += k
    assert int(status.item()) == 0 and fed == {"a": 150, "b": 77}


@pytest.mark.parametrize("dtype, tol", [(F32, 1e-5), (BF16, 3e-2)])
@pytest.mark.parametrize("H, G, D, V, window, pool", [(2, 1, 16, 24, 300, 4), (4, 2, 64, 64, 270, 2)])
def test_a_token_with_hundreds_of_keys(ops, dtype, tol, H, G, D, V, window, pool):
    """Positions up to 700 under a window of some hundred keys: a token sees more rows (token
    rows and mean rows) than one round of all the warps of its block takes, so every warp has
    keys, some walk twice, and their shares are joined.  Every position is compared."""
    W, w, m = _attention_case(H, G, D, V, window, pool, 8, 300.0, 1.3 / math.sqrt(D), 70)
    w64 = {k: v.double() for k, v in w.items()}
    eps, page, n = 1e-5, 16, 700
    rows = rnd(n, W, seed=71)
    if dtype == BF16:
        rows = rows.to(BF16).float()
    want = P.pooled_window_attention(rows.double(), w64, "m.", m, eps)
    n_pages = 72
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(72)).tolist()
    table = dev(torch.tensor([perm[:44]], dtype=I32))
    ctable = dev(torch.tensor([perm[44:68]], dtype=I32))
    fine = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
    coarse = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    fq, fv = dev(_frequencies(300.0, 8)), dev(_frequencies(300.0, V))
    wq, wk = dev(w["m.q.norm"], w["m.k.norm"])
    sizes = dict(n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, page_size=page, status=status)
    fed = 0
    for k in (333, 1, 1, 360, 1, 1, 1, 1, 1):
        proj = dev(rows[fed:fed + k])
        tok_pos, tok_req = ints(range(fed, fed + k)), ints([0] * k)
        q = torch.zeros(k, H * D, device=DEV)
        ops.pooled_prepare(q, fine, proj, wq, wk, fq, fv, table, tok_pos, tok_req, rot_dims=8,
                           eps=eps, writes=True, **sizes)
        ops.pooled_means(coarse, ctable, fine, table, tok_pos, tok_req, n_kv_heads=G, row=D + V,
                         block=pool, page_size=page, status=status)
        out = torch.full((k, H * V), float("nan"), dtype=dtype, device=DEV)
        ops.pooled_attention(out, q, fine, table, coarse, ctable, tok_pos, tok_req, fv,
                             window=window, block=pool, scale=m["scale"], plan=None, **sizes)
        close(out, want[fed:fed + k], tol)
        fed += k
    assert int(status.item()) == 0 and fed == n


def test_attention_reports_a_page_that_is_missing(ops):
    """A table without the page of a position: the status word says so, nothing is written
    outside the pool and the launch returns."""
    H = G = 1
    D = V = 8
    fine = torch.zeros(2, G, 16, D + V, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    table = torch.full((1, 2), -1, dtype=I32, device=DEV)
    proj, q = torch.ones(1, 3 * D, device=DEV), torch.zeros(1, D, device=DEV)
    ops.pooled_prepare(q, fine, proj, None, None, None, None, table, ints([3]), ints([0]),
                       n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, rot_dims=0, eps=1e-5,
                       writes=True, page_size=16, status=status)
    assert int(status.item()) != 0 and float(fine.abs().max()) == 0.0
