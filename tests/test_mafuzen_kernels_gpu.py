"""The kernels of the Mafuzen parts, each mechanism alone, against the plain implementation's
function of the same mechanism (tests/plain_mafuzen.py, float64 on the CPU): attention with a
distance slope, a window and kept first tokens over a paged cache whose pages are in no order,
retention with turned and scaled rows, time mixing with its blends and decays, head norms with
a gate, tables indexed by the token id, and experts without a gate."""

import math

import pytest
import torch

import plain_mafuzen as P

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


# -- attention -----------------------------------------------------------------------------------
def _plain_attention(rows, H, G, D, V, q_off, k_off, v_off, qk_norm, eps, scale, slopes, window,
                     keep, g_off, out_scale):
    T = rows.shape[0]
    r = rows.double()
    q = r[:, q_off:q_off + H * D].view(T, H, D)
    k = r[:, k_off:k_off + G * D].view(T, G, D)
    v = k if v_off is None else r[:, v_off:v_off + G * V].view(T, G, V)
    if qk_norm:
        q, k = P.unit_rms(q, eps), P.unit_rms(k, eps)
    o = P.softmax_attention(q, k, v, scale, slopes, window, keep).reshape(T, H * V)
    if g_off is not None:
        o = o * torch.sigmoid(r[:, g_off:g_off + H * V])
    return o * out_scale


@pytest.mark.parametrize("dtype, tol", [(F32, 1e-5), (BF16, 3e-2)])
@pytest.mark.parametrize("H, G, D, V, window, keep, slope, norm, own_v, gate", [
    (4, 2, 24, 16, 21, 3, True, False, True, False), (1, 1, 32, 32, 9, 0, False, True, False, True),
    (2, 2, 8, 6, 1, 2, True, True, True, True), (8, 2, 64, 64, 48, 16, False, True, False, True),
    (4, 4, 128, 128, 40, 7, True, False, True, False), (3, 1, 20, 258, 0, 0, True, False, True, False),
    (4, 1, 48, 48, 70, 6, False, True, False, True), (4, 2, 96, 96, 0, 0, True, False, True, False),
    (2, 1, 64, 128, 33, 40, True, False, True, True), (2, 2, 32, 32, 17, 17, False, False, False, False)])
@pytest.mark.parametrize("planned", [False, True])
def test_span_attention(ops, dtype, tol, H, G, D, V, window, keep, slope, norm, own_v, gate,
                        planned):
    """Two requests whose pages are scattered over the pool, in portions that end inside pages
    and windows; then single tokens.  Every position is compared.  With the step's work lists the
    portions of a bfloat16 cache run as tiles on the tensor cores where the sizes allow it.  The
    pages that neither the window nor the kept first tokens reach are taken out of the table:
    nothing may look them up.  Unused rows of the pool are NaN."""
    eps, page, scale, out_scale = 1e-5, 16, 1.3 / math.sqrt(D), 0.7
    q_off, k_off = 8, 8 + H * D
    v_off = k_off + G * D if own_v else None
    g_off = (k_off + G * D + (G * V if own_v else 0)) if gate else None
    width = 8 + H * D + G * D + (G * V if own_v else 0) + (H * V if gate else 0) + 8
    rows = {"a": rnd(150, width, seed=41), "b": rnd(77, width, seed=42)}
    slopes = [P.slope_of(h, H) * 3 for h in range(H)] if slope else None
    want = {r: _plain_attention(x, H, G, D, V, q_off, k_off, v_off, norm, eps, scale, slopes,
                                window, keep, g_off, out_scale) for r, x in rows.items()}
    if dtype == BF16:      # what the cache rounds: compare with keys and values rounded alike
        tol = 5e-2
    n_pages, max_pages = 24, 10
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(43)).tolist()
    table = torch.full((2, max_pages), -1, dtype=I32)
    table[0], table[1] = torch.tensor(perm[:10]), torch.tensor(perm[10:20])
    table = dev(table)
    pool = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    sl = dev(torch.tensor(slopes, dtype=F32)) if slope else None
    plan = [[("a", 37)], [("a", 2), ("b", 30)], [("b", 1), ("a", 58)], [("a", 1), ("b", 1)],
            [("b", 45), ("a", 1)], [("a", 1)]] + [[("a", 1)]] * 17 + [[("a", 33)]]
    fed = {"a": 0, "b": 0}
    idx = {"a": 0, "b": 1}
    for step in plan:
        proj = dev(torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step]))
        T = proj.shape[0]
        tok_pos = ints(p for r, k in step for p in range(fed[r], fed[r] + k))
        tok_req = ints(row for row, (r, k) in enumerate(step) for _ in range(k))
        tab = table[[idx[r] for r, k in step]].contiguous()
        q = torch.zeros(T, H * D, device=DEV)
        sizes = dict(n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, page_size=page, status=status)
        ops.span_prepare(q, pool, proj, tab, tok_pos, tok_req, q_off=q_off, k_off=k_off,
                         v_off=v_off, qk_norm=norm, eps=eps, writes=True, **sizes)
        if window:
            for row, (r, k) in enumerate(step):
                lo = max(0, fed[r] - window + 1) // page
                tab[row, -(-keep // page):lo] = -1
        out = torch.full((T, H * V), float("nan"), dtype=dtype, device=DEV)
        work = ops.make_plan([(row, row, fed[r], k) for row, (r, k) in enumerate(step)], T, page) \
            if planned else None
        before = ops.launches
        ops.span_attention(out, q, pool, tab, tok_pos, tok_req, scale=scale, slopes=sl,
                           window=window, keep_first=keep, gate=proj if gate else None,
                           gate_offset=g_off or 0, out_scale=out_scale, plan=work, **sizes)
        if planned and work.tile_cap and work.decode_cap:      # tiles and single tokens apart?
            tiled = dtype == BF16 and (D, V) in ((32, 32), (48, 48), (64, 64), (96, 96),
                                                 (128, 128), (64, 128), (128, 64))
            assert ops.launches - before == (2 if tiled else 1)
        at = 0
        for r, k in step:
            close(out[at:at + k], want[r][fed[r]:fed[r] + k], tol)
            fed[r] += k
            at += k
    assert int(status.item()) == 0 and fed == {"a": 150, "b": 77}


@pytest.mark.parametrize("dtype, tol", [(F32, 1e-5), (BF16, 3e-2)])
@pytest.mark.parametrize("window, keep", [(0, 0), (300, 5), (64, 64)])
def test_one_key_among_hundreds(ops, dtype, tol, window, keep):
    """A query at position 700 whose score with ONE key is far above all others, for the key
    at the first position, at page borders, at the window's edge on both sides and one position
    back: every warp of the token's block has rounds, and a lost or doubled key shows."""
    H, G, D, V, page, n = 2, 1, 16, 24, 16, 701
    base = rnd(n, (H + G) * D + G * V, seed=5, std=0.3)
    n_pages = -(-n // page)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6)).tolist()
    table = dev(torch.tensor([perm], dtype=I32))
    status = torch.zeros(1, dtype=I32, device=DEV)
    sizes = dict(n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, page_size=page, status=status)
    first = n - window if window else 0
    for at in (0, keep - 1, keep, 15, 16, first - 1, first, first + 1, 699, 700):
        if at < 0:
            continue
        rows = base.clone()
        rows[700, :H * D] = 0.0
        rows[700, D - 1], rows[700, 2 * D - 1] = 9.0, 9.0
        rows[at, H * D + D - 1] = 9.0
        want = _plain_attention(rows, H, G, D, V, 0, H * D, (H + G) * D, False, 0.0, 0.5,
                                [0.01, 0.0], window, keep, None, 1.0)[700]
        pool = torch.full((n_pages, G, page, D + V), float("nan"), dtype=dtype, device=DEV)
        proj = dev(rows)
        q = torch.zeros(n, H * D, device=DEV)
        ops.span_prepare(q, pool, proj, table.expand(1, -1).contiguous(), ints(range(n)),
                         ints([0] * n), q_off=0, k_off=H * D, v_off=(H + G) * D, qk_norm=False,
                         eps=0.0, writes=True, **sizes)
        out = torch.zeros(1, H * V, dtype=dtype, device=DEV)
        ops.span_attention(out, q[700:].contiguous(), pool, table, ints([700]), ints([0]),
                           scale=0.5, slopes=dev(torch.tensor([0.01, 0.0])), window=window,
                           keep_first=keep, gate=None, gate_offset=0, out_scale=1.0, **sizes)
        close(out[0], want, tol)
    assert int(status.item()) == 0


def test_a_reader_has_no_key_columns_and_a_missing_page_is_reported(ops):
    H, G, D, V, page = 2, 1, 8, 8, 16
    proj = dev(rnd(3, H * D, seed=1))                 # only queries
    pool = torch.zeros(2, G, page, D + V, device=DEV)
    status = torch.zeros(1, dtype=I32, device=DEV)
    table = dev(torch.tensor([[1, -1]], dtype=I32))
    q = torch.zeros(3, H * D, device=DEV)
    sizes = dict(n_heads=H, n_kv_heads=G, head_dim=D, value_dim=V, page_size=page, status=status)
    ops.span_prepare(q, pool, proj, table, ints([14, 15, 16]), ints([0, 0, 0]), q_off=0,
                     k_off=None, v_off=None, qk_norm=False, eps=0.0, writes=False, **sizes)
    assert torch.equal(q, proj) and int(status.item()) == 0 and float(pool.abs().sum()) == 0.0
    out = torch.zeros(3, H * V, device=DEV)
    ops.span_attention(out, q, pool, table, ints([14, 15, 16]), ints([0, 0, 0]), scale=1.0,
                       slopes=None, window=0, keep_first=0, gate=None, gate_offset=0,
                       out_scale=1.0, **sizes)
    assert int(status.item()) == 4                    # position 16 lies on a page that is not there


# -- retention -----------------------------------------------------------------------------------
def _selectors(sizes):
    """Matrices that cut a row [a | b | ...] into its parts: W_a x = the columns of a."""
    total, out, at = sum(sizes), [], 0
    for n in sizes:
        m = torch.zeros(n, total, dtype=F64)
        m[torch.arange(n), at + torch.arange(n)] = 1.0
        out.append(m)
        at += n
    return out


@pytest.mark.parametrize("H, D, V, rot", [(3, 12, 20, 8), (1, 8, 8, 0), (2, 64, 64, 64),
                                          (2, 16, 8, 16), (1, 200, 5, 100), (2, 128, 32, 2)])
def test_retention_in_portions_and_batches(ops, H, D, V, rot):
    """Rows [q | k | v | g] of two requests through the recurrence, the head norm and the gate,
    in portions of 1 to 70 tokens in two slots, against the plain mechanism on the whole."""
    eps, base = 1e-5, 300.0
    hd, hv = H * D, H * V
    decay = [1.0 - 0.5 ** (h + 2) for h in range(H)]
    sel = _selectors([hd, hd, hv, hv])
    w = {"m.q": sel[0], "m.k": sel[1], "m.v": sel[2], "m.g": sel[3],
         "m.o": torch.eye(hv, dtype=F64)}
    m = {"heads": H, "dim": D, "vdim": V, "decay": decay, "rot": {"base": base, "dims": rot}}
    rows = {"a": rnd(160, 2 * hd + 2 * hv, seed=11), "b": rnd(90, 2 * hd + 2 * hv, seed=12)}
    want = {r: P.retention(m, w, "m.", x.double(), eps) for r, x in rows.items()}
    state = torch.full((3, hd * V), float("nan"), device=DEV)
    slot = {"a": 2, "b": 0}
    state[2], state[0] = 0.0, 0.0
    freq = dev((base ** (-2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1))).float()) \
        if rot else None
    dec = dev(torch.tensor(decay, dtype=F32))
    plan = [[("a", 3)], [("a", 1), ("b", 2)], [("b", 70), ("a", 1)], [("a", 66)], [("a", 1), ("b", 1)],
            [("b", 17), ("a", 19)], [("a", 70)]]
    fed = {"a": 0, "b": 0}
    for step in plan:
        proj = dev(torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step]))
        T = proj.shape[0]
        starts, at = [], 0
        for r, k in step:
            starts.append(at)
            at += k
        o = torch.zeros(T, hv, device=DEV)
        ops.lightning_recurrence(o, state, proj, dec, ints(starts), ints(k for _, k in step),
                                 ints(slot[r] for r, _ in step), q_off=0, k_off=hd, v_off=2 * hd,
                                 heads=H, dim=D, vdim=V, act="none",
                                 tok_pos=ints(p for r, k in step for p in range(fed[r], fed[r] + k)),
                                 freq=freq, rot_dims=rot, k_scale=D ** -0.5)
        out = torch.zeros(T, hv, device=DEV)
        ops.head_norm_gate(out, o, None, proj, gate_offset=2 * hd + hv, heads=H, dim=V, eps=eps,
                           gate_act="silu")
        at = 0
        for r, k in step:
            close(out[at:at + k], want[r][fed[r]:fed[r] + k], 2e-4)
            fed[r] += k
            at += k
    assert bool(torch.isnan(state[1]).all())          # the slot nobody owns was not touched


def test_retention_gives_the_same_bits_however_the_rows_arrive(ops):
    """One portion of 150 tokens (rows turned and scaled by a pass of their own) against the
    same tokens one by one (turned while they are staged)."""
    H, D, V, rot = 2, 32, 16, 24
    hd, hv = H * D, H * V
    proj = dev(rnd(150, 2 * hd + hv, seed=3))
    dec, freq = dev(torch.tensor([0.9, 0.99])), dev(rnd(rot // 2, seed=4).abs())
    kw = dict(q_off=0, k_off=hd, v_off=2 * hd, heads=H, dim=D, vdim=V, act="none", freq=freq,
              rot_dims=rot, k_scale=0.3)
    s1, s2 = torch.zeros(1, hd * V, device=DEV), torch.zeros(1, hd * V, device=DEV)
    o1, o2 = torch.zeros(150, hv, device=DEV), torch.zeros(150, hv, device=DEV)
    ops.lightning_recurrence(o1, s1, proj, dec, ints([0]), ints([150]), ints([0]),
                             tok_pos=ints(range(150)), **kw)
    for t in range(150):
        ops.lightning_recurrence(o2[t:t + 1], s2, proj[t:t + 1], dec, ints([0]), ints([1]),
                                 ints([0]), tok_pos=ints([t]), **kw)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


# -- time mixing ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype, tol", [(F32, 1e-6), (BF16, 1e-2)])
def test_token_blends_in_portions(ops, dtype, tol):
    W, S = 70, 5
    mu = rnd(S, W, seed=1).abs()
    rows = {"a": rnd(40, W, seed=2).to(dtype), "b": rnd(9, W, seed=3).to(dtype)}
    state = torch.zeros(2, 33 + W, device=DEV)
    state[:, :33] = 7.0
    plan = [[("a", 1)], [("a", 5), ("b", 1)], [("b", 2), ("a", 1)], [("a", 33), ("b", 6)]]
    fed = {"a": 0, "b": 0}
    slot = {"a": 1, "b": 0}
    for step in plan:
        x = dev(torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step]))
        T = x.shape[0]
        starts, at = [], 0
        for r, k in step:
            starts.append(at)
            at += k
        out = torch.zeros(S, T, W, dtype=dtype, device=DEV)
        ops.token_shift_mix(out, x, dev(mu), state,
                            ints(row for row, (r, k) in enumerate(step) for _ in range(k)),
                            ints(starts), ints(k for _, k in step), ints(slot[r] for r, _ in step),
                            state_offset=33)
        at = 0
        for r, k in step:
            full = rows[r].double()
            prev = torch.cat([torch.zeros(1, W, dtype=F64), full[:-1]])
            for s in range(S):
                want = full + (prev - full) * mu[s].double()
                close(out[s, at:at + k], want[fed[r]:fed[r] + k], tol)
            fed[r] += k
            at += k
    assert float((state[:, :33] - 7.0).abs().max()) == 0.0
    assert torch.equal(state[1, 33:].cpu(), rows["a"][-1].float())


@pytest.mark.parametrize("H, D, rank", [(3, 12, 5), (1, 8, 1), (2, 64, 16), (2, 4, 3), (1, 200, 8),
                                        (2, 128, 32)])
def test_time_mixing_in_portions_and_batches(ops, H, D, rank):
    """Rows [r | k | v | g | inner decay row] through the decay, the recurrence with its bonus,
    the head norm with weight and gate, in portions in two slots against the plain mechanism on
    the whole (all blends 0: every stream reads the row itself)."""
    hd, eps = H * D, 1e-5
    sel = _selectors([hd, hd, hd, hd, rank])
    W = 4 * hd + rank
    w = {f"m.mu.{s}": torch.zeros(W, dtype=F64) for s in "rkvgw"}
    w.update({"m.r": sel[0], "m.k": sel[1], "m.v": sel[2], "m.g": sel[3], "m.w1": sel[4] * 50.0,
              "m.w2": rnd(hd, rank, seed=1, std=0.8).double(), "m.w0": rnd(hd, seed=2).double() - 1.5,
              "m.u": rnd(H, D, seed=3).double(), "m.norm": rnd(hd, seed=4).double() + 1.0,
              "m.o": torch.eye(hd, dtype=F64)})
    rows = {"a": rnd(120, W, seed=11, std=0.7), "b": rnd(50, W, seed=12, std=0.7)}
    for x in rows.values():
        x[:, 4 * hd:] *= 0.02                  # tanh(50 * 0.02 * n): not saturated
    want = {r: P.time_mix({"heads": H, "dim": D}, w, "m.", x.double(), eps) for r, x in rows.items()}
    state = torch.zeros(2, hd * D + 3, device=DEV)
    slot = {"a": 1, "b": 0}
    w2, w0, u, nw = dev(w["m.w2"].float().t(), w["m.w0"].float(), w["m.u"].float().reshape(-1),
                        w["m.norm"].float())
    plan = [[("a", 3)], [("a", 1), ("b", 2)], [("b", 40), ("a", 1)], [("a", 66)], [("a", 1), ("b", 1)],
            [("b", 7), ("a", 48)]]
    fed = {"a": 0, "b": 0}
    for step in plan:
        x = dev(torch.cat([rows[r][fed[r]:fed[r] + k] for r, k in step]))
        T = x.shape[0]
        starts, at = [], 0
        for r, k in step:
            starts.append(at)
            at += k
        parts = [x[:, i * hd:(i + 1) * hd].contiguous() for i in range(4)]
        decay = torch.zeros(T, hd, device=DEV)
        ops.timemix_decay(decay, (x[:, 4 * hd:] * 50.0).contiguous(), w2, w0)
        o = torch.zeros(T, hd, device=DEV)
        ops.timemix_recurrence(o, state, parts[0], parts[1], parts[2], decay, u, ints(starts),
                               ints(k for _, k in step), ints(slot[r] for r, _ in step), heads=H,
                               dim=D)
        out = torch.zeros(T, hd, device=DEV)
        ops.head_norm_gate(out, o, nw, parts[3], gate_offset=0, heads=H, dim=D, eps=eps,
                           gate_act="silu", out_scale=1.0)
        at = 0
        for r, k in step:
            close(out[at:at + k], want[r][fed[r]:fed[r] + k], 3e-4)
            fed[r] += k
            at += k
    assert float(state[:, hd * D:].abs().max()) == 0.0        # what lies behind S is not its


def test_head_norm_and_gates(ops):
    o, g = rnd(9, 3 * 10, seed=1, std=4.0), rnd(9, 40, seed=2)
    wt = rnd(30, seed=3) + 1.0
    n = P.unit_rms(o.double().view(9, 3, 10), 1e-3).reshape(9, 30)
    for dtype, tol in ((F32, 1e-6), (BF16, 1e-2)):
        out = torch.zeros(9, 30, dtype=dtype, device=DEV)
        ops.head_norm_gate(out, dev(o), dev(wt), dev(g), gate_offset=7, heads=3, dim=10, eps=1e-3,
                           gate_act="sigmoid", out_scale=0.5)
        close(out, n * wt.double() * torch.sigmoid(g.double()[:, 7:37]) * 0.5, tol)
        ops.head_norm_gate(out, dev(o), None, None, gate_offset=0, heads=3, dim=10, eps=1e-3)
        close(out, n, tol)


# -- tables indexed by the token id ------------------------------------------------------------------
def test_rows_of_a_table_by_token_id(ops):
    table = rnd(50, 24, seed=1)
    g = rnd(6, 5, seed=2)
    ids, req = ints([3, 49, -2, 0, 7, 7]), ints([0, 0, 1, -1, 2, 2])
    feedback = ints([11, 12, 13])                      # id -2 stands for feedback[1]
    out = torch.zeros(6, 5, device=DEV)
    ops.gather_mul(out, dev(g), dev(table), ids, req, col_offset=10, feedback=feedback)
    want = g.double() * table.double()[[3, 49, 12, 0, 7, 7], 10:15]
    want[3] = 0.0                                      # a padding row is left alone
    close(out, want, 1e-6)
    experts = torch.randint(0, 6, (50, 2), generator=torch.Generator().manual_seed(3)).to(I32)
    idx, wts = torch.zeros(6, 2, dtype=I32, device=DEV), torch.zeros(6, 2, device=DEV)
    ops.moe_route_table(idx, wts, dev(experts), ids, req, top=2, feedback=feedback, experts=6)
    rows = [3, 49, 12, None, 7, 7]
    for t, r in enumerate(rows):
        if r is not None:
            assert idx[t].tolist() == experts[r].tolist() and wts[t].tolist() == [0.5, 0.5]
    assert int(ops.status.item()) == 0
    ops.gather_mul(out, dev(g), dev(table), ints([50, 1, 1, 1, 1, 1]), req, col_offset=10)
    assert int(ops.status.item()) == 1                 # a token outside the table is reported
    ops.status.zero_()


@pytest.mark.parametrize("dtype, tol, T", [(F32, 1e-5, 9), (BF16, 3e-2, 9), (BF16, 3e-2, 300)])
def test_experts_without_a_gate(ops, dtype, tol, T):
    """Few tokens: a product per pair; many in bfloat16: sorted tiles on the tensor cores."""
    W, ff, E, top, vocab = 64, 96, 5, 2, 40
    w = {f"m.e{e}.up": rnd(ff, W, seed=10 + e, std=0.2).to(dtype).double() for e in range(E)}
    w.update({f"m.e{e}.down": rnd(W, ff, seed=20 + e, std=0.2).to(dtype).double() for e in range(E)})
    table = torch.rand(vocab, E, generator=torch.Generator().manual_seed(1)).argsort(1)[:, :top]
    w["m.table"] = table
    toks = torch.randint(0, vocab, (T,), generator=torch.Generator().manual_seed(2)).tolist()
    h = rnd(T, W, seed=3).to(dtype)
    want = P.table_moe({"router": {"top": top}}, w, "m.", h.double(), toks)
    idx, wts = torch.zeros(T, top, dtype=I32, device=DEV), torch.zeros(T, top, device=DEV)
    ops.moe_route_table(idx, wts, dev(table.to(I32)), ints(toks), ints([0] * T), top=top, experts=E)
    x = torch.zeros(T, W, device=DEV)
    y = torch.zeros(T * top, ff, device=DEV)
    up = dev(torch.stack([w[f"m.e{e}.up"] for e in range(E)]).to(dtype))
    down = dev(torch.stack([w[f"m.e{e}.down"] for e in range(E)]).to(dtype))
    ops.moe_experts(x, y, dev(h), None, up, down, idx, wts, ints([0] * T), limit=0.0, act="relu2")
    close(x, want, tol)
