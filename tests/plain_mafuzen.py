"""A plain, slow implementation of the Mafuzen decoder, one function per mechanism, written
from the design's equations in float64.  It is the oracle of the tests: it shares no code
with the package, processes a whole sequence at once (recurrences token by token, attention
query by query) and keeps no cache.

Notation: ``h`` is a [T, width] block of rows, matrices are stored [out, in] and applied as
``h @ W.T``; ``w`` maps tensor names to float64 tensors and ``pre`` is the prefix of a part's
tensors.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def prepare(raw, round_to=None):
    """float64 copies of the stored tensors; ``round_to`` rounds matrices to that type first,
    as a model bound for it holds them."""
    out = {}
    for name, t in raw.items():
        if not t.dtype.is_floating_point:
            out[name] = t.clone().long()
            continue
        if round_to is not None and t.dim() >= 2 and not name.endswith(".u"):
            t = t.to(round_to)
        out[name] = t.to(F64)
    return out


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------

def layer_norm(x, weight, bias, eps):
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_halves(vec, position, base, dims):
    """The first ``dims`` numbers of ``vec``: number i pairs with i + dims/2; the pair turns by
    position * base^(-2i/dims)."""
    out = vec.clone()
    half = dims // 2
    for i in range(half):
        a = position * base ** (-2.0 * i / dims)
        u, v = vec[i], vec[i + half]
        out[i] = u * math.cos(a) - v * math.sin(a)
        out[i + half] = v * math.cos(a) + u * math.sin(a)
    return out


# ---------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------

def retention(m, w, pre, h, eps):
    """Linear attention with a fixed decay per head, no softmax and no denominator."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    gate = silu(h @ w[pre + "g"].T)
    rot = m.get("rot")
    decay = m["decay"] if isinstance(m["decay"], (list, tuple)) else [m["decay"]] * H
    o = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            qt, kt = q[t, hd], k[t, hd]
            if rot and rot["dims"]:
                qt = rotate_halves(qt, t, rot["base"], rot["dims"])
                kt = rotate_halves(kt, t, rot["base"], rot["dims"])
            kt = kt * D ** -0.5
            S = decay[hd] * S + torch.outer(kt, v[t, hd])
            o[t, hd] = S.T @ qt
    o = unit_rms(o, eps).reshape(T, H * V)
    return (o * gate) @ w[pre + "o"].T


def visible(i, j, window, keep_first):
    if j > i:
        return False
    return window <= 0 or i - j < window or j < keep_first


def softmax_attention(q, k, v, scale, slopes=None, window=0, keep_first=0):
    """q [T, H, D], k [T, G, D], v [T, G, V]; query i sees the keys j for which
    :func:`visible` holds; score (q . k) * scale - slope_h * (i - j)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        jt = torch.tensor(js)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[jt, g] @ q[i, hd]) * scale
            if slopes is not None:
                s = s - slopes[hd] * (i - jt).to(F64)
            out[i, hd] = torch.softmax(s, 0) @ v[jt, g]
    return out


def slope_of(head, heads):
    return 2.0 ** (-8.0 * (head + 1) / heads)


def attention(m, w, pre, h, kv=None):
    """Grouped softmax attention with a bias of the distance; ``kv`` are another layer's keys
    and values for a layer without projections of its own.  Returns (output, (k, v))."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    if kv is None:
        kv = ((h @ w[pre + "k"].T).view(T, G, D), (h @ w[pre + "v"].T).view(T, G, V))
    slopes = [slope_of(hd, H) for hd in range(H)]
    o = softmax_attention(q, kv[0], kv[1], m["scale"], slopes)
    return o.reshape(T, H * V) @ w[pre + "o"].T, kv


def window_attention(m, w, pre, h, eps):
    """The left half of a parallel mixer: keys double as values, q and k are divided by their
    root mean square per head, a window with kept first tokens, an output gate."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = k
    mask = m.get("mask") or {"size": 0}                 # no mask: every earlier token is seen
    o = softmax_attention(unit_rms(q, eps), unit_rms(k, eps), v, m["scale"], None,
                          mask["size"], mask.get("keep_first", 0))
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (o.reshape(T, H * D) * gate) @ w[pre + "o"].T


def time_mix(m, w, pre, h, eps):
    """The right half of a parallel mixer: a recurrence with a decay per token, head and key
    channel, and a bonus for the current token."""
    T, W = h.shape
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=F64), h[:-1]])

    def mixed(s):
        return h + (prev - h) * w[pre + "mu." + s]
    r = (mixed("r") @ w[pre + "r"].T).view(T, H, D)
    k = (mixed("k") @ w[pre + "k"].T).view(T, H, D)
    v = (mixed("v") @ w[pre + "v"].T).view(T, H, D)
    gate = silu(mixed("g") @ w[pre + "g"].T)
    lw = torch.tanh(mixed("w") @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"]
    decay = torch.exp(-torch.exp(lw)).view(T, H, D)
    u = w[pre + "u"].view(H, D)
    o = torch.zeros(T, H, D, dtype=F64)
    for hd in range(H):
        S = torch.zeros(D, D, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    o = unit_rms(o, eps).reshape(T, H * D) * w[pre + "norm"] * gate
    return o @ w[pre + "o"].T


def parallel(m, w, pre, h, eps):
    left = window_attention(m["left"], w, pre + "left.", h, eps)
    right = time_mix(m["right"], w, pre + "right.", h, eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---------------------------------------------------------------------------------------
# feed-forwards and the token input
# ---------------------------------------------------------------------------------------

def dense_ff(w, pre, h):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def relu2_expert(w, pre, h):
    return torch.relu(h @ w[pre + "up"].T) ** 2 @ w[pre + "down"].T


def table_moe(mlp, w, pre, h, tokens):
    """Every token id has its experts in a table; each weighs 1/top."""
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for e in w[pre + "table"][tok].tolist():
            out[t] += relu2_expert(w, f"{pre}e{e}.", h[t:t + 1])[0] / top
    if mlp.get("shared") is not None:
        out = out + relu2_expert(w, pre + "shared.", h)
    return out


def token_side(cfg, w, i, x, tokens, eps):
    dim = cfg["token_side"]["dim"]
    pre = f"l{i}.side."
    e = w["side.embed"][torch.tensor(tokens)][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ w[pre + "gate"].T) * e
    y = g @ w[pre + "proj"].T
    return unit_rms(y, eps) * w[pre + "norm"]


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------

def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; ``layers_out`` (a list) receives the stream
    after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."

        def ln(name, v):
            return layer_norm(v, w[p + name], w[p + name + ".b"], eps)
        h = ln("norm1", x)
        m = layer["mixer"]
        if layer["type"] == "retention":
            y = retention(m, w, p + "mix.", h, eps)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            y, kept[i] = attention(m, w, p + "mix.", h, kept[src] if src is not None else None)
        elif layer["type"] == "parallel":
            y = parallel(m, w, p + "mix.", h, eps)
        else:
            raise ValueError(layer["type"])
        x = x + ln("norm1b", y)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = ln("norm2", x)
            y = dense_ff(w, p + "mlp.", h) if mlp["kind"] == "dense" else \
                table_moe(mlp, w, p + "mlp.", h, tokens)
            x = x + ln("norm2b", y)
        if cfg.get("token_side"):
            x = x + token_side(cfg, w, i, x, tokens, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return h @ w["embed"].T
