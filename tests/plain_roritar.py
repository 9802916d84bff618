"""A plain, slow implementation of the Roritar decoder, one function per mechanism, written
from the design's equations in float64.  It is the oracle of the tests: it shares no code
with the package, processes a whole sequence at once (the recurrence token by token, the
attention query by query) and keeps no cache.

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
            out[name] = t.clone()
            continue
        if round_to is not None and t.dim() >= 2 and name.rsplit(".", 1)[-1] not in (
                "ra", "ri", "conv"):
            t = t.to(round_to)
        out[name] = t.to(F64)
    return out


# ---------------------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------------------

def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * weight; no bias."""
    d = x - x.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * weight


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = aq * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def turn_halves(v, positions, base, dims, sign=1.0):
    """Rotate the first ``dims`` numbers of every vector: number i is paired with i + dims/2,
    the pair turning by position * base^(-2i/dims).  v: [T, ..., n]; positions: [T]."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = sign * positions.to(F64)[:, None] * f[None, :]                # [T, half]
    while a.dim() < v.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    lo, hi = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


# ---------------------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------------------

def pooled_window_attention(h, w, pre, m, eps):
    """Softmax attention over the last ``mask.size`` positions and, in the same softmax, one
    mean key and mean value for every block of ``mask.pool`` positions that lies wholly before
    the window.  Keys and queries are RMS-normed per head and rotated on their first
    ``rot.dims`` numbers; values are rotated by their own position over all of vdim and the
    head's output is turned back by the query's position."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P = m["mask"]["size"], m["mask"]["pool"]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = (h @ w[pre + "v"].T).view(T, G, V)
    q = turn_halves(rms_norm(q, w[pre + "q.norm"], eps), pos, base, dims)
    k = turn_halves(rms_norm(k, w[pre + "k.norm"], eps), pos, base, dims)
    v = turn_halves(v, pos, base, V)
    nb = T // P
    kp = k[:nb * P].view(nb, P, G, D).mean(1)
    vp = v[:nb * P].view(nb, P, G, V).mean(1)
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        first = max(0, i - size + 1)
        seen = max(0, (i - size + 1) // P)          # blocks b with bP + P - 1 <= i - size
        for hd in range(H):
            g = hd // (H // G)
            keys = torch.cat([kp[:seen, g], k[first:i + 1, g]])
            vals = torch.cat([vp[:seen, g], v[first:i + 1, g]])
            p = torch.softmax((keys @ q[i, hd]) * m["scale"], 0)
            out[i, hd] = p @ vals
    out = turn_halves(out, pos, base, V, sign=-1.0)
    return out.reshape(T, H * V) @ w[pre + "o"].T


def causal_conv(z, weight, bias):
    """Per channel: out[t] = bias + sum_j weight[:, taps-1-j] * z[t-j]; zeros before the start."""
    T, taps = z.shape[0], weight.shape[1]
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out[j:] += z[:T - j] * weight[:, taps - 1 - j]
    return out


def rglru(h, w, pre, m):
    """The recurrent block around a real-gated linear recurrent unit."""
    T = h.shape[0]
    B = m["blocks"]
    y = gelu_tanh(h @ w[pre + "y"].T + w[pre + "y.b"])
    u = causal_conv(h @ w[pre + "x"].T + w[pre + "x.b"], w[pre + "conv"], w[pre + "conv.b"])
    C = u.shape[1]
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ra"]) + w[pre + "ra.b"])
    g = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[pre + "ri"]) + w[pre + "ri.b"])
    r, g = r.reshape(T, C), g.reshape(T, C)
    log_a = -8.0 * r * softplus(w[pre + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * g * u
    S = torch.zeros(C, dtype=F64)
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w[pre + "o"].T


def dense_feed_forward(h, w, pre):
    act = w[pre + "act"]
    return xielu(h @ w[pre + "up"].T, act[0], act[1]) @ w[pre + "down"].T


# ---------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------

def layer_runs(cfg):
    """Indices of the layers in the order they run: a looped stretch is repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0; with ``return_layers`` also the
    residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids]
    layers = []
    for i in layer_runs(cfg):
        layer, pre = cfg["layers"][i], f"l{i}."
        hn = layer_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "attention":
            y = pooled_window_attention(hn, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "rglru":
            y = rglru(hn, w, pre + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, w[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = dense_feed_forward(layer_norm(x, w[pre + "norm2"], eps), w, pre + "mlp.")
            x = x + layer_norm(y, w[pre + "norm2b"], eps)
        layers.append(x.clone())
    z = layer_norm(x, w["final.norm"], eps) @ w["embed"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * torch.tanh(z / cap)
    return (z, layers) if return_layers else z
