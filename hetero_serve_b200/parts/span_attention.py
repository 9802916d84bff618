"""Grouped softmax attention over the paged cache with a linear bias of the distance, a sliding
window that keeps the first tokens, unit-RMS queries and keys, keys that double as values, and
an output gate: each a parameter, off by default.

Per token at position i (query head h uses key/value head h // (heads / kv_heads)):

    q = W_q x,  k = W_k x,  v = W_v x  (``values_are_keys``: v = k as projected, no W_v)
    ``qk_norm``: q, k <- q / rms(q), k / rms(k), per head over head_dim, no weight
    score(i, j) = (q_i . k_j) * scale - slope_h * (i - j)            (``slopes``: one per head)
    visible: j <= i and (window == 0 or i - j < window or j < keep_first)
    o_h = softmax(score) v;   ``gate``: o <- o * sigmoid(W_g x), element by element
    out = W_o [o_0 .. o_H-1] * out_scale

The cache keeps one row [key | value] per token and key/value head; with a window the pages
behind it are given back, except those of the first ``keep_first`` positions.  A layer with
``shares_cache`` has no key/value projections: it reads the rows another layer call wrote (the
schedule names the entry) with its own queries.  All projections of x are ONE product with
float32 results; norms, scores, softmax and the gate are float32 in both precisions.
"""

from __future__ import annotations

import torch

from .base import CacheRequest, Mixer, TensorRequest, register_mixer


class SpanAttention(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, prefix: str, slopes=None, window: int = 0,
                 keep_first: int = 0, qk_norm: bool = False, eps: float = 0.0,
                 values_are_keys: bool = False, gate: bool = False, out_scale: float = 1.0,
                 shares_cache: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        if window < 0 or keep_first < 0:
            raise ValueError("window and keep_first are not negative (0: none)")
        if values_are_keys and value_dim != head_dim:
            raise ValueError("keys that double as values have the keys' size")
        if slopes is not None and len(slopes) != n_heads:
            raise ValueError(f"{len(slopes)} slopes for {n_heads} heads")
        if shares_cache and values_are_keys:
            raise ValueError("a layer that reads another's rows has no keys of its own")
        self.width, self.H, self.G = width, n_heads, n_kv_heads
        self.D, self.V = head_dim, value_dim
        self.scale, self.window, self.keep_first = float(scale), int(window), int(keep_first)
        self.slope_values = None if slopes is None else [float(s) for s in slopes]
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.values_are_keys, self.gate = bool(values_are_keys), bool(gate)
        self.out_scale, self.shares_cache, self.p = float(out_scale), bool(shares_cache), prefix

    def tensor_requests(self):
        p, W = self.p, self.width
        req = {p + "q": TensorRequest((self.H * self.D, W), "matrix"),
               p + "o": TensorRequest((W, self.H * self.V), "matrix")}
        if not self.shares_cache:
            req[p + "k"] = TensorRequest((self.G * self.D, W), "matrix")
            if not self.values_are_keys:
                req[p + "v"] = TensorRequest((self.G * self.V, W), "matrix")
        if self.gate:
            req[p + "g"] = TensorRequest((self.H * self.V, W), "matrix")
        return req

    def bind(self, tensors):
        p, t = self.p, tensors
        w, at = [], 0
        self.q_off = self.k_off = self.v_off = self.g_off = None
        for name, attr in (("q", "q_off"), ("k", "k_off"), ("v", "v_off"), ("g", "g_off")):
            if p + name in t:
                setattr(self, attr, at)
                w.append(t[p + name])
                at += t[p + name].shape[0]
        pad = -at % 8
        if pad:
            w.append(w[0].new_zeros(pad, self.width))
        self.w_in = torch.cat(w).contiguous()
        self.w_out = t[p + "o"]
        self.slopes = None if self.slope_values is None else torch.tensor(
            self.slope_values, dtype=torch.float32, device=self.w_out.device)

    def cache_request(self):
        return CacheRequest(self.G, self.D + self.V, self.window, 1, 0, 0,
                            self.keep_first if self.window > 0 else 0)

    def forward(self, ctx, h, x, cache, fresh=False):
        ops, T = ctx.ops, h.shape[0]
        if cache.writes == self.shares_cache:
            raise ValueError("a layer with key/value projections writes its cache entry, a "
                             "layer without them only reads one")
        proj = ctx.buffer("span_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(proj, h, self.w_in)
        q = ctx.buffer("span_q", (T, self.H * self.D), torch.float32)
        sizes = dict(n_heads=self.H, n_kv_heads=self.G, head_dim=self.D, value_dim=self.V,
                     page_size=cache.page_size, status=ctx.status)
        ops.span_prepare(q, cache.pool, proj, cache.table, ctx.tok_pos, ctx.tok_req,
                         q_off=self.q_off, k_off=self.k_off, v_off=self.v_off,
                         qk_norm=self.qk_norm, eps=self.eps, writes=cache.writes, **sizes)
        att = ctx.buffer("span_att", (T, self.H * self.V), ctx.dtype)
        ops.span_attention(att, q, cache.pool, cache.table, ctx.tok_pos, ctx.tok_req,
                           scale=self.scale, slopes=self.slopes, window=self.window,
                           keep_first=self.keep_first, gate=proj if self.gate else None,
                           gate_offset=self.g_off or 0, out_scale=self.out_scale,
                           plan=getattr(ctx, "plan", None), **sizes)
        ops.linear(x, att, self.w_out, None, residual=None if fresh else x)


register_mixer("span_attention", SpanAttention)
