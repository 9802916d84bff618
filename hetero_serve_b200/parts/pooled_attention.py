"""Softmax attention over a sliding window plus pooled blocks of everything behind it, over the
paged cache.

Per token at position i (query head h uses key/value head h // (heads / kv_heads)):

    q = W_q x,  k = W_k x,  v = W_v x                                  no biases
    q, k <- rms(q) * w_q, rms(k) * w_k          per head over head_dim (``qk_norm``)
    q, k <- turned by their position on the first ``rot_dims`` numbers of each head: number d
            pairs with d + rot_dims/2, pair d turning by position * rot_base^(-2d/rot_dims)
    v   <- turned by ITS position over all of value_dim, in the same layout (``rotate_values``)
    visible: the positions j with 0 <= i - j < window, and for every block b of ``pool``
             positions with b*pool + pool - 1 <= i - window the mean of its keys and the mean
             of its values, as the cache holds them; one softmax over both kinds
    o_h = softmax(q_h . k * scale) v,   turned back by -i over value_dim;   out = W_o [o_0 ..]

The cache keeps one row [key | value] per token and key/value head for the window (and for as
long as the token's block is incomplete), and in the companion group one row of means per
complete block for the whole sequence.  q, k and v are ONE product; norms, angles, scores and
softmax are float32 in both precisions.
"""

from __future__ import annotations

import torch

from .base import CacheRequest, Mixer, TensorRequest, register_mixer


def rotary_frequencies(base: float, dims: int, device) -> torch.Tensor:
    """f_d = base^(-2d/dims), d < dims/2, formed in float64."""
    d = torch.arange(dims // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * d / max(dims, 1))).float().to(device).contiguous()


class PooledWindowAttention(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, window: int, pool: int, rot_base: float,
                 rot_dims: int, eps: float, prefix: str, rotate_values: bool = True,
                 qk_norm: bool = True):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        if window < 1 or pool < 1:
            raise ValueError("window and pool are positive")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim or (rotate_values and value_dim % 2):
            raise ValueError("rotated extents are even and lie inside the head")
        self.width, self.H, self.G = width, n_heads, n_kv_heads
        self.D, self.V = head_dim, value_dim
        self.scale, self.window, self.pool = float(scale), int(window), int(pool)
        self.rot_base, self.rot_dims = float(rot_base), int(rot_dims)
        self.rotate_values, self.qk_norm = bool(rotate_values), bool(qk_norm)
        self.eps, self.p = float(eps), prefix

    def tensor_requests(self):
        p, W = self.p, self.width
        req = {p + "q": TensorRequest((self.H * self.D, W), "matrix"),
               p + "k": TensorRequest((self.G * self.D, W), "matrix"),
               p + "v": TensorRequest((self.G * self.V, W), "matrix"),
               p + "o": TensorRequest((W, self.H * self.V), "matrix")}
        if self.qk_norm:
            req[p + "q.norm"] = TensorRequest((self.D,), "vector")
            req[p + "k.norm"] = TensorRequest((self.D,), "vector")
        return req

    def bind(self, tensors):
        p, t = self.p, tensors
        w = [t[p + "q"], t[p + "k"], t[p + "v"]]
        self.n_in = sum(m.shape[0] for m in w)
        pad = -self.n_in % 8
        if pad:
            w.append(w[0].new_zeros(pad, self.width))
        self.w_in = torch.cat(w).contiguous()
        self.w_qn = t[p + "q.norm"] if self.qk_norm else None
        self.w_kn = t[p + "k.norm"] if self.qk_norm else None
        dev = self.w_in.device
        self.freq_qk = rotary_frequencies(self.rot_base, self.rot_dims, dev) if self.rot_dims else None
        self.freq_v = rotary_frequencies(self.rot_base, self.V, dev) if self.rotate_values else None
        self.w_out = t[p + "o"]

    def cache_request(self):
        # A block's mean is formed in the step that brings its last position, from the rows of
        # its positions: they must still be resident then, so the token rows are kept for
        # max(window, pool) positions.
        return CacheRequest(self.G, self.D + self.V, max(self.window, self.pool), 1, 0, self.pool)

    def forward(self, ctx, h, x, cache, fresh=False):
        ops, T = ctx.ops, h.shape[0]
        proj = ctx.buffer("pooled_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(proj, h, self.w_in)
        q = ctx.buffer("pooled_q", (T, self.H * self.D), torch.float32)
        sizes = dict(n_heads=self.H, n_kv_heads=self.G, head_dim=self.D, value_dim=self.V,
                     page_size=cache.page_size, status=ctx.status)
        coarse = cache.coarse
        plan = getattr(ctx, "plan", None)
        # every request brings one token: the rows of a block that is completed now are of
        # earlier steps, and the launch that appends forms the block's mean as well
        folded = (cache.writes and plan is not None and plan.single_new and plan.tile_cap == 0
                  and getattr(ops, "folds_pooled_means", False))
        extra = dict(coarse_pool=coarse.pool, coarse_table=coarse.table, block=self.pool) \
            if folded else {}
        ops.pooled_prepare(q, cache.pool, proj, self.w_qn, self.w_kn, self.freq_qk, self.freq_v,
                           cache.table, ctx.tok_pos, ctx.tok_req, rot_dims=self.rot_dims,
                           eps=self.eps, writes=cache.writes, **sizes, **extra)
        if cache.writes and not folded:
            ops.pooled_means(coarse.pool, coarse.table, cache.pool, cache.table, ctx.tok_pos,
                             ctx.tok_req, n_kv_heads=self.G, row=self.D + self.V,
                             block=self.pool, page_size=cache.page_size, status=ctx.status)
        att = ctx.buffer("pooled_att", (T, self.H * self.V), ctx.dtype)
        ops.pooled_attention(att, q, cache.pool, cache.table, coarse.pool, coarse.table,
                             ctx.tok_pos, ctx.tok_req, self.freq_v, window=self.window,
                             block=self.pool, scale=self.scale, plan=plan, **sizes)
        ops.linear(x, att, self.w_out, None, residual=None if fresh else x)


register_mixer("pooled_window_attention", PooledWindowAttention)
