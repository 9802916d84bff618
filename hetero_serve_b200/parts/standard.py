"""The parts GPT-2 is made of: learned position table, token embedding, LayerNorm,
causal multi-head attention over the paged cache, dense feed-forward, tied head.

Each takes its sizes, constants and tensor names as parameters and calls the
kernel interface of the step context; none refers to a model.
"""

from __future__ import annotations


import torch

from ..kernels.ops import ACTIVATIONS, LEARNED_ACTIVATIONS, AttentionGeometry
from .base import (CacheRequest, Embedding, FeedForward, Head, Mixer, Norm, PositionEncoding,
                   TensorRequest, register_embedding, register_feed_forward, register_head,
                   register_mixer, register_norm, register_position)


class LearnedPositions(PositionEncoding):
    """A learned absolute table added to the token embedding
    (heteroserve/model/torch_engine.py:89-90)."""

    def __init__(self, *, max_positions: int, width: int, table: str):
        self.n, self.width, self.name = max_positions, width, table
        self.table = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.n, self.width), "table")}

    def bind(self, tensors):
        self.table = tensors[self.name]

    def embedding_table(self):
        return self.table

    def max_positions(self):
        return self.n

    def fused_decode_params(self):
        return dict(table=self.table, width=self.width)


class NoPositions(PositionEncoding):
    def __init__(self, **_):
        pass


class TokenEmbedding(Embedding):
    """x = table[token] * scale (+ the position table's row); ``scale`` is 1 unless the
    architecture multiplies its embeddings."""

    def __init__(self, *, vocab_size: int, width: int, table: str, scale: float = 1.0):
        self.vocab, self.width, self.name = vocab_size, width, table
        self.scale = float(scale)
        self.table = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.vocab, self.width), "table")}

    def bind(self, tensors):
        self.table = tensors[self.name]

    def forward(self, ctx, x, position):
        more = {"scale": self.scale} if self.scale != 1.0 else {}
        ctx.ops.embed(x, ctx.tok_ids, ctx.tok_pos, ctx.tok_req, self.table,
                      position.embedding_table(), ctx.status, feedback=ctx.feedback, **more)

    def fused_decode_params(self):
        if self.scale != 1.0:
            return None
        return dict(table=self.table, width=self.width)


class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * weight + bias, statistics in float32
    (heteroserve/model/numpy_engine.py:26-30).  ``bias=None``: a norm with a weight alone.

    Besides ``forward`` it can be applied to a sublayer's OUTPUT and added into the stream in
    one pass (``add_normed``), which an arrangement with norms behind its sublayers calls; the
    same launch can form the rows the NEXT norm of the layer hands on (``then``)."""

    def __init__(self, *, width: int, eps: float, weight: str, bias: str | None):
        self.width, self.eps, self.wn, self.bn = width, float(eps), weight, bias
        self.weight = self.bias = None

    def tensor_requests(self):
        req = {self.wn: TensorRequest((self.width,), "vector")}
        if self.bn:
            req[self.bn] = TensorRequest((self.width,), "vector")
        return req

    def bind(self, tensors):
        self.weight = tensors[self.wn]
        self.bias = tensors[self.bn] if self.bn else torch.zeros_like(self.weight)

    def add_normed(self, ctx, x, y, h=None, then=None):
        """x += norm(y) for a float32 block ``y``.  With ``then=(norm, out)``, ``out`` also
        receives ``norm(x)`` of the new rows (another layer norm's output, for the sublayer
        that follows); with ``h`` (and no ``then``) it receives the new rows of x themselves
        in the compute type."""
        if then is None and h is not None:
            ctx.ops.layernorm_add(x, y, self.weight, self.bias, self.eps, out=h)
            return
        if then is not None and isinstance(then[0], LayerNorm):
            nxt, out = then
            ctx.ops.layernorm_add(x, y, self.weight, self.bias, self.eps, out=out,
                                  out_gamma=nxt.weight, out_beta=nxt.bias, out_eps=nxt.eps)
            return
        ctx.ops.layernorm_add(x, y, self.weight, self.bias, self.eps)
        if then is not None:
            then[0].forward(ctx, then[1], x)

    def forward(self, ctx, out, x, rows=None):
        ctx.ops.layernorm(out, x, self.weight, self.bias, self.eps, rows)

    def linear(self, ctx, out, h, x, w, bias=None, act="none"):
        ctx.ops.norm_linear(out, h, x, self.weight, self.bias, self.eps, w, bias, act)

    def fused_decode_params(self):
        return dict(weight=self.weight, bias=self.bias, eps=self.eps, width=self.width)


class CausalAttention(Mixer):
    """Multi-head (or grouped-query) causal attention over the paged cache.

    Fused projection ``qkv = h @ W + b`` with columns ``q | k | v``
    (heteroserve/model/torch_engine.py:299-303), keys and values appended to the pages,
    ``softmax(q k^T * scale) v`` over positions ``0..p`` (or the last ``window``), then the
    output projection added into the residual stream (torch_engine.py:306-316).
    ``scale`` arrives as a number: whoever builds the spec decides it.
    """

    def __init__(self, *, width: int, n_heads: int, head_dim: int, scale: float,
                 n_kv_heads: int | None = None, window: int = 0,
                 qkv_weight: str, qkv_bias: str | None, out_weight: str, out_bias: str | None,
                 stored_in_out: bool = True):
        self.width, self.H, self.D = width, n_heads, head_dim
        self.HK = n_kv_heads or n_heads
        if self.H % self.HK:
            raise ValueError(f"n_heads {self.H} is not a multiple of n_kv_heads {self.HK}")
        if head_dim % 16 or head_dim <= 0:
            raise ValueError(f"head_dim must be a positive multiple of 16, got {head_dim}")
        self.scale = float(torch.tensor(float(scale), dtype=torch.float64).to(torch.float32))
        self.window = int(window)
        self.qkv_width = (self.H + 2 * self.HK) * self.D
        self.names = (qkv_weight, qkv_bias, out_weight, out_bias)
        self.stored_in_out = stored_in_out
        self.w_qkv = self.b_qkv = self.w_out = self.b_out = None

    def tensor_requests(self):
        qw, qb, ow, ob = self.names
        hd = self.H * self.D
        io = self.stored_in_out
        req = {
            qw: TensorRequest((self.width, self.qkv_width) if io else (self.qkv_width, self.width),
                              "matrix", transpose=io),
            ow: TensorRequest((hd, self.width) if io else (self.width, hd), "matrix", transpose=io),
        }
        if qb:
            req[qb] = TensorRequest((self.qkv_width,), "vector")
        if ob:
            req[ob] = TensorRequest((self.width,), "vector")
        return req

    def bind(self, tensors):
        qw, qb, ow, ob = self.names
        self.w_qkv, self.w_out = tensors[qw], tensors[ow]
        self.b_qkv = tensors[qb] if qb else None
        self.b_out = tensors[ob] if ob else None

    def cache_request(self):
        return CacheRequest(self.HK, self.D, self.window)

    def geometry(self, cache) -> AttentionGeometry:
        return AttentionGeometry(
            n_heads=self.H, n_kv_heads=self.HK, head_dim=self.D, page_size=cache.page_size,
            num_pages=cache.num_pages, max_pages=cache.table.shape[1], q_off=0,
            k_off=self.H * self.D, v_off=(self.H + self.HK) * self.D, qkv_stride=self.qkv_width,
            window=self.window)

    takes_norm = True

    def fused_decode_params(self):
        return dict(w_qkv=self.w_qkv, b_qkv=self.b_qkv, w_out=self.w_out, b_out=self.b_out,
                    width=self.width, n_heads=self.H, n_kv_heads=self.HK, head_dim=self.D,
                    window=self.window, scale=self.scale)

    def forward(self, ctx, h, x, cache, norm=None):
        T = h.shape[0]
        qkv = ctx.buffer("qkv", (T, self.qkv_width), ctx.dtype)
        if norm is not None:
            norm.linear(ctx, qkv, h, x, self.w_qkv, self.b_qkv)
        else:
            ctx.ops.linear(qkv, h, self.w_qkv, self.b_qkv)
        g = self.geometry(cache)
        position = getattr(ctx, "position", None)
        if position is not None and position.acts_in_mixer:
            position.transform_qk(ctx, qkv, g)
        att = ctx.buffer("attn_out", (T, self.H * self.D), ctx.dtype)
        ctx.ops.attention_append(att, qkv, cache.pool, cache.table, ctx.tok_pos, ctx.tok_req, g,
                                 self.scale, ctx.status, ctx.plan, cache.writes)
        ctx.ops.linear(x, att, self.w_out, self.b_out, residual=x)


class DenseFeedForward(FeedForward):
    """x += act(h @ W_in + b_in) @ W_out + b_out (heteroserve/model/torch_engine.py:77-79)."""

    def __init__(self, *, width: int, inner: int, activation: str, in_weight: str,
                 in_bias: str | None, out_weight: str, out_bias: str | None,
                 stored_in_out: bool = True, act_params: str | None = None):
        if activation not in ACTIVATIONS and activation not in LEARNED_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: "
                             f"{sorted(ACTIVATIONS) + sorted(LEARNED_ACTIVATIONS)}")
        if (activation in LEARNED_ACTIVATIONS) != (act_params is not None):
            raise ValueError(f"activation {activation!r}: act_params names the tensor of an "
                             f"activation's learned numbers, and only of such a one")
        self.width, self.inner, self.act = width, inner, activation
        self.act_name = act_params
        self.names = (in_weight, in_bias, out_weight, out_bias)
        self.stored_in_out = stored_in_out
        self.w_in = self.b_in = self.w_out = self.b_out = None

    def tensor_requests(self):
        iw, ib, ow, ob = self.names
        io = self.stored_in_out
        req = {
            iw: TensorRequest((self.width, self.inner) if io else (self.inner, self.width),
                              "matrix", transpose=io),
            ow: TensorRequest((self.inner, self.width) if io else (self.width, self.inner),
                              "matrix", transpose=io),
        }
        if ib:
            req[ib] = TensorRequest((self.inner,), "vector")
        if ob:
            req[ob] = TensorRequest((self.width,), "vector")
        if self.act_name:
            req[self.act_name] = TensorRequest((LEARNED_ACTIVATIONS[self.act],), "vector")
        return req

    def bind(self, tensors):
        iw, ib, ow, ob = self.names
        self.w_in, self.w_out = tensors[iw], tensors[ow]
        self.b_in = tensors[ib] if ib else None
        self.b_out = tensors[ob] if ob else None
        # the learned numbers of the activation are read once and handed to the kernel by value
        self.act_values = (tuple(float(v) for v in tensors[self.act_name].double().cpu())
                           if self.act_name else ())

    takes_norm = True
    writes_fresh = True       # with fresh=True the result is written to x, not added into it

    def fused_decode_params(self):
        if self.act not in ("none", "gelu_tanh", "gelu_erf"):
            return None
        return dict(w_in=self.w_in, b_in=self.b_in, w_out=self.w_out, b_out=self.b_out,
                    width=self.width, inner=self.inner, activation=self.act)

    def forward(self, ctx, h, x, norm=None, fresh=False):
        T = h.shape[0]
        u = ctx.buffer("ff_inner", (T, self.inner), ctx.dtype)
        if self.act_name and norm is None:
            # an activation with learned numbers, on the float32 sums of the product
            ctx.ops.linear(u, h, self.w_in, self.b_in, act=self.act, act_values=self.act_values)
        elif self.act_name:
            # behind a norm that is fused into the product: the product leaves float32
            # numbers, the activation reads them and writes the rows the second product takes
            z = ctx.buffer("ff_inner_f32", (T, self.inner), torch.float32)
            norm.linear(ctx, z, h, x, self.w_in, self.b_in)
            ctx.ops.learned_act(u, z, self.act, self.act_values)
        elif norm is not None:
            norm.linear(ctx, u, h, x, self.w_in, self.b_in, act=self.act)
        else:
            ctx.ops.linear(u, h, self.w_in, self.b_in, act=self.act)
        ctx.ops.linear(x, u, self.w_out, self.b_out, residual=None if fresh else x)


class GatedFeedForward(FeedForward):
    """x += W_down (act(W_gate h) * (W_up h)) * s, with s = sigmoid(w_s . h), one number per
    token, when a token gate is named (else 1).  Gate and up are one product; the token gate
    is applied to the inner activations, which the down projection then carries through."""

    writes_fresh = True

    def __init__(self, *, width: int, inner: int, activation: str, gate_weight: str,
                 up_weight: str, down_weight: str, token_gate: str | None = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        self.width, self.inner, self.act = width, inner, activation
        self.names = (gate_weight, up_weight, down_weight, token_gate)

    def tensor_requests(self):
        gw, uw, dw, tg = self.names
        req = {gw: TensorRequest((self.inner, self.width), "matrix"),
               uw: TensorRequest((self.inner, self.width), "matrix"),
               dw: TensorRequest((self.width, self.inner), "matrix")}
        if tg:
            req[tg] = TensorRequest((1, self.width), "matrix")
        return req

    def bind(self, tensors):
        gw, uw, dw, tg = self.names
        self.w_gu = torch.cat([tensors[gw], tensors[uw]]).contiguous()
        self.w_down = tensors[dw]
        self.w_s = tensors[tg].reshape(-1).contiguous() if tg else None

    def forward(self, ctx, h, x, fresh=False):
        T = h.shape[0]
        gu = ctx.buffer("gated_gu", (T, 2 * self.inner), ctx.dtype)
        ctx.ops.linear(gu, h, self.w_gu)
        u = ctx.buffer("gated_inner", (T, self.inner), ctx.dtype)
        ctx.ops.gated_act(u, gu, h, self.w_s, ctx.tok_req, act=self.act)
        ctx.ops.linear(x, u, self.w_down, None, residual=None if fresh else x)


class LinearHead(Head):
    """logits = h @ W^T in float32, W being [vocab, width]: the token table itself when the
    head is tied (heteroserve/model/weights.py:40-43, torch_engine.py:86-87)."""

    def __init__(self, *, vocab_size: int, width: int, weight: str, scale: float = 1.0,
                 softcap: float = 0.0):
        self.vocab, self.width, self.name = vocab_size, width, weight
        self.scale = float(scale)          # logits = (h @ W^T) * scale
        self.softcap = float(softcap)      # > 0: then logits = softcap * tanh(logits / softcap)
        self.weight = None

    def tensor_requests(self):
        return {self.name: TensorRequest((self.vocab, self.width), "table")}

    def bind(self, tensors):
        self.weight = tensors[self.name]

    def forward(self, ctx, logits, h):
        # a step that samples and whose rows all take the argmax: the few-row kernel picks the
        # tokens while it streams the table (and stores the status word behind them)
        plain = self.scale == 1.0 and self.softcap == 0.0
        fused = getattr(ctx.ops, "linear_argmax", None) if plain else None
        if fused is not None and getattr(ctx, "sampling", False) \
                and getattr(ctx, "greedy_only", False):
            tokens = ctx.buffer(getattr(ctx, "tokens_name", "sampled"), (logits.shape[0] + 1,), torch.int32)
            if fused(logits, h, self.weight, tokens, feedback=ctx.feedback,
                     feedback_slot=ctx.samp_slot, status_word=ctx.status):
                ctx.fused_tokens = tokens
                return
        ctx.ops.linear(logits, h, self.weight)
        if self.softcap > 0.0:
            ctx.ops.scale_softcap_(logits, self.scale, self.softcap)
        elif self.scale != 1.0:
            ctx.ops.scale_(logits, self.scale)

    def fused_decode_params(self):
        if self.scale != 1.0 or self.softcap != 0.0:
            return None
        return dict(weight=self.weight, vocab=self.vocab, width=self.width)


register_position("learned", LearnedPositions)
register_position("none", NoPositions)
register_embedding("token_table", TokenEmbedding)
register_norm("layernorm", LayerNorm)
register_mixer("causal_attention", CausalAttention)
register_feed_forward("dense", DenseFeedForward)
register_feed_forward("gated", GatedFeedForward)
register_head("linear", LinearHead)
