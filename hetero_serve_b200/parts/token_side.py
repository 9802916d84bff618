"""A per-layer token input: a second, narrow embedding of the token id gates a projection of
the stream, and the result is RMS-normed and added to the stream.

    e = table[token][offset : offset + dim]           the layer's part of a row of the table
    g = act(W_gate x) * e                             x is the stream itself (not a normed copy)
    y = W_proj g;     x += y / sqrt(mean(y^2) + eps) * w_norm

It runs as the last part of a block (slot ``side`` of the ``sandwich_norm`` arrangement).  The
two products are ordinary linears; the gather-and-multiply between them is one launch and the
norm with the residual sum is the launch every RMS norm behind a sublayer uses, float32; it
also forms the layer norm in front of the block that runs next.
"""

from __future__ import annotations

import torch

from ..kernels.ops import ACTIVATIONS
from .base import FeedForward, TensorRequest, register_feed_forward


class TokenSideInput(FeedForward):
    def __init__(self, *, width: int, dim: int, offset: int, table: str, table_shape,
                 gate_weight: str, proj_weight: str, norm_weight: str, eps: float,
                 activation: str = "gelu_tanh"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ACTIVATIONS)}")
        rows, cols = table_shape
        if not 0 <= offset <= cols - dim:
            raise ValueError(f"columns {offset}..{offset + dim} lie outside a row of {cols}")
        self.width, self.dim, self.offset, self.eps = width, dim, int(offset), float(eps)
        self.act, self.table_shape = activation, (int(rows), int(cols))
        self.names = (table, gate_weight, proj_weight, norm_weight)

    def tensor_requests(self):
        tb, gw, pw, nw = self.names
        return {tb: TensorRequest(self.table_shape, "table"),
                gw: TensorRequest((self.dim, self.width), "matrix"),
                pw: TensorRequest((self.width, self.dim), "matrix"),
                nw: TensorRequest((self.width,), "vector")}

    def bind(self, tensors):
        tb, gw, pw, nw = self.names
        self.table, self.w_gate, self.w_proj, self.w_norm = (tensors[tb], tensors[gw],
                                                             tensors[pw], tensors[nw])

    forms_next_norm = True       # its last launch can form the norm of the block that runs next
    takes_stream_copy = True     # in a 16-bit engine it reads a copy of the stream the caller has

    def forward(self, ctx, h, x, then=None, x_copy=None):
        """``then=(norm, out)``: ``out`` also receives ``norm(x)`` of the new rows; a layer norm
        is formed by the launch that adds into the stream.  ``x_copy``: the stream's rows in the
        compute type, when the launch before left them (else they are cast here)."""
        ops, T = ctx.ops, x.shape[0]
        if ctx.dtype == torch.float32:
            src = x
        elif x_copy is not None:
            src = x_copy
        else:
            src = ctx.buffer("side_in", (T, self.width), ctx.dtype)
            ops.cast_rows(src, x)
        g = ctx.buffer("side_gate", (T, self.dim), torch.float32)
        ops.linear(g, src, self.w_gate, None, act=self.act)
        ge = ctx.buffer("side_gated", (T, self.dim), ctx.dtype)
        ops.gather_mul(ge, g, self.table, ctx.tok_ids, ctx.tok_req, col_offset=self.offset,
                       feedback=ctx.feedback)
        y = ctx.buffer("side_out", (T, self.width), torch.float32)
        ops.linear(y, ge, self.w_proj, None)
        nxt = then[0] if then is not None else None
        if nxt is not None and nxt.kind == "layernorm":
            ops.rms_norm_add(x, y, self.w_norm, self.eps, h=then[1],
                             ln=(nxt.weight, nxt.bias, nxt.eps))
            return
        ops.rms_norm_add(x, y, self.w_norm, self.eps)
        if nxt is not None:
            nxt.forward(ctx, then[1], x)


register_feed_forward("token_side_input", TokenSideInput)
