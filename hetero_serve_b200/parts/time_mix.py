"""Time mixing with a decay per token, head and key channel: a recurrent mixer whose
per-request state is one float32 matrix S [dim, dim] per head and the previous token's input.

With x' the previous token's input (zeros before the first token), every stream s of r, k, v, g,
w reads its own blend  x_s = x + (x' - x) * mu_s.  Per token:

    r, k, v = W_r x_r, W_k x_k, W_v x_v   [heads, dim];    gate = silu(W_g x_g)
    w = exp(-exp(W_w2 tanh(W_w1 x_w) + w0))                 per head and key channel
    o_h = (S_h + diag(u_h) k_h v_h^T)^T r_h                 the bonus u only for this token
    S_h <- diag(w_h) S_h + k_h v_h^T
    out = W_o [ (o_h / rms(o_h))_h * w_norm * gate ] * out_scale

The blends are one launch (which also keeps the step's last input of every request in the state),
the five projections ordinary linears with float32 results; the decay with its two exponentials,
the state, the bonus, the norm and the gate are float32 in both precisions.  The state starts at
zero (the runner clears a slot when a request is opened) and is carried from step to step.
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, register_mixer

STREAMS = ("r", "k", "v", "g", "w")


class TimeMix(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, dim: int, eps: float, prefix: str,
                 out_scale: float = 1.0):
        self.width, self.H, self.D = width, n_heads, dim
        self.eps, self.p, self.out_scale = float(eps), prefix, float(out_scale)

    def tensor_requests(self):
        p, W, hd = self.p, self.width, self.H * self.D
        req = {p + "mu." + s: TensorRequest((W,), "vector") for s in STREAMS}
        for s in ("r", "k", "v", "g"):
            req[p + s] = TensorRequest((hd, W), "matrix")
        req[p + "w1"] = TensorRequest((None, W), "matrix")      # the inner size is the tensor's
        req[p + "w2"] = TensorRequest((hd, None), "float32")
        req[p + "w0"] = TensorRequest((hd,), "vector")
        req[p + "u"] = TensorRequest((self.H, self.D), "float32")
        req[p + "norm"] = TensorRequest((hd,), "vector")
        req[p + "o"] = TensorRequest((W, hd), "matrix")
        return req

    def bind(self, tensors):
        p, t = self.p, tensors
        self.mu = torch.stack([t[p + "mu." + s] for s in STREAMS]).contiguous()     # [5, W]
        self.w_r, self.w_k, self.w_v, self.w_g = (t[p + s] for s in ("r", "k", "v", "g"))
        self.w1, self.w0 = t[p + "w1"], t[p + "w0"]
        self.w2t = t[p + "w2"].t().contiguous()                # [inner, channels]: read side by side
        self.u, self.norm_w, self.w_out = t[p + "u"].reshape(-1).contiguous(), t[p + "norm"], t[p + "o"]
        self.rank = self.w1.shape[0]
        if self.w2t.shape[0] != self.rank:
            raise ValueError("the two matrices of the decay do not share their inner size")

    def state_shape(self):
        return (self.H * self.D * self.D + self.width,)

    def forward(self, ctx, h, x, cache, fresh=False):
        ops, T = ctx.ops, h.shape[0]
        W, hd = self.width, self.H * self.D
        state = ctx.state()
        mixes = ctx.buffer("timemix_in", (len(STREAMS), T, W), ctx.dtype)
        ops.token_shift_mix(mixes, h, self.mu, state, ctx.tok_req, ctx.req_start, ctx.req_len,
                            ctx.req_slot, state_offset=hd * self.D)
        rkvg = ctx.buffer("timemix_rkvg", (4, T, hd), torch.float32)
        for i, wm in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            ops.linear(rkvg[i], mixes[i], wm)
        low = ctx.buffer("timemix_low", (T, self.rank), torch.float32)
        ops.linear(low, mixes[4], self.w1)
        decay = ctx.buffer("timemix_decay", (T, hd), torch.float32)
        ops.timemix_decay(decay, low, self.w2t, self.w0)
        o = ctx.buffer("timemix_o", (T, hd), torch.float32)
        ops.timemix_recurrence(o, state, rkvg[0], rkvg[1], rkvg[2], decay, self.u,
                               ctx.req_start, ctx.req_len, ctx.req_slot, heads=self.H,
                               dim=self.D)
        gated = ctx.buffer("timemix_gated", (T, hd), ctx.dtype)
        ops.head_norm_gate(gated, o, self.norm_w, rkvg[3], gate_offset=0, heads=self.H,
                           dim=self.D, eps=self.eps, gate_act="silu", out_scale=self.out_scale)
        ops.linear(x, gated, self.w_out, None, residual=None if fresh else x)


register_mixer("time_mix", TimeMix)
