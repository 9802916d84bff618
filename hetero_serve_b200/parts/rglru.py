"""A recurrent block around a real-gated linear recurrent unit: a mixer whose per-request state
is one float32 number per channel, plus the last ``taps - 1`` inputs of its short convolution.

Per token, with C channels split into ``blocks`` equal parts:

    y = gelu_tanh(W_y h + b_y)                                   the gate branch
    u = conv(W_x h + b_x)              causal, per channel, ``taps`` taps, zeros before the start
    r = sigmoid(R_b u_b + c_b),  i = sigmoid(I_b u_b + d_b)      per part b, square matrices
    log a = -decay_scale * r * softplus(lam);   a = exp(log a)
    S <- a * S + sqrt(1 - a^2) * i * u          from S = 0, the first token like every other
    out = W_o (S * y)

The two projections of h are one product; the two gates of a part are one block-diagonal
product; everything behind the projections that enters the recurrence (the convolution's
output, the gates, the decay, the state) is float32 in both precisions.  ``softplus(lam)`` is
formed once at binding.
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, register_mixer


class RealGatedRecurrence(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, channels: int, blocks: int, taps: int, decay_scale: float,
                 prefix: str):
        if channels % blocks:
            raise ValueError(f"{channels} channels do not split into {blocks} equal parts")
        if taps < 1:
            raise ValueError("a short convolution has at least one tap")
        self.width, self.C, self.B, self.taps = width, channels, blocks, int(taps)
        self.n = channels // blocks
        self.decay_scale, self.p = float(decay_scale), prefix

    def tensor_requests(self):
        p, W, C, B, n = self.p, self.width, self.C, self.B, self.n
        return {
            p + "y": TensorRequest((C, W), "matrix"), p + "y.b": TensorRequest((C,), "vector"),
            p + "x": TensorRequest((C, W), "matrix"), p + "x.b": TensorRequest((C,), "vector"),
            p + "conv": TensorRequest((C, self.taps), "float32"),
            p + "conv.b": TensorRequest((C,), "vector"),
            p + "ra": TensorRequest((B, n, n), "float32"), p + "ra.b": TensorRequest((B, n), "float32"),
            p + "ri": TensorRequest((B, n, n), "float32"), p + "ri.b": TensorRequest((B, n), "float32"),
            p + "lam": TensorRequest((C,), "vector"),
            p + "o": TensorRequest((W, C), "matrix"),
        }

    def bind(self, tensors):
        p, t = self.p, tensors
        self.w_in = torch.cat([t[p + "y"], t[p + "x"]]).contiguous()          # columns y | x
        self.b_in = torch.cat([t[p + "y.b"], t[p + "x.b"]]).contiguous()
        self.conv_w, self.conv_b = t[p + "conv"], t[p + "conv.b"]
        # the gates of part b side by side, summed index slowest: [B, n (in), 2n (r | i)]
        self.w_gates = torch.cat([t[p + "ra"].transpose(1, 2), t[p + "ri"].transpose(1, 2)],
                                 dim=2).contiguous()
        self.b_gates = torch.cat([t[p + "ra.b"], t[p + "ri.b"]], dim=1).reshape(-1).contiguous()
        # gate matrices that are bfloat16 numbers (a checkpoint stored in bfloat16): prompt
        # portions of a bfloat16 engine form the gates on the tensor cores, the float32 input
        # entering as three bfloat16 terms, which is the float32 product
        self.w_gates_nk = None
        if self.w_in.dtype == torch.bfloat16:
            nk = self.w_gates.transpose(1, 2).contiguous()
            if bool((nk.bfloat16().float() == nk).all()):
                self.w_gates_nk = nk.bfloat16()
        self.rate = torch.nn.functional.softplus(t[p + "lam"].double()).float().contiguous()
        self.w_out = t[p + "o"]

    def state_shape(self):
        return (self.C * self.taps,)          # S | the last taps - 1 inputs of the convolution

    def forward(self, ctx, h, x, cache, fresh=False):
        ops, T, C = ctx.ops, h.shape[0], self.C
        f32 = torch.float32
        proj = ctx.buffer("rglru_proj", (T, 2 * C), f32)
        ops.linear(proj, h, self.w_in, self.b_in)
        state = ctx.state()
        mixed = ctx.buffer("rglru_mixed", (T, C), ctx.dtype)
        plan = getattr(ctx, "plan", None)
        step = getattr(ops, "rglru_step", None)
        if (step is not None and plan is not None and plan.single_new and plan.tile_cap == 0
                and step(mixed, state, proj, self.conv_w, self.conv_b, self.w_gates,
                         self.b_gates, self.rate, ctx.tok_req, ctx.req_slot, channels=C,
                         blocks=self.B, taps=self.taps, decay_scale=self.decay_scale, y_off=0,
                         x_off=C)):
            # every request brings one token: convolution, gates and the state's step at once
            ops.linear(x, mixed, self.w_out, None, residual=None if fresh else x)
            return
        u = ctx.buffer("rglru_u", (T, C), f32)
        ops.rglru_conv(u, proj, self.conv_w, self.conv_b, state, ctx.tok_req, ctx.req_start,
                       ctx.req_slot, x_off=C, channels=C, taps=self.taps)
        z = ctx.buffer("rglru_gates", (T, 2 * C), f32)
        ops.grouped_linear(z, u, self.w_gates, w_nk=self.w_gates_nk, exact=True)
        ops.rglru_scan(mixed, state, u, z, proj, self.b_gates, self.rate, ctx.req_start,
                       ctx.req_len, ctx.req_slot, channels=C, blocks=self.B, taps=self.taps,
                       decay_scale=self.decay_scale, y_off=0, x_off=C)
        ops.linear(x, mixed, self.w_out, None, residual=None if fresh else x)


register_mixer("rglru", RealGatedRecurrence)
