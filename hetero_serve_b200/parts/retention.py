"""Retention: linear attention with a fixed decay per head, no softmax and no denominator, a
recurrent mixer whose per-request state is one float32 matrix S [dim, vdim] per head.

Per token at position p:

    q, k = W_q x, W_k x   [heads, dim];   v = W_v x   [heads, vdim]
    q, k <- turned by p on their first ``rot_dims`` numbers: number i pairs with i + rot_dims/2,
            the pair turns by p * rot_base^(-2i/rot_dims);   k <- k * k_scale
    S_h <- decay_h * S_h + k_h v_h^T ;   o_h = S_h^T q_h
    out = W_o [ (o_h / rms(o_h))_h  *  silu(W_g x) ]           (a norm per head, no weight)

The four projections of x are one product with float32 results; rotation, scale, state, norm and
gate are float32 in both precisions.  The recurrence is the launch lightning attention uses,
which turns and scales q and k while it stages them.  The state starts at zero (the runner
clears a slot when a request is opened) and is carried from step to step.
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, register_mixer
from .pooled_attention import rotary_frequencies


class Retention(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, n_heads: int, dim: int, vdim: int, decay, eps: float,
                 prefix: str, rot_base: float = 10000.0, rot_dims: int = 0,
                 k_scale: float | None = None, gate_act: str = "silu"):
        decay = [float(d) for d in decay]
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError("the rotated extent is even and lies inside the head")
        self.width, self.H, self.D, self.V = width, n_heads, dim, vdim
        self.decay_values, self.eps, self.p = decay, float(eps), prefix
        self.rot_base, self.rot_dims = float(rot_base), int(rot_dims)
        self.k_scale = float(dim) ** -0.5 if k_scale is None else float(k_scale)
        self.gate_act = gate_act
        self.n_in = 2 * self.H * self.D + 2 * self.H * self.V             # q | k | v | gate

    def tensor_requests(self):
        p, W, hd, hv = self.p, self.width, self.H * self.D, self.H * self.V
        return {p + "q": TensorRequest((hd, W), "matrix"), p + "k": TensorRequest((hd, W), "matrix"),
                p + "v": TensorRequest((hv, W), "matrix"), p + "g": TensorRequest((hv, W), "matrix"),
                p + "o": TensorRequest((W, hv), "matrix")}

    def bind(self, tensors):
        p, t = self.p, tensors
        pad = -self.n_in % 8
        w = [t[p + "q"], t[p + "k"], t[p + "v"], t[p + "g"]]
        if pad:
            w.append(w[0].new_zeros(pad, self.width))
        self.w_in = torch.cat(w).contiguous()
        self.w_out = t[p + "o"]
        dev = self.w_out.device
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=dev)
        self.freq = rotary_frequencies(self.rot_base, self.rot_dims, dev) if self.rot_dims else None

    def state_shape(self):
        return (self.H * self.D * self.V,)

    def forward(self, ctx, h, x, cache, fresh=False):
        ops, T = ctx.ops, h.shape[0]
        hd, hv = self.H * self.D, self.H * self.V
        proj = ctx.buffer("retention_proj", (T, self.w_in.shape[0]), torch.float32)
        ops.linear(proj, h, self.w_in)
        o = ctx.buffer("retention_o", (T, hv), torch.float32)
        ops.lightning_recurrence(o, ctx.state(), proj, self.decay, ctx.req_start, ctx.req_len,
                                 ctx.req_slot, q_off=0, k_off=hd, v_off=2 * hd, heads=self.H,
                                 dim=self.D, vdim=self.V, act="none", tok_pos=ctx.tok_pos,
                                 freq=self.freq, rot_dims=self.rot_dims, k_scale=self.k_scale)
        gated = ctx.buffer("retention_gated", (T, hv), ctx.dtype)
        ops.head_norm_gate(gated, o, None, proj, gate_offset=2 * hd + hv, heads=self.H,
                           dim=self.V, eps=self.eps, gate_act=self.gate_act)
        ops.linear(x, gated, self.w_out, None, residual=None if fresh else x)


register_mixer("retention", Retention)
