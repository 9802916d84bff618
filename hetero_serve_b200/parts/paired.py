"""Two mixers side by side.  Both read the same input; each output is RMS-normed over the model
width with a weight of its own, and the pair's output is ``mix`` times their sum:

    out = mix * (rms(left(x)) * w_left + rms(right(x)) * w_right)          mix = 1/2

The two sub-mixers are ordinary mixers given as :class:`PartSpec`; at most one of them may keep
a cache entry and at most one a state (a layer call addresses one of each).  Sub-mixers that
offer ``input_projection`` / ``forward_projected`` share ONE product of the input (their weights
are stacked at binding); others run on their own into a zeroed block.  Under an arrangement
that norms its sublayers' outputs the pair is not formed here: the two blocks are handed on as
a :class:`NormedPair` and the norm behind the sublayer forms it in the same pass.
"""

from __future__ import annotations

import torch

from .base import Mixer, TensorRequest, build_part, register_mixer
from .rms_norm import NormedPair
from .spec import PartSpec


class NormedMixerPair(Mixer):
    writes_fresh = True

    def __init__(self, *, width: int, eps: float, left: PartSpec, right: PartSpec,
                 left_weight: str, right_weight: str, mix: float = 0.5):
        self.width, self.eps, self.mix = width, float(eps), float(mix)
        self.subs = (build_part("mixer", left), build_part("mixer", right))
        self.names = (left_weight, right_weight)
        if sum(s.cache_request() is not None for s in self.subs) > 1 or \
                sum(s.state_shape() is not None for s in self.subs) > 1:
            raise ValueError("both mixers of a pair keep a cache entry (or both a state); a "
                             "layer call addresses one of each")
        self.capturable = all(s.capturable for s in self.subs)

    def tensor_requests(self):
        req = {n: TensorRequest((self.width,), "vector") for n in self.names}
        for s in self.subs:
            req.update(s.tensor_requests())
        return req

    def bind(self, tensors):
        for s in self.subs:
            s.bind({n: tensors[n] for n in s.tensor_requests()})
        self.out_w = tuple(tensors[n] for n in self.names)
        # one product for the sub-mixers that can run on a slice of it
        self.offsets, ws, bs, at = [], [], [], 0
        for s in self.subs:
            if not hasattr(s, "input_projection"):
                self.offsets.append(None)
                continue
            w, b = s.input_projection()
            self.offsets.append(at)
            ws.append(w)
            bs.append(b if b is not None else torch.zeros(w.shape[0], dtype=torch.float32,
                                                          device=w.device))
            at += w.shape[0]
        self.w_in = torch.cat(ws).contiguous() if ws else None
        self.b_in = torch.cat(bs).contiguous() if ws and any(
            s.input_projection()[1] is not None for s in self.subs
            if hasattr(s, "input_projection")) else None

    def cache_request(self):
        for s in self.subs:
            if s.cache_request() is not None:
                return s.cache_request()
        return None

    def state_shape(self):
        for s in self.subs:
            if s.state_shape() is not None:
                return s.state_shape()
        return None

    def forward(self, ctx, h, x, cache, fresh=False):
        T = h.shape[0]
        proj = None
        if self.w_in is not None:
            proj = ctx.buffer("pair_proj", (T, self.w_in.shape[0]), torch.float32)
            ctx.ops.linear(proj, h, self.w_in, self.b_in)
        outs = []
        for i, (s, off) in enumerate(zip(self.subs, self.offsets)):
            y = ctx.buffer(f"pair_out{i}", (T, self.width), torch.float32)
            if off is not None:
                s.forward_projected(ctx, h, proj, off, y, cache, accumulate=False)
            elif getattr(s, "writes_fresh", False):
                s.forward(ctx, h, y, cache, fresh=True)
            else:
                y.zero_()
                s.forward(ctx, h, y, cache)
            outs.append(y)
        pair = NormedPair(outs[0], self.out_w[0], outs[1], self.out_w[1], self.mix, self.eps)
        if fresh:
            return pair                      # the norm behind the sublayer forms it
        ctx.ops.rms_norm_add(x, pair.a, None, self.eps, b=pair.b, wa=pair.wa, wb=pair.wb,
                             mix=pair.mix)
        return None


register_mixer("normed_pair", NormedMixerPair)


class SummedMixerPair(Mixer):
    """Two mixers side by side whose outputs are added: ``out = left(x) + right(x)``.  Weights
    of the two halves are the sub-mixers' business (an ``out_scale`` of their own); at most one
    of them may keep a cache entry and at most one a state.  The first writes the block, the
    second adds into it."""

    writes_fresh = True

    def __init__(self, *, left: PartSpec, right: PartSpec):
        self.subs = (build_part("mixer", left), build_part("mixer", right))
        if sum(s.cache_request() is not None for s in self.subs) > 1 or \
                sum(s.state_shape() is not None for s in self.subs) > 1:
            raise ValueError("both mixers of a pair keep a cache entry (or both a state); a "
                             "layer call addresses one of each")
        self.capturable = all(s.capturable for s in self.subs)

    def tensor_requests(self):
        req = {}
        for s in self.subs:
            req.update(s.tensor_requests())
        return req

    def bind(self, tensors):
        for s in self.subs:
            s.bind({n: tensors[n] for n in s.tensor_requests()})

    cache_request = NormedMixerPair.cache_request
    state_shape = NormedMixerPair.state_shape

    def forward(self, ctx, h, x, cache, fresh=False):
        first = fresh
        for s in self.subs:
            if first and getattr(s, "writes_fresh", False):
                s.forward(ctx, h, x, cache, fresh=True)
            else:
                if first:
                    x.zero_()
                s.forward(ctx, h, x, cache)
            first = False


register_mixer("summed_pair", SummedMixerPair)
