"""A routed feed-forward (mixture of experts), and the feed-forward that is not there.

Router: z = W_r h in float32, scores s = sigmoid(z).  The experts form ``groups`` equal groups
of neighbours; a group's score is the sum of its two largest scores; only experts of the
``keep`` best groups are eligible, and of those the ``top`` with the largest scores are chosen.
Their weights are their scores divided by the scores' sum (+ 1e-20).  An expert is

    g = min(W_gate h, limit);  u = clamp(W_up h, -limit, limit)
    y = g * sigmoid(1.702 g) * (u + 1);   output W_down y

and the layer adds the weighted sum of the chosen experts' outputs into the stream.  The
experts' matrices are stacked once at binding so that one kernel serves all experts.
Routing happens on the device; cache and scheduler know nothing of it.

A second rule (``scoring="softmax_top"``): z = W_r h + b_r in float32, the ``top`` largest
logits are chosen (the lower index wins a tie) and weighted by the softmax over the chosen
logits alone; and a second expert (``activation="silu"``): y = silu(W_gate h) * (W_up h).
``shared`` names a feed-forward (a :class:`PartSpec`) that runs for every token beside the
experts and is added to their sum.

A third rule (``scoring="table"``) has no router: an integer table [vocab, top] names the
experts of every token id, each weighing 1/top; and a third expert (``activation="relu2"``) has
no gate matrix: y = relu(W_up h)^2.
"""

from __future__ import annotations

import torch

from .base import FeedForward, TensorRequest, build_part, register_feed_forward

SCORINGS = ("sigmoid_groups", "softmax_top", "table")


class RoutedExperts(FeedForward):
    writes_fresh = True

    def __init__(self, *, width: int, ff: int, experts: int, top: int, router: str,
                 expert_prefix: str, groups: int = 1, keep: int = 1, limit: float = 0.0,
                 scoring: str = "sigmoid_groups", activation: str = "clamped",
                 router_bias: str | None = None, shared=None, table_rows: int = 0):
        if scoring not in SCORINGS:
            raise ValueError(f"unknown scoring {scoring!r}; known: {SCORINGS}")
        if activation not in ("clamped", "silu", "relu2"):
            raise ValueError(f"unknown expert activation {activation!r}")
        if scoring == "sigmoid_groups":
            if experts % groups:
                raise ValueError(f"{experts} experts do not form {groups} equal groups")
            if not 0 < keep <= groups or not 0 < top <= keep * (experts // groups):
                raise ValueError("top experts must fit into the kept groups")
            if router_bias is not None:
                raise ValueError("the grouped sigmoid rule takes no router bias")
        elif not 0 < top <= experts:
            raise ValueError(f"{top} chosen experts of {experts}")
        if scoring == "table" and (table_rows <= 0 or router_bias is not None):
            raise ValueError("the table rule needs the table's rows and takes no router bias")
        self.table_rows = int(table_rows)
        self.width, self.ff, self.E, self.top = width, ff, experts, top
        self.groups, self.keep, self.limit = groups, keep, float(limit)
        self.scoring, self.activation = scoring, activation
        self.gated = activation != "relu2"
        self.router_name, self.bias_name, self.prefix = router, router_bias, expert_prefix
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        if self.shared is not None:
            self.capturable = self.shared.capturable

    def _expert(self, e: int, which: str) -> str:
        return f"{self.prefix}{e}.{which}"

    def tensor_requests(self):
        if self.scoring == "table":
            req = {self.router_name: TensorRequest((self.table_rows, self.top), "int")}
        else:
            req = {self.router_name: TensorRequest((self.E, self.width), "float32")}
        if self.bias_name:
            req[self.bias_name] = TensorRequest((self.E,), "vector")
        if self.shared is not None:
            req.update(self.shared.tensor_requests())
        for e in range(self.E):
            if self.gated:
                req[self._expert(e, "gate")] = TensorRequest((self.ff, self.width), "matrix")
            req[self._expert(e, "up")] = TensorRequest((self.ff, self.width), "matrix")
            req[self._expert(e, "down")] = TensorRequest((self.width, self.ff), "matrix")
        return req

    def bind(self, tensors):
        self.w_router = tensors[self.router_name]
        self.b_router = tensors[self.bias_name] if self.bias_name else None
        if self.shared is not None:
            self.shared.bind({n: tensors[n] for n in self.shared.tensor_requests()})
        # prompt portions in bfloat16 form the logits as one product on the tensor cores (exact
        # products, float32 sums) when the router's values are bfloat16 numbers to begin with
        self.w_router_lp = None
        first = tensors[self._expert(0, "up")]
        if self.scoring != "table":
            low = self.w_router.to(torch.bfloat16)
            if first.dtype == torch.bfloat16 and torch.equal(low.to(torch.float32), self.w_router):
                self.w_router_lp = low.contiguous()

        def stack(which):          # [E, out, in], as stored: the summed index runs fastest
            return torch.stack([tensors[self._expert(e, which)]
                                for e in range(self.E)]).contiguous()
        self.w_gate = stack("gate") if self.gated else None
        self.w_up, self.w_down = stack("up"), stack("down")

    def forward(self, ctx, h, x, fresh=False):
        ops, T = ctx.ops, h.shape[0]
        if self.shared is not None:          # first: with ``fresh`` it is what opens x
            if fresh and getattr(self.shared, "writes_fresh", False):
                self.shared.forward(ctx, h, x, fresh=True)
            else:
                if fresh:
                    x.zero_()
                self.shared.forward(ctx, h, x)
        elif fresh:
            x.zero_()
        idx = ctx.buffer("route_idx", (T, self.top), torch.int32)
        wts = ctx.buffer("route_w", (T, self.top), torch.float32)
        z = None
        if self.w_router_lp is not None and T >= 64:
            z = ctx.buffer("route_z", (T, self.E), torch.float32)
            ops.linear(z, h, self.w_router_lp)
        if self.scoring == "table":
            ops.moe_route_table(idx, wts, self.w_router, ctx.tok_ids, ctx.tok_req, top=self.top,
                                feedback=ctx.feedback, experts=self.E)
        elif self.scoring == "softmax_top":
            ops.moe_route_top(idx, wts, h, self.w_router, self.b_router, ctx.tok_req,
                              top=self.top, z=z)
        else:
            ops.moe_route(idx, wts, h, self.w_router, ctx.tok_req, top=self.top,
                          n_groups=self.groups, keep=self.keep, z=z)
        y = ctx.buffer("expert_act", (T * self.top, self.ff), torch.float32)
        more = {"act": self.activation} if self.activation != "clamped" else {}
        ops.moe_experts(x, y, h, self.w_gate, self.w_up, self.w_down, idx, wts, ctx.tok_req,
                        limit=self.limit, **more)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward: adds nothing."""

    def __init__(self, **_):
        pass

    def forward(self, ctx, h, x, norm=None):
        return None


register_feed_forward("routed_experts", RoutedExperts)
register_feed_forward("none", NoFeedForward)
