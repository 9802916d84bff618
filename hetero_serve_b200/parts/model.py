"""Assembles a model from a :class:`ModelSpec`: builds the parts, collects the tensors
they ask for, derives what the cache must hold, and runs the schedule.

The model is the same object for every architecture; what differs is the spec.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

import torch

from .base import CacheRequest, TensorRequest, build_part
from .spec import LayerCall, LayerSpec, ModelSpec


class Block:
    """A layer: its parts and the way they are wired.

    An arrangement is a subclass that names its parts and their families in ``slots`` and
    wires them in ``forward``.  The parts are built from the layer's spec and become
    attributes of the same names.  At most one part of the mixer family may ask for a cache
    entry or a state slot (a :class:`LayerCall` addresses one of each)."""

    slots: Mapping[str, str] = {}          # part name -> family ("mixer", "feed_forward", "norm")
    optional: tuple[str, ...] = ()         # slots a layer may leave out (the attribute is None)

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        missing = [n for n in self.slots if n not in spec.parts and n not in self.optional]
        extra = [n for n in spec.parts if n not in self.slots]
        if missing or extra:
            raise ValueError(f"arrangement {spec.arrangement!r} has the parts "
                             f"{sorted(self.slots)}; missing {missing}, unknown {extra}")
        self.named = {name: build_part(family, spec.parts[name])
                      for name, family in self.slots.items() if name in spec.parts}
        for name in self.slots:
            setattr(self, name, self.named.get(name))
        holders = [p for n, p in self.named.items() if self.slots[n] == "mixer"
                   and (p.cache_request() is not None or p.state_shape() is not None)]
        if len(holders) > 1:
            raise ValueError("a layer has two mixers that keep a cache or state; a layer call "
                             "addresses one cache entry and one state slot")
        mixers = [p for n, p in self.named.items() if self.slots[n] == "mixer"]
        self.cache_holder = holders[0] if holders else (mixers[0] if mixers else None)

    def parts(self):
        return tuple(self.named.values())

    def forward(self, ctx, x, cache) -> None:
        raise NotImplementedError


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += feed_forward(norm2(x))
    (heteroserve/model/torch_engine.py:297-317)."""

    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, x, cache):
        h = ctx.buffer("normed", (x.shape[0], x.shape[1]), ctx.dtype)
        if self.mixer.takes_norm:           # the mixer forms norm + input projection itself
            self.mixer.forward(ctx, h, x, cache, norm=self.norm1)
        else:
            self.norm1.forward(ctx, h, x)
            self.mixer.forward(ctx, h, x, cache)
        if self.feed_forward.takes_norm:
            self.feed_forward.forward(ctx, h, x, norm=self.norm2)
        else:
            self.norm2.forward(ctx, h, x)
            self.feed_forward.forward(ctx, h, x)


class ParallelBlock(Block):
    """One norm, both sublayers read its output:  h = norm1(x);  x += mixer(h) + feed_forward(h).
    Each sublayer adds its share into the float32 stream."""

    slots = {"norm1": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, ctx, x, cache):
        h = ctx.buffer("normed", (x.shape[0], x.shape[1]), ctx.dtype)
        self.norm1.forward(ctx, h, x)
        self.mixer.forward(ctx, h, x, cache)
        self.feed_forward.forward(ctx, h, x)


class OutputNormBlock(Block):
    """Norms behind the sublayers, which read the stream itself:

        x += norm1(mixer(x));  x += norm2(feed_forward(x))

    The sublayers' input ``h`` is the stream in the compute type (the stream itself in
    float32).  A sublayer's output goes to a float32 block of its own: parts that can write
    one (``writes_fresh``) are called with ``fresh=True`` and may hand back a deferred output
    the norm forms on the way (:class:`hetero_serve_b200.parts.rms_norm.NormedPair`); for the
    others the block is zeroed and they add into it as they add into a stream.  The norms
    must offer ``add_normed``.  A layer may leave ``norm2`` and ``feed_forward`` out (both or
    neither): it then ends after the mixer."""

    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}
    optional = ("norm2", "feed_forward")
    keeps_stream_copy = True

    def __init__(self, spec: LayerSpec):
        super().__init__(spec)
        if (self.norm2 is None) != (self.feed_forward is None):
            raise ValueError("arrangement 'output_norm': norm2 and feed_forward come together")
        for name, part in self.named.items():
            if self.slots[name] == "norm" and not hasattr(part, "add_normed"):
                raise ValueError(f"arrangement 'output_norm': {name} of kind {part.kind!r} "
                                 f"cannot be applied to a sublayer's output (no add_normed)")
        self.has_ff = self.feed_forward is not None

    @staticmethod
    def _run(part, ctx, h, y, *more):
        if getattr(part, "writes_fresh", False):
            out = part.forward(ctx, h, y, *more, fresh=True)
            return y if out is None else out
        y.zero_()
        part.forward(ctx, h, y, *more)
        return y

    def forward(self, ctx, x, cache):
        T, W = x.shape
        low = ctx.dtype != torch.float32
        if low:
            h = ctx.buffer("stream_copy", (T, W), ctx.dtype)
            if not getattr(ctx, "stream_copy_fresh", False):
                ctx.ops.cast_rows(h, x)
        else:
            h = x
        y = ctx.buffer("sublayer_out", (T, W), torch.float32)
        out = self._run(self.mixer, ctx, h, y, cache)
        self.norm1.add_normed(ctx, x, out, h=h if low else None)
        if self.has_ff:
            out = self._run(self.feed_forward, ctx, h, y)
            self.norm2.add_normed(ctx, x, out, h=h if low else None)
        ctx.stream_copy_fresh = low


class SandwichNormBlock(Block):
    """Norms before AND behind each sublayer:

        x += norm1b(mixer(norm1(x)));  x += norm2b(feed_forward(norm2(x)))

    A sublayer's output goes to a float32 block of its own (as under ``output_norm``); the norm
    behind it is added into the stream by ``add_normed``, which in the same launch forms the
    rows of the norm in front of the feed-forward.  A layer may leave ``norm2``,
    ``feed_forward`` and ``norm2b`` out (all or none): it then ends after the mixer.  When the
    block that runs next is of this arrangement too, the layer's last launch also forms the
    rows of THAT block's first norm (``ctx.normed_ahead``), which then skips it.

    ``side`` (optional, a feed-forward part) runs last and reads the STREAM itself, not a
    normed copy: ``x += side(x)``.  It is handed ``then=(norm, out)`` like the norms, so that a
    part that can form the next block's first norm in its last launch does so; with any other
    part nothing is formed ahead."""

    slots = {"norm1": "norm", "mixer": "mixer", "norm1b": "norm", "norm2": "norm",
             "feed_forward": "feed_forward", "norm2b": "norm", "side": "feed_forward"}
    optional = ("norm2", "feed_forward", "norm2b", "side")

    def __init__(self, spec: LayerSpec):
        super().__init__(spec)
        present = [getattr(self, n) is not None for n in ("norm2", "feed_forward", "norm2b")]
        if any(present) != all(present):
            raise ValueError("arrangement 'sandwich_norm': norm2, feed_forward and norm2b "
                             "come together")
        for name in ("norm1b", "norm2b"):
            part = getattr(self, name)
            if part is not None and not hasattr(part, "add_normed"):
                raise ValueError(f"arrangement 'sandwich_norm': {name} of kind {part.kind!r} "
                                 f"cannot be applied to a sublayer's output (no add_normed)")
        self.has_ff = self.feed_forward is not None

    def forward(self, ctx, x, cache):
        T, W = x.shape
        h = ctx.buffer("normed", (T, W), ctx.dtype)
        y = ctx.buffer("sublayer_out", (T, W), torch.float32)
        if not getattr(ctx, "normed_ahead", False):
            self.norm1.forward(ctx, h, x)
        nxt = getattr(ctx, "next_block", None)
        ahead = (nxt.norm1, h) if isinstance(nxt, SandwichNormBlock) else None
        side_ahead = self.side is not None and getattr(self.side, "forms_next_norm", False)
        if self.side is not None and not side_ahead:
            ahead = None                      # the stream still changes behind the last norm
        ctx.normed_ahead = ahead is not None
        last = None if self.side is not None else ahead
        # a side part that reads the stream in the compute type gets its copy from the launch of
        # the last norm (a 16-bit engine; in float32 it reads the stream itself)
        more = {}
        if self.side is not None and ctx.dtype != torch.float32 \
                and getattr(self.side, "takes_stream_copy", False):
            more["h"] = ctx.buffer("side_stream_copy", (T, W), ctx.dtype)
        out = OutputNormBlock._run(self.mixer, ctx, h, y, cache)
        if not self.has_ff:
            self.norm1b.add_normed(ctx, x, out, then=last, **more)
        else:
            self.norm1b.add_normed(ctx, x, out, then=(self.norm2, h))
            out = OutputNormBlock._run(self.feed_forward, ctx, h, y)
            self.norm2b.add_normed(ctx, x, out, then=last, **more)
        if self.side is not None:
            extra = {"x_copy": more["h"]} if more else {}
            if side_ahead:
                self.side.forward(ctx, h, x, then=ahead, **extra)
            else:
                self.side.forward(ctx, h, x, **extra)


_ARRANGEMENTS: dict[str, Callable[[LayerSpec], Block]] = {"pre_norm": PreNormBlock,
                                                          "parallel": ParallelBlock,
                                                          "output_norm": OutputNormBlock,
                                                          "sandwich_norm": SandwichNormBlock}


def register_arrangement(name: str, factory: Callable[[LayerSpec], Block], *, replace=False):
    if name in _ARRANGEMENTS and not replace:
        raise ValueError(f"arrangement {name!r} is already registered")
    _ARRANGEMENTS[name] = factory


@dataclass(frozen=True)
class CacheGroup:
    """Cache entries with the same needs share a pool of pages and a block table."""

    kv_heads: int
    head_dim: int
    window: int
    entries: tuple[int, ...]        # cache entry numbers, in pool order
    planes: int = 2                 # rows kept per token and head (keys and values: two)
    chunk: int = 0                  # > 0: only the rows of the chunk the request is in are kept
    stride: int = 1                 # > 1: one row per block of this many positions
    keep_first: int = 0             # with a window: the first positions' rows stay as well


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.position = build_part("position", spec.position)
        self.blocks: list[Block] = []
        for ls in spec.layers:
            if ls.arrangement not in _ARRANGEMENTS:
                raise ValueError(f"unknown arrangement {ls.arrangement!r}; "
                                 f"registered: {sorted(_ARRANGEMENTS)}")
            self.blocks.append(_ARRANGEMENTS[ls.arrangement](ls))
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.schedule: tuple[LayerCall, ...] = spec.resolved_schedule()
        self.capturable = all(part.capturable for part in self.parts())
        self._derive_cache()
        self.dtype = None
        self.device = None

    # -- structure ----------------------------------------------------------
    def parts(self):
        yield self.embedding
        yield self.position
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    def tensor_requests(self) -> dict[str, TensorRequest]:
        out: dict[str, TensorRequest] = {}
        for part in self.parts():
            for name, req in part.tensor_requests().items():
                if name in out and out[name] != req:
                    raise ValueError(f"tensor {name!r} is requested twice with different "
                                     f"shapes or roles: {out[name]} and {req}")
                out[name] = req
        return out

    def _derive_cache(self) -> None:
        entry_req: dict[int, CacheRequest] = {}
        self.state_shapes: dict[int, tuple[int, ...]] = {}     # schedule index -> shape
        for idx, call in enumerate(self.schedule):
            mixer = self.blocks[call.layer].cache_holder
            if mixer is None:
                continue
            req = mixer.cache_request()
            if req is not None:
                if call.cache in entry_req and entry_req[call.cache] != req:
                    raise ValueError(f"cache entry {call.cache} is shared by mixers with "
                                     f"different needs: {entry_req[call.cache]} and {req}")
                entry_req[call.cache] = req
            shape = mixer.state_shape()
            if shape is not None:
                self.state_shapes[idx] = tuple(shape)
        groups: dict[CacheRequest, list[int]] = {}
        for entry in sorted(entry_req):
            groups.setdefault(entry_req[entry], []).append(entry)
        self.cache_groups: list[CacheGroup] = [
            CacheGroup(r.kv_heads, r.head_dim, r.window, tuple(es), r.planes, r.chunk,
                       keep_first=r.keep_first)
            for r, es in groups.items()]
        self.entry_location: dict[int, tuple[int, int]] = {}
        for gi, g in enumerate(self.cache_groups):
            for k, e in enumerate(g.entries):
                self.entry_location[e] = (gi, k)
        # entries that also keep one row per block of positions: companion groups at that rate
        # (every position's block stays, so no window), behind the token groups
        coarse: dict[tuple, list[int]] = {}
        for entry in sorted(entry_req):
            r = entry_req[entry]
            if r.pool > 0:
                coarse.setdefault((r.kv_heads, r.head_dim, r.planes, r.pool), []).append(entry)
        self.coarse_location: dict[int, tuple[int, int]] = {}
        for (kv_heads, head_dim, planes, pool), es in coarse.items():
            gi = len(self.cache_groups)
            self.cache_groups.append(CacheGroup(kv_heads, head_dim, 0, tuple(es), planes, 0, pool))
            for k, e in enumerate(es):
                self.coarse_location[e] = (gi, k)

    def kv_bytes_per_token(self, itemsize: int) -> int:
        return sum(-(-g.planes * g.kv_heads * g.head_dim * len(g.entries) * itemsize // g.stride)
                   for g in self.cache_groups)

    # -- weights --------------------------------------------------------------
    def bind(self, stored: Mapping[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Convert the stored tensors once and hand every part its own.

        matrix/table → ``dtype`` (bfloat16 or float32); vector → float32; int → int32.
        A tensor asked for by two parts (a tied head) is converted once and shared."""
        requests = self.tensor_requests()
        converted: dict[str, torch.Tensor] = {}
        for name, req in requests.items():
            t = stored[name]
            if req.role in ("matrix", "table"):
                t = t.to(device=device, dtype=dtype)
                if req.transpose:
                    t = t.t()
            elif req.role in ("vector", "float32"):
                t = t.to(device=device, dtype=torch.float32)
            elif req.role == "int":
                t = t.to(device=device, dtype=torch.int32)
            else:
                raise ValueError(f"tensor {name!r}: unknown role {req.role!r}")
            converted[name] = t.contiguous()
        for part in self.parts():
            part.bind({n: converted[n] for n in part.tensor_requests()})
        self.dtype, self.device = dtype, device
        self.tensors = converted

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())

    # -- the forward pass ---------------------------------------------------
    def forward(self, ctx):
        """Run the tokens of ``ctx`` through the schedule; returns float32 logits
        ``[n_logit_rows, vocab]`` at ``ctx.logit_rows`` (None when none are wanted)."""
        spec = self.spec
        fused = getattr(ctx, "fused", None)
        if fused is not None and fused.applies(ctx):
            # single decoded tokens only, and a model the persistent kernel serves: one launch
            logits, ctx.fused_tokens = fused.run(ctx)
            return logits
        T = ctx.n_rows
        x = ctx.buffer("residual", (T, spec.width), torch.float32)
        ctx.position = self.position          # mixers ask it whether it acts on queries and keys
        self.embedding.forward(ctx, x, self.position)
        ctx.stream_copy_fresh = False         # no copy of the stream in the compute type yet
        ctx.normed_ahead = False              # nobody has formed the next block's first norm
        for idx, call in enumerate(self.schedule):
            ctx.call_index = idx
            cache = ctx.cache_view(call) if call.cache in self.entry_location else None
            block = self.blocks[call.layer]
            ctx.next_block = (self.blocks[self.schedule[idx + 1].layer]
                              if idx + 1 < len(self.schedule) else None)
            block.forward(ctx, x, cache)
            if not getattr(block, "keeps_stream_copy", False):
                ctx.stream_copy_fresh = False
        ctx.call_index = None
        W = ctx.n_logit_rows
        if W == 0:
            return None
        hf = ctx.buffer("final_normed", (W, spec.width), ctx.dtype)
        self.final_norm.forward(ctx, hf, x, rows=ctx.logit_rows)
        logits = ctx.buffer("logits", (W, spec.vocab_size), torch.float32)
        self.head.forward(ctx, logits, hf)
        return logits
