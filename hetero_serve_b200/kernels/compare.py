"""Per-operation timing of whole steps, for comparing one architecture with another.

:class:`TimedOps` stands in front of a :class:`CudaOps`: every operation a step calls is
bracketed by two CUDA events on the step's stream, and after the step the times are read and
summed per operation name, together with the operation's algorithmic FLOPs and bytes (from the
shapes of its arguments and the batch the caller describes).  The roofline time of an operation
is the larger of FLOPs / peak and bytes / bandwidth; the fraction reported is roofline time over
measured time.  Steps run eagerly (no CUDA graph), so a time includes the launch gap before the
kernel; operations of a few microseconds are dominated by it.
"""

from __future__ import annotations

from collections import defaultdict

import torch


def _nbytes(*ts) -> int:
    return sum(t.numel() * t.element_size() for t in ts if isinstance(t, torch.Tensor))


class TimedOps:
    """A proxy: ``ops`` with a stopwatch around each operation."""

    def __init__(self, ops):
        object.__setattr__(self, "_ops", ops)
        object.__setattr__(self, "_events", [])
        object.__setattr__(self, "batch", [])          # [(start, n)] of the step being run

    def __getattr__(self, name):
        target = getattr(self._ops, name)
        if not callable(target) or name.startswith("_") or name in _UNTIMED:
            return target

        def timed(*args, **kw):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = target(*args, **kw)
            b.record()
            self._events.append((name, a, b, _flops_and_bytes(name, args, kw, self.batch)))
            return out
        return timed

    def __setattr__(self, name, value):
        if name == "batch":
            object.__setattr__(self, name, value)
        else:
            setattr(self._ops, name, value)

    def collect(self) -> dict:
        """{operation: [ms, flops, bytes, calls]} since the last call; synchronises."""
        torch.cuda.synchronize()
        out = defaultdict(lambda: [0.0, 0, 0, 0])
        for name, a, b, (flops, nbytes) in self._events:
            rec = out[name]
            rec[0] += a.elapsed_time(b)
            rec[1] += flops
            rec[2] += nbytes
            rec[3] += 1
        self._events.clear()
        return dict(out)


_UNTIMED = {"stream", "register_kernel", "load_extension", "attention_plan_ints",
            "plan_attention", "make_plan", "decode_wide", "decode_splits"}


def _contexts(batch):
    """Sum over the step's tokens of the keys each sees, and the distinct cache rows read."""
    seen = sum(n * start + n * (n + 1) // 2 for start, n in batch)
    rows = sum(start + n for start, n in batch)
    return seen, rows


def _flops_and_bytes(name, args, kw, batch):
    """(FLOPs, bytes) an operation has to do, from its arguments."""
    try:
        if name == "linear":
            out, a, w = args[:3]
            res = kw.get("residual") if "residual" in kw else (args[5] if len(args) > 5 else None)
            return 2 * a.shape[0] * a.shape[1] * w.shape[0], _nbytes(out, a, w, res)
        if name == "norm_linear":
            out, _h, x = args[:3]
            w = args[6]
            return 2 * x.shape[0] * x.shape[1] * w.shape[0], _nbytes(out, x, w)
        if name == "linear_argmax":
            out, a, w = args[:3]
            return 2 * a.shape[0] * a.shape[1] * w.shape[0], _nbytes(out, a, w)
        if name in ("layernorm", "dyt_norm"):
            return 0, _nbytes(args[0]) + args[0].numel() * 4
        if name == "attention_append":
            out, qkv, pool = args[:3]
            g = args[6]
            seen, rows = _contexts(batch)
            kv_row = 2 * g.n_kv_heads * g.head_dim * pool.element_size()
            return 4 * g.n_heads * g.head_dim * seen, _nbytes(out, qkv) + rows * kv_row
        if name == "latent_attention":
            out, qa = args[:2]
            pool = args[3]
            H, R, P = kw["n_heads"], kw["rank"], kw["rot_dim"]
            seen, rows = _contexts(batch)
            return 2 * H * (2 * R + P) * seen, _nbytes(out, qa) + rows * (R + P) * pool.element_size()
        if name == "grouped_linear":
            out, a, w = args[:3]
            groups, k, n = w.shape
            return 2 * out.shape[0] * groups * k * n, _nbytes(out, w) + out.shape[0] * groups * k * 4
        if name == "delta_prepare":
            return 0, _nbytes(*args[:6])
        if name == "delta_recurrence":
            o, state = args[:2]
            shape = args[-1]
            T = o.shape[0]
            live = len([1 for _s, n in batch if n > 0])
            st = 2 * live * shape["heads"] * shape["dim"] * shape["vdim"] * 4
            return 7 * T * shape["heads"] * shape["dim"] * shape["vdim"], _nbytes(*args[2:7], o) + st
        if name == "delta_finish":
            return 0, _nbytes(args[0], args[1])
        if name in ("rms_norm", "cast_rows"):
            return 0, _nbytes(args[0]) + args[0].numel() * 4
        if name == "rms_norm_add":
            x, a = args[:2]
            return 0, 2 * _nbytes(x) + _nbytes(a, kw.get("b"), kw.get("h"))
        if name == "gated_act":
            return 0, _nbytes(args[0], args[1])
        if name == "qk_prepare":
            q_out = args[0]
            kv = q_out.shape[0] * kw["n_kv_heads"] * kw["head_dim"]
            return 0, _nbytes(q_out) + q_out.numel() * 4 + kv * 4 + 2 * kv * q_out.element_size()
        if name == "biased_attention":
            out, q, pool = args[:3]
            H, G, D, chunk = kw["n_heads"], kw["n_kv_heads"], kw["head_dim"], kw["chunk"]
            seen = rows = 0
            for start, n in batch:
                for i in range(start, start + n):
                    seen += (i % chunk if chunk else i) + 1
                first = start // chunk * chunk if chunk else 0
                rows += start + n - first               # distinct cache rows the portion reads
            return 4 * H * D * seen, _nbytes(out, q) + rows * 2 * G * D * pool.element_size()
        if name == "lightning_recurrence":
            o, state, proj = args[:3]
            H, D, V = kw["heads"], kw["dim"], kw["vdim"]
            live = len([1 for _s, n in batch if n > 0])
            cols = (2 * H * D + H * V) * 4
            return 5 * o.shape[0] * H * D * V, _nbytes(o) + o.shape[0] * cols + 2 * live * H * D * V * 4
        if name in ("moe_route", "moe_route_top"):
            h, wr = args[2], args[3]
            return 2 * h.shape[0] * wr.shape[0] * wr.shape[1], _nbytes(h, wr)
        if name == "moe_experts":
            x, _y, h, wg, wu = args[:5]
            idx = args[6]
            E, width, ff = wu.shape
            mats = 3 if wg is not None else 2          # an expert without a gate: up and down
            pairs = idx.shape[0] * idx.shape[1]
            touched = min(E, pairs) * mats * width * ff * wu.element_size()
            return 2 * pairs * mats * width * ff, _nbytes(h) + 2 * _nbytes(x) + touched
        if name == "moe_route_table":
            return 0, 3 * _nbytes(args[0])
        if name == "span_prepare":
            q_out, pool, proj = args[:3]
            rows = q_out.shape[0] * kw["n_kv_heads"] * (kw["head_dim"] + kw["value_dim"])
            return 0, _nbytes(q_out) + proj.numel() * 4 + (rows * pool.element_size()
                                                           if kw["writes"] else 0)
        if name == "span_attention":
            out, q, pool = args[:3]
            H, G, D, V = kw["n_heads"], kw["n_kv_heads"], kw["head_dim"], kw["value_dim"]
            win, keep = kw["window"], kw["keep_first"]
            seen = rows = 0
            for start, n in batch:
                for i in range(start, start + n):
                    seen += min(i + 1, win) + min(keep, max(0, i - win + 1)) if win else i + 1
                last = start + n - 1
                lo = max(0, start - win + 1) if win else 0
                rows += last + 1 - lo + min(keep, lo)    # distinct cache rows the portion reads
            gate = out.numel() * 4 if kw.get("gate") is not None else 0
            return (2 * H * (D + V) * seen,
                    _nbytes(out, q) + gate + rows * G * (D + V) * pool.element_size())
        if name == "token_shift_mix":
            out, x = args[:2]
            return 0, _nbytes(out, x)
        if name == "timemix_decay":
            out, low, w2t = args[:3]
            return 2 * out.numel() * low.shape[1], _nbytes(out, low, w2t)
        if name == "timemix_recurrence":
            o, state = args[:2]
            H, D = kw["heads"], kw["dim"]
            live = len([1 for _s, n in batch if n > 0])
            return 6 * o.shape[0] * H * D * D, 5 * _nbytes(o) + 2 * live * H * D * D * 4
        if name == "head_norm_gate":
            out, o = args[:2]
            return 0, _nbytes(out, o) + (o.numel() * 4 if args[3] is not None else 0)
        if name == "gather_mul":
            return 0, 2 * _nbytes(args[0]) + _nbytes(args[1])
        if name == "layernorm_add":
            x, y = args[:2]
            return 0, 2 * _nbytes(x) + _nbytes(y, kw.get("out"))
        if name == "learned_act":
            return 0, _nbytes(args[0], args[1])
        if name == "scale_softcap_":
            return 0, 2 * _nbytes(args[0])
        if name == "rglru_conv":
            return 0, 2 * _nbytes(args[0])
        if name == "rglru_scan":
            out, _state, u, z = args[:4]
            return 0, _nbytes(out, u, z) + u.numel() * 4
        if name == "rglru_step":
            out, state, proj = args[:3]
            w_gates = args[5]
            T, C = out.shape
            return (4 * T * C * w_gates.shape[1],
                    _nbytes(out, proj, w_gates) + 2 * T * C * kw["taps"] * 4)
        if name == "pooled_prepare":
            q_out, pool, proj = args[:3]
            rows = q_out.shape[0] * kw["n_kv_heads"] * (kw["head_dim"] + kw["value_dim"])
            return 0, _nbytes(q_out) + proj.numel() * 4 + rows * pool.element_size()
        if name == "pooled_means":
            pool = args[2]
            done = sum((start + n) // kw["block"] - start // kw["block"] for start, n in batch)
            return 0, done * (kw["block"] + 1) * kw["n_kv_heads"] * kw["row"] * pool.element_size()
        if name == "pooled_attention":
            out, q, pool = args[:3]
            H, G, D, V = kw["n_heads"], kw["n_kv_heads"], kw["head_dim"], kw["value_dim"]
            win, blk = kw["window"], kw["block"]
            seen = rows = 0
            for start, n in batch:
                for i in range(start, start + n):
                    seen += min(i + 1, win) + max(0, (i - win + 1) // blk)
                last = start + n - 1
                rows += last + 1 - max(0, start - win + 1) + max(0, (last - win + 1) // blk)
            return 2 * H * (D + V) * seen, _nbytes(out, q) + rows * G * (D + V) * pool.element_size()
        if name in ("embed", "scale_", "rotary_pairs", "latent_append", "sample", "argmax",
                    "kv_append"):
            return 0, _nbytes(args[0])
    except Exception:                                   # an estimate must never stop a step
        pass
    return 0, 0


def fractions(table: dict, peak_tflops: float, hbm_gbs: float) -> dict:
    """{operation: {"ms", "calls", "roof_ms", "frac", "bound"}} from :meth:`TimedOps.collect`."""
    out = {}
    for name, (ms, flops, nbytes, calls) in sorted(table.items(), key=lambda kv: -kv[1][0]):
        t_f = flops / (peak_tflops * 1e12) * 1e3
        t_b = nbytes / (hbm_gbs * 1e9) * 1e3
        roof = max(t_f, t_b)
        out[name] = {"ms": round(ms, 4), "calls": calls, "roof_ms": round(roof, 5),
                     "frac": round(roof / ms, 4) if ms > 0 else None,
                     "bound": "flops" if t_f >= t_b else "bytes"}
    return out
