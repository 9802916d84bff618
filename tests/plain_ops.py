"""Plain PyTorch twins of the kernel operations, one function per kernel, with the
signatures of ``hetero_serve_b200.kernels.CudaOps``.

They serve two purposes: each CUDA kernel is compared with its twin (in float64
where the twin is the reference), and, since they run on CPU tensors, the engine's
step function, cache and scheduler can be exercised without a GPU in the tests.
They are written for clarity (loops over tokens and heads), not for speed, and are
never imported by the package.
"""

from __future__ import annotations

import math

import torch

try:
    from .plain_gpt2 import gelu_erf, gelu_new, philox4x32, sample_token, uniform_for
except ImportError:  # run as a top-level module
    from plain_gpt2 import gelu_erf, gelu_new, philox4x32, sample_token, uniform_for

_ACT = {"none": lambda u: u, "gelu_tanh": gelu_new, "gelu_erf": gelu_erf,
        "relu2": lambda u: torch.relu(u) ** 2, "silu": lambda u: u * torch.sigmoid(u)}


_GATE = {"silu": lambda u: u * torch.sigmoid(u), "sigmoid": torch.sigmoid}


class PlainOps:
    name = "plain"

    def __init__(self, compute_dtype=torch.float64):
        self.cd = compute_dtype

    def embed(self, x, ids, pos, req, wte, wpe, status, feedback=None, scale=1.0):
        n = x.shape[0]
        for t in range(n):
            if int(req[t]) < 0:
                x[t] = 0
                continue
            tok = int(ids[t])
            if tok < 0 and feedback is not None:
                tok = int(feedback[-(tok + 1)])
            row = wte[tok].to(self.cd) * scale
            if wpe is not None:
                row = row + wpe[int(pos[t])].to(self.cd)
            x[t] = row.to(x.dtype)

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        n = out.shape[0]
        src = x[rows[:n].long()] if rows is not None else x[:n]
        v = src.to(self.cd)
        mu = v.mean(-1, keepdim=True)
        c = v - mu
        var = (c * c).mean(-1, keepdim=True)
        out.copy_((c / torch.sqrt(var + eps) * gamma.to(self.cd) + beta.to(self.cd)).to(out.dtype))

    def linear(self, out, a, w, bias=None, act="none", residual=None, act_values=()):
        v = a.to(self.cd) @ w.to(self.cd).T
        if bias is not None:
            v = v + bias.to(self.cd)
        if act_values:
            tmp = torch.empty_like(v)
            self.learned_act(tmp, v, act, act_values)
            v = tmp
        else:
            v = _ACT[act](v)
        if residual is not None:
            v = v + residual.to(self.cd)
        out.copy_(v.to(out.dtype))

    def norm_linear(self, out, h, x, gamma, beta, eps, w, bias=None, act="none"):
        self.layernorm(h, x, gamma, beta, eps)
        self.linear(out, h, w, bias, act=act)

    @staticmethod
    def _pool_view(pool, g):
        return pool.view(g.num_pages, 2, g.n_kv_heads, g.page_size, g.head_dim)

    def kv_append(self, pool, qkv, table, tok_pos, tok_req, g, status, n_tokens=None):
        n = qkv.shape[0] if n_tokens is None else n_tokens
        pv = self._pool_view(pool, g)
        kw = g.n_kv_heads * g.head_dim
        for t in range(n):
            r = int(tok_req[t])
            if r < 0:
                continue
            p = int(tok_pos[t])
            page = int(table[r, p // g.page_size])
            slot = p % g.page_size
            pv[page, 0, :, slot, :] = qkv[t, g.k_off:g.k_off + kw].view(g.n_kv_heads, g.head_dim)
            pv[page, 1, :, slot, :] = qkv[t, g.v_off:g.v_off + kw].view(g.n_kv_heads, g.head_dim)

    def attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan=None):
        n = out.shape[0]
        pv = self._pool_view(pool, g)
        D, H, HK = g.head_dim, g.n_heads, g.n_kv_heads
        scale32 = float(torch.tensor(scale, dtype=torch.float32))
        for t in range(n):
            r = int(tok_req[t])
            if r < 0:
                out[t] = 0
                continue
            p = int(tok_pos[t])
            lo = max(0, p - g.window + 1) if g.window > 0 else 0
            js = torch.arange(lo, p + 1)
            pages = table[r, (js // g.page_size).to(table.device)].long()
            slots = (js % g.page_size).to(table.device)
            k = pv[pages, 0, :, slots, :].to(self.cd)       # [n_keys, HK, D]
            v = pv[pages, 1, :, slots, :].to(self.cd)
            q = qkv[t, g.q_off:g.q_off + H * D].view(H, D).to(self.cd)
            for h in range(H):
                hk = h // (H // HK)
                s = (k[:, hk, :] @ q[h]) * scale32
                pr = torch.softmax(s, 0)
                out[t, h * D:(h + 1) * D] = (pr @ v[:, hk, :]).to(out.dtype)

    def attention_append(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status,
                         plan=None, writes=True):
        if writes:
            self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
        self.attention(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan)

    def argmax(self, out, logits):
        rows = logits.shape[0]
        out[:rows] = torch.argmax(logits, dim=-1).to(torch.int32)

    def sample(self, out, logits, temperature, top_k, seed_lo, seed_hi, position,
               feedback=None, feedback_slot=None):
        for r in range(logits.shape[0]):
            seed = (int(seed_lo[r]) & 0xFFFFFFFF) | ((int(seed_hi[r]) & 0xFFFFFFFF) << 32)
            u = uniform_for(seed, int(position[r]))
            out[r] = sample_token(logits[r].cpu(), float(temperature[r]), int(top_k[r]), u)
            if feedback is not None and int(feedback_slot[r]) >= 0:
                feedback[int(feedback_slot[r])] = out[r]

    # -- twins of the kernels of the other parts (norm without statistics, rotary pairs,
    #    block-diagonal linear, attention over a shared latent, gated delta rule, routed
    #    experts) ------------------------------------------------------------------------
    def dyt_norm(self, out, x, weight, bias, alpha, rows=None):
        n = out.shape[0]
        src = x[rows[:n].long()] if rows is not None else x[:n]
        v = torch.tanh(alpha * src.to(self.cd)) * weight.to(self.cd) + bias.to(self.cd)
        out.copy_(v.to(out.dtype))

    def scale_(self, t, factor):
        t.mul_(factor)

    def rotary_pairs(self, buf, tok_pos, tok_req, freq, *, n_vec, vec_stride, offset, dims):
        half = dims // 2
        f = freq[:half].to(self.cd)
        for t in range(buf.shape[0]):
            if int(tok_req[t]) < 0:
                continue
            ang = float(tok_pos[t]) * f
            c, s = torch.cos(ang), torch.sin(ang)
            for v in range(n_vec):
                lo = offset + v * vec_stride
                seg = buf[t, lo:lo + dims].to(self.cd)
                a, b = seg[0::2].clone(), seg[1::2].clone()
                seg[0::2] = a * c - b * s
                seg[1::2] = b * c + a * s
                buf[t, lo:lo + dims] = seg.to(buf.dtype)

    def grouped_linear(self, out, a, w, *, a_offset=0, a_group_stride=None, w_nk=None, exact=False):
        groups, k, n = w.shape
        gs = k if a_group_stride is None else a_group_stride
        T = out.shape[0]
        for g in range(groups):
            lo = a_offset + g * gs
            v = a[:T, lo:lo + k].to(self.cd) @ w[g].to(self.cd)
            out[:, g * n:(g + 1) * n] = v.to(out.dtype)

    def _turned(self, vec, position, freq, rot_dims):
        """vec with the interleaved pairs of its first rot_dims entries rotated (a copy)."""
        out = vec.to(self.cd).clone()
        if freq is None or not rot_dims:
            return out
        ang = float(position) * freq[:rot_dims // 2].to(self.cd)
        c, s = torch.cos(ang), torch.sin(ang)
        a, b = out[0:rot_dims:2].clone(), out[1:rot_dims:2].clone()
        out[0:rot_dims:2] = a * c - b * s
        out[1:rot_dims:2] = b * c + a * s
        return out

    def latent_append(self, pool, proj, norm_w, table, tok_pos, tok_req, *, c_offset, rank,
                      rot_dim, eps, page_size, status, freq=None, rot_dims=0):
        rows = pool.view(-1, page_size, rank + rot_dim)
        for t in range(proj.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            p = int(tok_pos[t])
            page = int(table[r, p // page_size])
            c = proj[t, c_offset:c_offset + rank].to(self.cd)
            c = c / torch.sqrt((c * c).mean() + eps) * norm_w.to(self.cd)
            rows[page, p % page_size, :rank] = c.to(pool.dtype)
            kr = self._turned(proj[t, c_offset + rank:c_offset + rank + rot_dim], p, freq, rot_dims)
            rows[page, p % page_size, rank:] = kr.to(pool.dtype)

    def latent_attention(self, out, qa, qr, pool, table, tok_pos, tok_req, sink, *, n_heads,
                         rank, rot_dim, qr_head_stride, qr_offset, scale, page_size, status,
                         freq=None, rot_dims=0, plan=None):
        rows = pool.view(-1, page_size, rank + rot_dim)
        scale32 = float(torch.tensor(scale, dtype=torch.float32))
        for t in range(out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                out[t] = 0
                continue
            p = int(tok_pos[t])
            js = torch.arange(0, p + 1)
            keys = rows[table[r, js // page_size].long(), js % page_size].to(self.cd)
            c, kr = keys[:, :rank], keys[:, rank:]
            for h in range(n_heads):
                qh = qa[t, h * rank:(h + 1) * rank].to(self.cd)
                lo = qr_offset + h * qr_head_stride
                s = (c @ qh + kr @ self._turned(qr[t, lo:lo + rot_dim], p, freq, rot_dims)) * scale32
                top = torch.maximum(s.max(), sink[h].to(self.cd))
                e = torch.exp(s - top)
                den = e.sum() + torch.exp(sink[h].to(self.cd) - top)
                out[t, h * rank:(h + 1) * rank] = ((e / den) @ c).to(out.dtype)

    def delta_prepare(self, qn, kn, vv, beta, decay, proj, conv_w, a2, dt_bias, a_log, state,
                      tok_req, req_start, req_len, req_slot, shape, z_a=None):
        H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
        taps, ra = shape["taps"], shape["a_rank"]
        C = 2 * HK * D + H * V
        hist = taps - 1
        cw = conv_w.to(self.cd)
        for r in range(req_start.shape[0]):
            n, first = int(req_len[r]), int(req_start[r])
            if n <= 0:
                continue
            st = state[int(req_slot[r])]
            old = st[H * D * V:].view(hist, C).to(self.cd) if hist else torch.zeros(0, C)
            xs = torch.cat([old, proj[first:first + n, :C].to(self.cd)])      # [hist + n, C]
            for l in range(n):
                t = first + l
                y = (xs[l:l + taps] * cw.T).sum(0)
                y = y * torch.sigmoid(y)
                q = y[:HK * D].view(HK, D)
                k = y[HK * D:2 * HK * D].view(HK, D)
                q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
                k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
                qn[t] = q.reshape(-1).to(qn.dtype)
                kn[t] = k.reshape(-1).to(kn.dtype)
                vv[t] = y[2 * HK * D:].to(vv.dtype)
                row = proj[t].to(self.cd)
                beta[t] = torch.sigmoid(row[C:C + H]).to(beta.dtype)
                z = (row[C + H:C + H + ra] @ a2.to(self.cd) if z_a is None else z_a[t].to(self.cd)) \
                    + dt_bias.to(self.cd)                                        # a2 [ra, H*D]
                sp = torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))
                rate = torch.exp(a_log.to(self.cd)).repeat_interleave(D)
                decay[t] = torch.exp(-rate * sp).to(decay.dtype)
            if hist:
                st[H * D * V:] = xs[n:n + hist].reshape(-1).to(st.dtype)

    def delta_recurrence(self, o, state, qn, kn, vv, beta, decay, req_start, req_len, req_slot,
                         shape):
        H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
        for r in range(req_start.shape[0]):
            n, first = int(req_len[r]), int(req_start[r])
            if n <= 0:
                continue
            st = state[int(req_slot[r])]
            S = st[:H * D * V].view(H, D, V).to(self.cd)
            for t in range(first, first + n):
                for h in range(H):
                    kh = h // (H // HK)
                    k = kn[t, kh * D:(kh + 1) * D].to(self.cd)
                    q = qn[t, kh * D:(kh + 1) * D].to(self.cd)
                    S[h] = decay[t, h * D:(h + 1) * D].to(self.cd).view(D, 1) * S[h]
                    u = beta[t, h].to(self.cd) * (vv[t, h * V:(h + 1) * V].to(self.cd) - S[h].T @ k)
                    S[h] = S[h] + torch.outer(k, u)
                    o[t, h * V:(h + 1) * V] = (S[h].T @ q).to(o.dtype)
            st[:H * D * V] = S.reshape(-1).to(st.dtype)

    def delta_finish(self, out, o, proj, g2, norm_w, tok_req, eps, shape, z_g=None):
        H, HK, D, V = shape["heads"], shape["kv_heads"], shape["dim"], shape["vdim"]
        ra, rg = shape["a_rank"], shape["g_rank"]
        g_off = 2 * HK * D + H * V + H + ra
        T = out.shape[0]
        v = o[:T].to(self.cd).view(T, H, V)
        v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * norm_w.to(self.cd)
        zg = proj[:T, g_off:g_off + rg].to(self.cd) @ g2.to(self.cd) if z_g is None \
            else z_g[:T].to(self.cd)                                             # g2 [rg, H*V]
        gate = torch.sigmoid(zg)
        out.copy_((v.view(T, H * V) * gate).to(out.dtype))

    def moe_route(self, sel_idx, sel_w, h, w_router, tok_req, *, top, n_groups, keep, z=None):
        E = w_router.shape[0]
        per = E // n_groups
        for t in range(sel_idx.shape[0]):
            if int(tok_req[t]) < 0:
                continue
            s = torch.sigmoid(w_router.to(self.cd) @ h[t].to(self.cd) if z is None
                              else z[t].to(self.cd))
            gs = torch.topk(s.view(n_groups, per), min(2, per), dim=-1).values.sum(-1)
            kept = torch.zeros(n_groups, dtype=torch.bool)
            kept[torch.topk(gs, keep).indices] = True
            masked = torch.where(kept.repeat_interleave(per), s, torch.full_like(s, -1.0))
            idx = torch.topk(masked, top).indices
            sel_idx[t] = idx.to(torch.int32)
            sel_w[t] = (s[idx] / (s[idx].sum() + 1e-20)).to(sel_w.dtype)

    def moe_experts(self, x, y, h, w_gate, w_up, w_down, sel_idx, sel_w, tok_req, *, limit,
                    act="clamped"):
        T, top = sel_idx.shape
        if act == "relu2":
            for t in range(T):
                if int(tok_req[t]) < 0:
                    continue
                hv = h[t].to(self.cd)
                add = torch.zeros(x.shape[1], dtype=self.cd)
                for k in range(top):
                    e = int(sel_idx[t, k])
                    inner = torch.relu(w_up[e].to(self.cd) @ hv) ** 2
                    add = add + sel_w[t, k].to(self.cd) * (w_down[e].to(self.cd) @ inner)
                x[t] = (x[t].to(self.cd) + add).to(x.dtype)
            return
        if act == "silu":
            for t in range(T):
                if int(tok_req[t]) < 0:
                    continue
                hv = h[t].to(self.cd)
                add = torch.zeros(x.shape[1], dtype=self.cd)
                for k in range(top):
                    e = int(sel_idx[t, k])
                    g = w_gate[e].to(self.cd) @ hv
                    inner = g * torch.sigmoid(g) * (w_up[e].to(self.cd) @ hv)
                    add = add + sel_w[t, k].to(self.cd) * (w_down[e].to(self.cd) @ inner)
                x[t] = (x[t].to(self.cd) + add).to(x.dtype)
            return
        for t in range(T):
            if int(tok_req[t]) < 0:
                continue
            hv = h[t].to(self.cd)
            add = torch.zeros(x.shape[1], dtype=self.cd)
            for k in range(top):
                e = int(sel_idx[t, k])
                g = torch.clamp(w_gate[e].to(self.cd) @ hv, max=limit)
                u = torch.clamp(w_up[e].to(self.cd) @ hv, min=-limit, max=limit)
                act = g * torch.sigmoid(1.702 * g) * (u + 1.0)
                add = add + sel_w[t, k].to(self.cd) * (w_down[e].to(self.cd) @ act)
            x[t] = (x[t].to(self.cd) + add).to(x.dtype)

    def moe_route_top(self, sel_idx, sel_w, h, w_router, bias, tok_req, *, top, z=None):
        for t in range(sel_idx.shape[0]):
            if int(tok_req[t]) < 0:
                continue
            logits = (w_router.to(self.cd) @ h[t].to(self.cd)) if z is None else z[t].to(self.cd)
            if bias is not None:
                logits = logits + bias.to(self.cd)
            order = sorted(range(logits.shape[0]), key=lambda e: (-float(logits[e]), e))[:top]
            idx = torch.tensor(order)
            sel_idx[t] = idx.to(torch.int32)
            sel_w[t] = torch.softmax(logits[idx], 0).to(sel_w.dtype)

    def gated_act(self, out, gu, h=None, w_s=None, tok_req=None, act="silu"):
        ff = out.shape[1]
        v = gu.to(self.cd)
        r = _ACT[act](v[:, :ff]) * v[:, ff:]
        if w_s is not None:
            r = r * torch.sigmoid(h.to(self.cd) @ w_s.to(self.cd))[:, None]
        out.copy_(r.to(out.dtype))

    # -- root-mean-square norms, attention with a distance bias, lightning attention ----------
    def _rms(self, v, eps):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)

    def rms_norm(self, out, x, weight, eps, rows=None, one_plus=False, gate=None, gate_offset=0):
        n, width = out.shape
        sel = rows[:n].long() if rows is not None else torch.arange(n)
        w = weight.to(self.cd)
        v = self._rms(x[sel].to(self.cd), eps) * ((1.0 + w) if one_plus else w)
        if gate is not None:
            v = v * torch.sigmoid(gate[sel, gate_offset:gate_offset + width].to(self.cd))
        out.copy_(v.to(out.dtype))

    def rms_norm_add(self, x, a, weight, eps, h=None, b=None, wa=None, wb=None, mix=0.5,
                     eps_in=None, ln=None):
        n = x.shape[0]
        y = a[:n].to(self.cd)
        if b is not None:
            e_in = eps if eps_in is None else eps_in
            y = mix * (self._rms(y, e_in) * wa.to(self.cd)
                       + self._rms(b[:n].to(self.cd), e_in) * wb.to(self.cd))
        if weight is not None:
            y = self._rms(y, eps) * weight.to(self.cd)
        x.copy_((x.to(self.cd) + y).to(x.dtype))
        if h is not None and ln is not None:
            beta = ln[1] if ln[1] is not None else torch.zeros_like(ln[0])
            h.copy_(self._ln(x.to(self.cd), ln[0], beta, ln[2]).to(h.dtype))
        elif h is not None:
            h.copy_(x.to(h.dtype))

    def cast_rows(self, out, x):
        out.copy_(x.to(out.dtype).view_as(out))

    def qk_prepare(self, q_out, pool, proj, wq, wk, table, tok_pos, tok_req, *, q_off, k_off,
                   v_off, eps, writes, n_heads, n_kv_heads, head_dim, page_size, status):
        qw, kw = n_heads * head_dim, n_kv_heads * head_dim
        pv = pool.view(-1, 2, n_kv_heads, page_size, head_dim)
        for t in range(q_out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            row = proj[t].to(self.cd)
            q, k = row[q_off:q_off + qw], row[k_off:k_off + kw]
            v = k if v_off is None else row[v_off:v_off + kw]
            if wq is not None:
                q = self._rms(q, eps) * wq.to(self.cd)
            kn = self._rms(k, eps) * wk.to(self.cd) if wk is not None else k
            q_out[t] = q.to(q_out.dtype)
            if not writes:
                continue
            p = int(tok_pos[t])
            page = int(table[r, p // page_size])
            pv[page, 0, :, p % page_size] = kn.view(n_kv_heads, head_dim).to(pool.dtype)
            pv[page, 1, :, p % page_size] = v.view(n_kv_heads, head_dim).to(pool.dtype)

    def biased_attention(self, out, q, pool, table, tok_pos, tok_req, *, bias, gate, gate_offset,
                         n_heads, n_kv_heads, head_dim, page_size, scale, cap, chunk, window,
                         status, plan=None):
        pv = pool.view(-1, 2, n_kv_heads, page_size, head_dim)
        group = n_heads // n_kv_heads
        for t in range(out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            i = int(tok_pos[t])
            lo = i // chunk * chunk if chunk > 0 else 0
            if window > 0:
                lo = max(lo, i - window + 1)
            js = list(range(lo, i + 1))
            pages = [int(table[r, j // page_size]) for j in js]
            slots = [j % page_size for j in js]
            qt = q[t].to(self.cd).view(n_heads, head_dim)
            for hd in range(n_heads):
                g = hd // group
                keys = torch.stack([pv[pg, 0, g, sl] for pg, sl in zip(pages, slots)]).to(self.cd)
                vals = torch.stack([pv[pg, 1, g, sl] for pg, sl in zip(pages, slots)]).to(self.cd)
                s = (keys @ qt[hd]) * scale
                if cap > 0:
                    s = cap * torch.tanh(s / cap)
                if bias is not None:
                    dist = torch.tensor([min(i - j, bias.shape[1] - 1) for j in js])
                    s = s + bias[hd, dist].to(self.cd)
                o = torch.softmax(s, 0) @ vals
                if gate is not None:
                    o = o * torch.sigmoid(gate[t, gate_offset + hd].to(self.cd))
                out[t, hd * head_dim:(hd + 1) * head_dim] = o.to(out.dtype)

    def lightning_recurrence(self, o, state, proj, decay, req_start, req_len, req_slot, *, q_off,
                             k_off, v_off, heads, dim, vdim, act="silu", tok_pos=None,
                             freq=None, rot_dims=0, k_scale=1.0):
        f = _ACT[act]
        for r in range(req_start.shape[0]):
            n = int(req_len[r])
            if n <= 0:
                continue
            t0, slot = int(req_start[r]), int(req_slot[r])
            S = state[slot].to(self.cd).view(heads, dim, vdim).clone()
            for t in range(t0, t0 + n):
                row = proj[t].to(self.cd)
                q = f(row[q_off:q_off + heads * dim]).view(heads, dim)
                k = f(row[k_off:k_off + heads * dim]).view(heads, dim)
                v = f(row[v_off:v_off + heads * vdim]).view(heads, vdim)
                if freq is not None and rot_dims:
                    q = self._turn_halves(q, int(tok_pos[t]), freq, rot_dims)
                    k = self._turn_halves(k, int(tok_pos[t]), freq, rot_dims)
                k = k * k_scale
                for hd in range(heads):
                    S[hd] = decay[hd].to(self.cd) * S[hd] + torch.outer(k[hd], v[hd])
                    o[t, hd * vdim:(hd + 1) * vdim] = (S[hd].T @ q[hd]).to(o.dtype)
            state[slot] = S.reshape(-1).to(state.dtype)

    # -- layer norm behind a sublayer, learned activation, capped logits ------------------
    def _ln(self, v, gamma, beta, eps):
        c = v - v.mean(-1, keepdim=True)
        return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gamma.to(self.cd) \
            + beta.to(self.cd)

    def layernorm_add(self, x, y, gamma, beta, eps, out=None, out_gamma=None, out_beta=None,
                      out_eps=None):
        n = x.shape[0]
        new = x.to(self.cd) + self._ln(y[:n].to(self.cd), gamma, beta, eps)
        x.copy_(new.to(x.dtype))
        if out is not None and out_gamma is None:
            out.copy_(x.to(out.dtype))
        elif out is not None:
            out.copy_(self._ln(x.to(self.cd), out_gamma, out_beta, out_eps).to(out.dtype))

    def learned_act(self, out, z, act, values):
        assert act == "xielu"
        p, q = (torch.tensor(v, dtype=self.cd) for v in values)
        sp = torch.nn.functional.softplus
        v = z.to(self.cd)
        pos = sp(p) * v * v + 0.5 * v
        neg = (0.5 + sp(q)) * (torch.expm1(torch.clamp(v, max=0.0)) - v) + 0.5 * v
        out.copy_(torch.where(v > 0, pos, neg).to(out.dtype))

    def scale_softcap_(self, t, factor, cap):
        t.copy_((cap * torch.tanh(t.to(self.cd) * factor / cap)).to(t.dtype))

    # -- the real-gated linear recurrent unit ------------------------------------------------
    def rglru_conv(self, u, proj, conv_w, conv_b, state, tok_req, req_start, req_slot, *, x_off,
                   channels, taps):
        C = channels
        for t in range(u.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            local, slot = t - int(req_start[r]), int(req_slot[r])
            hist = state[slot, C:].view(taps - 1, C)            # oldest first
            acc = conv_b.to(self.cd).clone()
            for j in range(taps):
                if local - j >= 0:
                    src = proj[t - j, x_off:x_off + C]
                else:
                    src = hist[taps - 1 + (local - j)]
                acc = acc + conv_w[:, taps - 1 - j].to(self.cd) * src.to(self.cd)
            u[t] = acc.to(u.dtype)

    def rglru_scan(self, out, state, u, z, proj, b_gates, rate, req_start, req_len, req_slot, *,
                   channels, blocks, taps, decay_scale, y_off, x_off):
        C, n = channels, channels // blocks
        for r in range(req_start.shape[0]):
            cnt = int(req_len[r])
            if cnt <= 0:
                continue
            t0, slot = int(req_start[r]), int(req_slot[r])
            S = state[slot, :C].to(self.cd)
            for t in range(t0, t0 + cnt):
                zz = (z[t].to(self.cd) + b_gates.to(self.cd)).view(blocks, 2, n)
                rg = torch.sigmoid(zz[:, 0]).reshape(C)
                ig = torch.sigmoid(zz[:, 1]).reshape(C)
                log_a = -decay_scale * rg * rate.to(self.cd)
                a = torch.exp(log_a)
                S = a * S + torch.sqrt(-torch.expm1(2.0 * log_a)) * ig * u[t].to(self.cd)
                y = _ACT["gelu_tanh"](proj[t, y_off:y_off + C].to(self.cd))
                out[t] = (S * y).to(out.dtype)
            state[slot, :C] = S.to(state.dtype)
            if taps > 1:
                old = state[slot, C:].view(taps - 1, C)
                rows = torch.cat([old, proj[t0:t0 + cnt, x_off:x_off + C].to(state.dtype)])
                state[slot, C:] = rows[-(taps - 1):].reshape(-1)

    # -- attention over a window and pooled blocks ---------------------------------------------
    def _turn_halves(self, vec, position, freq, dims, sign=1.0):
        out = vec.to(self.cd).clone()
        if freq is None or not dims:
            return out
        half = dims // 2
        ang = sign * float(position) * freq[:half].to(self.cd)
        c, s = torch.cos(ang), torch.sin(ang)
        lo, hi = out[..., :half].clone(), out[..., half:dims].clone()
        out[..., :half] = lo * c - hi * s
        out[..., half:dims] = hi * c + lo * s
        return out

    def pooled_prepare(self, q_out, pool, proj, wq, wk, freq_qk, freq_v, table, tok_pos, tok_req,
                       *, n_heads, n_kv_heads, head_dim, value_dim, rot_dims, eps, writes,
                       page_size, status):
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        rows = pool.view(-1, G, page_size, D + V)
        for t in range(q_out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            p = int(tok_pos[t])
            row = proj[t].to(self.cd)
            q = row[:H * D].view(H, D)
            k = row[H * D:(H + G) * D].view(G, D)
            v = row[(H + G) * D:(H + G) * D + G * V].view(G, V)
            if wq is not None:
                q = self._rms(q, eps) * wq.to(self.cd)
            if wk is not None:
                k = self._rms(k, eps) * wk.to(self.cd)
            q_out[t] = self._turn_halves(q, p, freq_qk, rot_dims).reshape(-1).to(q_out.dtype)
            if not writes:
                continue
            k = self._turn_halves(k, p, freq_qk, rot_dims)
            v = self._turn_halves(v, p, freq_v, V if freq_v is not None else 0)
            page = int(table[r, p // page_size])
            rows[page, :, p % page_size] = torch.cat([k, v], dim=1).to(pool.dtype)

    def pooled_means(self, coarse_pool, coarse_table, pool, table, tok_pos, tok_req, *,
                     n_kv_heads, row, block, page_size, status):
        src = pool.view(-1, n_kv_heads, page_size, row)
        dst = coarse_pool.view(-1, n_kv_heads, page_size, row)
        for t in range(tok_pos.shape[0]):
            r, p = int(tok_req[t]), int(tok_pos[t])
            if r < 0 or (p + 1) % block:
                continue
            b = p // block
            acc = torch.zeros(n_kv_heads, row, dtype=self.cd)
            for j in range(b * block, p + 1):
                acc += src[int(table[r, j // page_size]), :, j % page_size].to(self.cd)
            dst[int(coarse_table[r, b // page_size]), :, b % page_size] = \
                (acc / block).to(coarse_pool.dtype)

    def pooled_attention(self, out, q, pool, table, coarse_pool, coarse_table, tok_pos, tok_req,
                         freq_v, *, n_heads, n_kv_heads, head_dim, value_dim, window, block,
                         scale, page_size, status, plan=None):
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        fine = pool.view(-1, G, page_size, D + V)
        coarse = coarse_pool.view(-1, G, page_size, D + V)
        for t in range(out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            i = int(tok_pos[t])
            seen = max(0, (i - window + 1) // block)
            first = max(0, i - window + 1)
            o = torch.zeros(H, V, dtype=self.cd)
            for g in range(G):
                rows = [coarse[int(coarse_table[r, b // page_size]), g, b % page_size]
                        for b in range(seen)]
                rows += [fine[int(table[r, j // page_size]), g, j % page_size]
                         for j in range(first, i + 1)]
                kv = torch.stack(rows).to(self.cd)
                for h in range(g * (H // G), (g + 1) * (H // G)):
                    qv = q[t, h * D:(h + 1) * D].to(self.cd)
                    w = torch.softmax((kv[:, :D] @ qv) * scale, 0)
                    o[h] = w @ kv[:, D:]
            if freq_v is not None:
                o = self._turn_halves(o, i, freq_v, V, sign=-1.0)
            out[t] = o.reshape(-1).to(out.dtype)

    # -- parts of the Mafuzen design ---------------------------------------------------------
    @staticmethod
    def _token(ids, t, feedback):
        tok = int(ids[t])
        return int(feedback[-(tok + 1)]) if tok < 0 and feedback is not None else tok

    def gather_mul(self, out, g, table, tok_ids, tok_req, *, col_offset, feedback=None):
        n, dim = out.shape
        for t in range(n):
            if int(tok_req[t]) < 0:
                continue
            e = table[self._token(tok_ids, t, feedback), col_offset:col_offset + dim]
            out[t] = (g[t].to(self.cd) * e.to(self.cd)).to(out.dtype)

    def moe_route_table(self, sel_idx, sel_w, table, tok_ids, tok_req, *, top, feedback=None,
                        experts=None):
        for t in range(sel_idx.shape[0]):
            if int(tok_req[t]) < 0:
                continue
            sel_idx[t] = table[self._token(tok_ids, t, feedback), :top].to(torch.int32)
            sel_w[t] = 1.0 / top

    def head_norm_gate(self, out, o, weight, gate, *, gate_offset, heads, dim, eps,
                       gate_act="silu", out_scale=1.0):
        n = out.shape[0]
        v = self._rms(o[:n].to(self.cd).view(n, heads, dim), eps).reshape(n, heads * dim)
        if weight is not None:
            v = v * weight.to(self.cd)
        if gate is not None:
            v = v * _GATE[gate_act](gate[:n, gate_offset:gate_offset + heads * dim].to(self.cd))
        out.copy_((v * out_scale).to(out.dtype))

    def span_prepare(self, q_out, pool, proj, table, tok_pos, tok_req, *, n_heads, n_kv_heads,
                     head_dim, value_dim, q_off, k_off, v_off, qk_norm, eps, writes, page_size,
                     status):
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        pv = pool.view(-1, G, page_size, D + V)
        for t in range(q_out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            row = proj[t].to(self.cd)
            q = row[q_off:q_off + H * D].view(H, D)
            q_out[t] = (self._rms(q, eps) if qk_norm else q).reshape(-1).to(q_out.dtype)
            if not writes:
                continue
            k = row[k_off:k_off + G * D].view(G, D)
            v = k if v_off is None else row[v_off:v_off + G * V].view(G, V)
            kn = self._rms(k, eps) if qk_norm else k
            p = int(tok_pos[t])
            page = int(table[r, p // page_size])
            pv[page, :, p % page_size, :D] = kn.to(pool.dtype)
            pv[page, :, p % page_size, D:] = v.to(pool.dtype)

    def span_attention(self, out, q, pool, table, tok_pos, tok_req, *, n_heads, n_kv_heads,
                       head_dim, value_dim, scale, slopes, window, keep_first, gate, gate_offset,
                       out_scale, page_size, status, plan=None):
        H, G, D, V = n_heads, n_kv_heads, head_dim, value_dim
        pv = pool.view(-1, G, page_size, D + V)
        for t in range(out.shape[0]):
            r = int(tok_req[t])
            if r < 0:
                continue
            i = int(tok_pos[t])
            first = max(0, i - window + 1) if window > 0 else 0
            js = list(range(min(keep_first, first))) + list(range(first, i + 1))
            rows = torch.stack([pv[int(table[r, j // page_size]), :, j % page_size]
                                for j in js]).to(self.cd)                     # [keys, G, D + V]
            dist = torch.tensor([i - j for j in js], dtype=self.cd)
            qt = q[t].to(self.cd).view(H, D)
            for hd in range(H):
                g = hd // (H // G)
                s = (rows[:, g, :D] @ qt[hd]) * scale
                if slopes is not None:
                    s = s - slopes[hd].to(self.cd) * dist
                o = torch.softmax(s, 0) @ rows[:, g, D:]
                if gate is not None:
                    o = o * torch.sigmoid(
                        gate[t, gate_offset + hd * V:gate_offset + (hd + 1) * V].to(self.cd))
                out[t, hd * V:(hd + 1) * V] = (o * out_scale).to(out.dtype)

    def token_shift_mix(self, out, h, mu, state, tok_req, req_start, req_len, req_slot, *,
                        state_offset):
        W = h.shape[1]
        for r in range(req_start.shape[0]):
            n = int(req_len[r])
            if n <= 0:
                continue
            t0, slot = int(req_start[r]), int(req_slot[r])
            prev = state[slot, state_offset:state_offset + W].to(self.cd)
            for t in range(t0, t0 + n):
                cur = h[t].to(self.cd)
                for s in range(out.shape[0]):
                    out[s, t] = (cur + (prev - cur) * mu[s].to(self.cd)).to(out.dtype)
                prev = cur
            state[slot, state_offset:state_offset + W] = prev.to(state.dtype)

    def timemix_decay(self, out, low, w2t, w0):
        n = out.shape[0]
        lw = torch.tanh(low[:n].to(self.cd)) @ w2t.to(self.cd) + w0.to(self.cd)
        out.copy_(torch.exp(-torch.exp(lw)).to(out.dtype))

    def timemix_recurrence(self, o, state, r, k, v, w, u, req_start, req_len, req_slot, *,
                           heads, dim):
        H, D = heads, dim
        uu = u.to(self.cd).view(H, D)
        for q in range(req_start.shape[0]):
            n = int(req_len[q])
            if n <= 0:
                continue
            t0, slot = int(req_start[q]), int(req_slot[q])
            S = state[slot, :H * D * D].to(self.cd).view(H, D, D).clone()
            for t in range(t0, t0 + n):
                rt, kt, vt, wt = (a[t].to(self.cd).view(H, D) for a in (r, k, v, w))
                for hd in range(H):
                    kv = torch.outer(kt[hd], vt[hd])
                    o[t, hd * D:(hd + 1) * D] = ((S[hd] + uu[hd][:, None] * kv).T @ rt[hd]).to(o.dtype)
                    S[hd] = wt[hd][:, None] * S[hd] + kv
            state[slot, :H * D * D] = S.reshape(-1).to(state.dtype)
