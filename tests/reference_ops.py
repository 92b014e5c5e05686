"""Plain PyTorch restatements of the package's kernels, one per operation, with
the same call signatures as ``chibillm_b200.kernels.ops.CudaKernels``.

Two uses, both in tests only: each CUDA kernel is compared with its
restatement here; and the engine's logic (batching, paging, windows, the
scheduler) is exercised on a machine without a GPU by handing an instance of
:class:`ReferenceKernels` to the runtime in place of the CUDA kernels.  The
arithmetic is 32-bit throughout, results are rounded to the output's type.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


class ReferenceKernels:
    name = "reference"

    def __init__(self):
        self.calls = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def check_error_word(self):
        return None

    def embed(self, tokens, table, out):
        self._count("embed")
        out.copy_(table[tokens.long()].float())

    def rmsnorm(self, x, weight, eps, offset, out):
        self._count("rmsnorm")
        xf = x.float()
        n = xf.shape[-1]
        inv = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / n + eps)
        out.copy_(((xf * inv) * (weight.float() + offset)).to(out.dtype))

    def linear_partial(self, x, w, max_splits=0):
        return None

    def linear(self, x, w, out, residual=None, defer=False):
        self._count("linear")
        y = x.float() @ w.float().t()
        if residual is not None:
            y = residual + y
        out.copy_(y.to(out.dtype))

    def qk_norm_rope_append(self, qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, inv_freq,
                            rotary_dim, eps, norm_offset, positions, seq_of_token, block_table,
                            nq, nkv, d, page_size, seq_rows=None):
        self._count("qk_norm_rope_append")
        T = qkv.shape[0]
        qw, kw = nq * d, nkv * d
        append = k_cache is not None
        q = qkv[:, :qw].float().reshape(T, nq, d)

        def norm(x, w):
            if w is None:
                return x
            inv = torch.rsqrt((x * x).sum(-1, keepdim=True) / d + eps)
            return (x * inv) * (w.float() + norm_offset)

        def rotate(x):
            if not rotary_dim:
                return x
            half = rotary_dim // 2
            angle = positions.float()[:, None] * inv_freq[:half].float()[None, :]
            c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            lo, hi = x[..., :half], x[..., half:rotary_dim]
            return torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., rotary_dim:]], dim=-1)

        q_out.copy_(rotate(norm(q, q_norm_w)).reshape(T, qw).to(q_out.dtype))
        if not append:
            return
        k = rotate(norm(qkv[:, qw:qw + kw].float().reshape(T, nkv, d), k_norm_w))
        pos = positions.long()
        rows = seq_of_token.long() if seq_rows is None else seq_rows.long()[seq_of_token.long()]
        pages = block_table[rows, pos // page_size].long()
        assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
        slots = pos % page_size
        k_cache[pages, :, slots, :] = k.to(k_cache.dtype)
        if v_cache is not None:             # None: the values are the keys, the cache holds keys only
            v = qkv[:, qw + kw:qw + 2 * kw].float().reshape(T, nkv, d)
            v_cache[pages, :, slots, :] = v.to(v_cache.dtype)

    def attention(self, q, k_cache, v_cache, out, block_table, q_start, ctx_len, seq_of_token,
                  positions, nq, nkv, d, page_size, scale, window, max_q_len, max_ctx_len, min_q_len=0,
                  seq_rows=None, softcap=None, distance_bias=None, chunk=None, value_dim=None, sink=None,
                  kv_share=1):
        self._count("attention")
        T = q.shape[0]
        group = nq // nkv
        dv = d if value_dim is None else value_dim
        qf = q.float().reshape(T, nq, d)
        res = torch.zeros(T, nq, dv, dtype=torch.float32, device=q.device)
        for t in range(T):
            s = int(seq_of_token[t])
            if seq_rows is not None:
                s = int(seq_rows[s])
            p = int(positions[t])
            first = max(0, p - window + 1) if window else 0
            if chunk:
                first = max(first, p - p % chunk)
            idx = torch.arange(first, p + 1, device=q.device)
            pages = block_table[s, idx // page_size].long()
            assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "attention outside the pool"
            keys = k_cache[pages, :, idx % page_size, :].float()      # [n, nkv, d]
            vals = v_cache[pages, :, idx % page_size, :].float()
            for h in range(nq):
                g = h // group
                sc = (keys[:, g, :] @ qf[t, h]) * scale
                if softcap is not None:
                    sc = softcap * torch.tanh(sc / softcap)
                if distance_bias is not None:
                    r1, r2 = distance_bias
                    if r2 is None:
                        sc = sc - r1[h].float() * (p - idx).float()
                    else:
                        sc = sc - r1[h].float() * torch.log1p(r2[h].float() * (p - idx).float())
                if sink is not None:
                    pr = torch.softmax(torch.cat([sc, sink[h].float().reshape(1)]), dim=0)[:-1]
                else:
                    pr = torch.softmax(sc, dim=0)
                res[t, h] = pr @ vals[:, g // kv_share, :]
        out.copy_(res.reshape(T, nq * dv).to(out.dtype))

    # ---- the operations of layer_ops.cu
    def heads_rotate_append(self, qkv, q_out, k_cache, v_cache, inv_freq, rotary_dim, amplitude, unit_norm, eps,
                            positions, seq_of_token, block_table, nq, nkv, d, dv, page_size, seq_rows=None):
        self._count("heads_rotate_append")
        T = qkv.shape[0]

        def finish(x):
            if rotary_dim:
                half = rotary_dim // 2
                angle = positions.float()[:, None] * inv_freq[:half].float()[None, :]
                c, s = (torch.cos(angle) * amplitude)[:, None, :], (torch.sin(angle) * amplitude)[:, None, :]
                lo, hi = x[..., :half], x[..., half:rotary_dim]
                x = torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., rotary_dim:]], dim=-1)
            if unit_norm:
                x = x * torch.rsqrt((x * x).sum(-1, keepdim=True) / d + eps)
            return x

        q_out.copy_(finish(qkv[:, :nq * d].float().reshape(T, nq, d)).reshape(T, nq * d).to(q_out.dtype))
        if k_cache is None:
            return
        k = finish(qkv[:, nq * d:(nq + nkv) * d].float().reshape(T, nkv, d))
        v = qkv[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv].float().reshape(T, nkv, dv)
        pos = positions.long()
        rows = seq_of_token.long() if seq_rows is None else seq_rows.long()[seq_of_token.long()]
        pages = block_table[rows, pos // page_size].long()
        assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
        k_cache[pages, :, pos % page_size, :] = k.to(k_cache.dtype)
        v_cache[pages, :, pos % page_size, :] = v.to(v_cache.dtype)

    def _act(self, z, kind):
        t = z.clone()
        self.activation(t, kind)
        return t

    def combine_experts(self, y, route, acc, top, experts, weight):
        self._count("combine_experts")
        T = acc.shape[0]
        rows = route[experts + 1 + T * top:experts + 1 + 2 * T * top].long().view(T, top)
        total = torch.zeros_like(acc)
        for s in range(top):
            total += y[rows[:, s]]
        acc.add_(weight * total)

    def gated_activation(self, gate_up, bias, out, kind, interleaved=False):
        self._count("gated_activation")
        assert not interleaved
        n = out.shape[1]
        gu = gate_up.float() + (bias.float() if bias is not None else 0.0)
        out.copy_((self._act(gu[:, :n], kind) * gu[:, n:]).to(out.dtype))

    def route_words(self, pairs, experts):
        return 1

    def routed_experts(self, x, tokens, table, gate_up, down, acc, route, act, y, kind, weight, interleaved=False,
                       sorted_x=None):
        assert not interleaved
        self._count("routed_experts")
        F = down.shape[2]
        for t in range(x.shape[0]):
            total = torch.zeros_like(acc[t])
            for e in table[int(tokens[t])].tolist():
                gu = gate_up[e].float() @ x[t].float()
                hidden = (self._act(gu[:F], kind) * gu[F:]).to(x.dtype).float()
                total += down[e].float() @ hidden
            acc[t] += weight * total

    def layer_end(self, residual, delta, mult, side=None, y_in=None, norm=None, copy_out=None):
        self._count("layer_end")
        if delta is not None:
            residual.add_(mult * delta)
        if side is not None:
            tokens, table, offset, gate, proj, side_w, act, eps = side
            if y_in is None:
                e = table[tokens.long(), offset:offset + gate.shape[0]].float()
                y = (self._act(residual @ gate.float().t(), act) * e) @ proj.float().t()
            else:
                y = y_in
            residual.add_(mult * y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps) * side_w.float())
        if norm is not None:
            w, eps, offset, out = norm
            self.rmsnorm(residual, w, eps, offset, out)
        if copy_out is not None:
            copy_out.copy_(residual.to(copy_out.dtype))

    # ---- the operations of mixer_ops.cu
    def norm_rows(self, y, weight, bias, eps, offset, centered, residual=None, out=None):
        self._count("norm_rows")
        v = y.float()
        if centered:
            v = v - v.mean(-1, keepdim=True)
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * (weight.float() + offset)
        if bias is not None:
            v = v + bias.float()
        if residual is not None:
            residual.add_(v)
            v = residual
        if out is not None:
            out.copy_(v.to(out.dtype))

    def token_shift(self, residual, mix, state, q_start, seq_of_token, state_slots, out):
        self._count("token_shift")
        starts = q_start.tolist()
        for s in range(len(starts) - 1):
            a, b = starts[s], starts[s + 1]
            if a == b:
                continue
            slot = int(state_slots[s])
            x = residual[a:b]
            before = torch.cat([state[slot][None, :], x[:-1]], dim=0)
            out[a:b] = (x + (before - x) * mix.float()).to(out.dtype)
            state[slot] = x[-1]

    @staticmethod
    def _rotate_front(x, positions, inv_freq, rot):
        if not rot:
            return x
        half = rot // 2
        angle = positions.float()[:, None] * inv_freq[:half].float()[None, :]
        c, s = torch.cos(angle), torch.sin(angle)
        while c.dim() < x.dim():
            c, s = c[:, None], s[:, None]
        lo, hi = x[..., :half], x[..., half:rot]
        return torch.cat([lo * c - hi * s, hi * c + lo * s, x[..., rot:]], dim=-1)

    def latent_prepare(self, proj, cq, k_cache, q_norm, kv_norm, eps, inv_freq, q_rank, kv_rank, rot, positions,
                       seq_of_token, block_table, page_size, seq_rows=None):
        self._count("latent_prepare")
        p = proj.float()
        a = p[:, :q_rank]
        cq.copy_((a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps) * q_norm.float()).to(cq.dtype))
        if k_cache is None:
            return
        c = p[:, q_rank:q_rank + kv_rank]
        c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * kv_norm.float()
        shared = self._rotate_front(p[:, q_rank + kv_rank:q_rank + kv_rank + rot], positions, inv_freq, rot)
        pos = positions.long()
        rows = seq_of_token.long() if seq_rows is None else seq_rows.long()[seq_of_token.long()]
        pages = block_table[rows, pos // page_size].long()
        assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
        k_cache[pages, 0, pos % page_size, :] = torch.cat([shared, c], dim=-1).to(k_cache.dtype)

    def qkv_bias_norm_append(self, proj, q_out, k_cache, v_cache, bias, q_norm, k_norm, eps, inv_freq, rot, positions,
                             seq_of_token, block_table, nq, nkv, d, dv, page_size, seq_rows=None):
        self._count("qkv_bias_norm_append")
        T = proj.shape[0]
        qw, kw, vw = nq * d, nkv * d, nkv * dv
        append = k_cache is not None
        width = qw + (kw + vw if append else 0)
        p = proj[:, :width].float()
        if bias is not None:
            p = p + bias.float()[:width]

        def whole(x, w):
            if w is None:
                return x
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()

        q = self._rotate_front(whole(p[:, :qw], q_norm).reshape(T, nq, d), positions, inv_freq, rot)
        q_out.copy_(q.reshape(T, qw).to(q_out.dtype))
        if not append:
            return
        kk = self._rotate_front(whole(p[:, qw:qw + kw], k_norm).reshape(T, nkv, d), positions, inv_freq, rot)
        v = p[:, qw + kw:].reshape(T, nkv, dv)
        pos = positions.long()
        rows = seq_of_token.long() if seq_rows is None else seq_rows.long()[seq_of_token.long()]
        pages = block_table[rows, pos // page_size].long()
        assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
        k_cache[pages, :, pos % page_size, :] = kk.to(k_cache.dtype)
        v_cache[pages, :, pos % page_size, :] = v.to(v_cache.dtype)

    def sigmoid_gate(self, x, gate):
        self._count("sigmoid_gate")
        x.copy_((x.float() * torch.sigmoid(gate.float())).to(x.dtype))

    def recurrence_gates(self, proj, bias, floor, out, kw):
        self._count("recurrence_gates")
        q = proj[:, :kw].float()
        out[:, :kw] = q * torch.sigmoid(q)
        out[:, kw:2 * kw] = floor + (1.0 - floor) * torch.sigmoid(proj[:, kw:2 * kw].float() + bias)
        out[:, 2 * kw:] = proj[:, 2 * kw:].float()

    def gated_recurrence(self, qfv, state, o, q_start, state_slots, heads, d, e, max_q_len=0):
        self._count("gated_recurrence")
        starts = q_start.tolist()
        kw = heads * d
        for s in range(len(starts) - 1):
            slot = int(state_slots[s])
            S = state[slot]
            for t in range(starts[s], starts[s + 1]):
                q = qfv[t, :kw].view(heads, d)
                f = qfv[t, kw:2 * kw].view(heads, d)
                vt = qfv[t, 2 * kw:].view(heads, e)
                S = f[:, :, None] * S + (1.0 - f)[:, :, None] * vt[:, None, :]
                o[t] = torch.einsum("hde,hd->he", S, q).reshape(-1)
            state[slot] = S

    def router_top(self, logits, chosen, share):
        self._count("router_top")
        top = chosen.shape[1]
        best, idx = torch.topk(logits, top, dim=-1)
        chosen.copy_(idx.to(chosen.dtype))
        share.copy_(torch.softmax(best, dim=-1))

    def chosen_experts(self, x, chosen, share, up, down, acc, route, act, y, kind, sorted_x=None, gated=False,
                       interleaved=False, identity=0):
        self._count("chosen_experts")
        assert not interleaved
        F = down.shape[2]
        for t in range(x.shape[0]):
            total = torch.zeros_like(acc[t])
            for s in range(chosen.shape[1]):
                e = int(chosen[t, s])
                if identity and e >= up.shape[0] - 1:
                    total += share[t, s] * x[t].float()
                    continue
                z = up[e].float() @ x[t].float()
                hidden = (self._act(z[:F], kind) * z[F:]) if gated else self._act(z, kind)
                total += share[t, s] * (down[e].float() @ hidden.to(x.dtype).float())
            acc[t] += total

    # ---- the operations of hybrid_ops.cu
    def bigram_embed(self, residual, table, kept, tokens, positions, seq_of_token, q_start, state_slots, mul_prev,
                     mul_cur):
        self._count("bigram_embed")
        buckets = table.shape[0] - 1
        for s in range(state_slots.numel()):
            a, b = int(q_start[s]), int(q_start[s + 1])
            slot = int(state_slots[s])
            prev = int(kept[slot, 0])
            for t in range(a, b):
                tok = int(tokens[t])
                row = buckets if int(positions[t]) == 0 else (prev * mul_prev + tok * mul_cur) % buckets
                residual[t] += table[row].float()
                prev = tok
            if b > a:
                kept[slot, 0] = prev

    def stream_enter(self, x, x0, vec):
        self._count("stream_enter")
        if x0 is not None:
            x.add_(x0)
        if vec is not None:
            x.add_(vec)

    def add_weighted(self, acc, a, wa, b=None, wb=0.0):
        self._count("add_weighted")
        acc.add_(wa * a.view_as(acc))
        if b is not None:
            acc.add_(wb * b.view_as(acc))

    def heads_prepare_append(self, proj, q_out, k_cache, v_cache, bias, q_norm, k_norm, eps, inv_freq, rotary_dim,
                             positions, seq_of_token, block_table, nq, nk, nv, d, dv, page_size, seq_rows=None):
        self._count("heads_prepare_append")
        T = proj.shape[0]
        append = k_cache is not None
        width = nq * d + ((nk * d + nv * dv) if append else 0)
        row = proj[:, :width].float()
        if bias is not None:
            row = row + bias[:width].float()
        pos = positions.float()

        def finish(x, w):
            if w is not None:
                x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()
            if rotary_dim:
                half = rotary_dim // 2
                ang = pos[:, None] * inv_freq[:half].float()[None, :]
                c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                u, v = x[..., :half], x[..., half:rotary_dim]
                x = torch.cat([u * c - v * s_, v * c + u * s_, x[..., rotary_dim:]], -1)
            return x

        q_out.copy_(finish(row[:, :nq * d].reshape(T, nq, d), q_norm).reshape(T, nq * d).to(q_out.dtype))
        if append:
            k = finish(row[:, nq * d:nq * d + nk * d].reshape(T, nk, d), k_norm)
            v = row[:, nq * d + nk * d:].reshape(T, nv, dv)
            seqs = seq_of_token.long()
            rows = seq_rows.long()[seqs] if seq_rows is not None else seqs
            pages = block_table[rows, (positions // page_size).long()].long()
            assert (pages >= 0).all() and (pages < k_cache.shape[0]).all(), "append outside the pool"
            slots = (positions % page_size).long()
            k_cache[pages, :, slots, :] = k.to(k_cache.dtype)
            v_cache[pages, :, slots, :] = v.to(v_cache.dtype)

    def differential_combine(self, att, gate, lam, eps, out_scale, out, heads, dv, group):
        self._count("differential_combine")
        T = att.shape[0]
        a = att.float().view(T, heads // group, 2, group, dv)
        o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, heads, dv)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * out_scale
        if gate is not None:
            o = o * torch.sigmoid(gate.float())[:, :, None]
        out.copy_(o.reshape(T, heads * dv).to(out.dtype))

    def causal_conv(self, x, weight, bias, history, out, q_start, state_slots, max_q_len, activation=None,
                    weight_t=None):
        self._count("causal_conv")
        taps = weight.shape[1]
        keep = taps - 1
        for s in range(state_slots.numel()):
            a, b = int(q_start[s]), int(q_start[s + 1])
            slot = int(state_slots[s])
            past = history[slot, :keep].float() if keep else x.new_zeros((0, x.shape[1])).float()
            seq = torch.cat([past, x[a:b].float()], dim=0)
            y = torch.zeros(b - a, x.shape[1]) + (bias.float() if bias is not None else 0.0)
            for j in range(taps):
                y = y + weight[:, j].float() * seq[j:j + (b - a)]
            out[a:b] = (self._act(y, activation) if activation is not None else y).to(out.dtype)
            if keep:
                history[slot, :keep] = seq[seq.shape[0] - keep:].to(history.dtype)

    def state_space_scan(self, xbc, dt, dt_bias, a_log, skip, state, y, q_start, state_slots, heads, groups, e, n):
        self._count("state_space_scan")
        inner = heads * e
        per = heads // groups
        for s in range(state_slots.numel()):
            a, b = int(q_start[s]), int(q_start[s + 1])
            slot = int(state_slots[s])
            S = state[slot].clone()                              # [heads, e, n]
            for t in range(a, b):
                row = xbc[t].float()
                x = row[:inner].view(heads, e)
                B = row[inner:inner + groups * n].view(groups, n).repeat_interleave(per, 0)
                C = row[inner + groups * n:].view(groups, n).repeat_interleave(per, 0)
                step = torch.nn.functional.softplus(dt[t].float() + dt_bias)
                decay = torch.exp(-torch.exp(a_log) * step)
                S = decay[:, None, None] * S + (step[:, None] * x)[:, :, None] * B[:, None, :]
                y[t] = (torch.einsum("hen,hn->he", S, C) + skip[:, None] * x).reshape(-1)
            state[slot] = S

    def gated_group_rms(self, y, z, weight, eps, parts, out):
        self._count("gated_group_rms")
        T, W = y.shape
        v = y * torch.nn.functional.silu(z.float())
        v = v.view(T, parts, W // parts)
        v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
        out.copy_((v.reshape(T, W) * weight).to(out.dtype))

    def clamped_swish_gate(self, gate_up, out, limit, slope):
        self._count("clamped_swish_gate")
        n = out.shape[1]
        g = gate_up[:, :n].float().clamp(max=limit)
        u = gate_up[:, n:].float().clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(slope * g) * (u + 1.0)).to(out.dtype))

    def router_choose(self, logits, correction, chosen, share, group_count, group_keep, scale, last_choice=None):
        self._count("router_choose")
        T, n = logits.shape
        top = chosen.shape[1]
        s = torch.softmax(logits.float(), -1)
        choice = s + correction if correction is not None else s.clone()
        if group_count > 1 and group_keep < group_count:
            per = n // group_count
            best = choice.view(T, group_count, per).max(-1).values
            kept = best.topk(group_keep, -1).indices
            allow = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
            choice = choice.masked_fill(~allow.repeat_interleave(per, 1), float("-inf"))
        idx = choice.topk(top, -1).indices
        share.copy_(s.gather(1, idx) * scale)
        if last_choice is not None:
            idx = idx.clamp(max=last_choice)
        chosen.copy_(idx.to(chosen.dtype))

    def scaled_add_norm(self, residual, delta, vec, norm=None):
        self._count("scaled_add_norm")
        residual.add_(delta * vec if vec is not None else delta)
        if norm is not None:
            w, eps, offset, out = norm
            self.rmsnorm(residual, w, eps, offset, out)

    def side_gate(self, gate, tokens, table, offset, kind):
        e = table[tokens.long(), offset:offset + gate.shape[1]].float()
        gate.copy_((self._act(gate.float(), kind) * e).to(gate.dtype))

    def softcap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    def zero(self, x):
        x.zero_()

    def apply_table_updates(self, table, updates, capacity):
        n = int(updates[0])
        assert n <= capacity
        for i in range(n):
            row, index, page = (int(v) for v in updates[1 + 3 * i:4 + 3 * i])
            table[row, index] = page

    def swiglu(self, gate_up, out):
        self._count("swiglu")
        inter = out.shape[1]
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def scale(self, x, factor):
        self._count("scale")
        x.mul_(factor)

    def cast_rows(self, x, out, activation=None):
        out.copy_(x.to(out.dtype))
        if activation is not None:
            self.activation(out, activation)

    def add_row_vector(self, acc, vec):
        acc.add_(vec.float()[None, :])

    def activation(self, x, kind):
        self._count("activation")
        z = x.float()
        if kind == "gelu":
            y = 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))
        elif kind == "gelu_tanh":
            y = 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        elif kind == "silu":
            y = z / (1.0 + torch.exp(-z))
        elif kind == "relu":
            y = torch.clamp(z, min=0.0)
        elif kind == "relu2":
            y = torch.clamp(z, min=0.0) ** 2
        elif kind == "tanh":
            y = torch.tanh(z)
        else:
            raise ValueError(kind)
        x.copy_(y.to(x.dtype))

    def short_conv(self, x, weight, history, out, q_start, positions, state_slots, max_q_len, weight_t=None):
        """y_t = x_t + sum_j w[:, j] x_(t - taps + 1 + j); what lies before a step's
        first token comes from ``history`` [slots, taps - 1, D] (oldest first), which
        then takes the sequence's last taps - 1 inputs."""
        self._count("short_conv")
        taps = weight.shape[1]
        keep = taps - 1
        for s in range(state_slots.numel()):
            a, b = int(q_start[s]), int(q_start[s + 1])
            slot = int(state_slots[s])
            past = history[slot, :keep].float() if keep else x.new_zeros((0, x.shape[1])).float()
            seq = torch.cat([past, x[a:b].float()], dim=0)
            y = x[a:b].float().clone()
            for j in range(taps):
                y = y + weight[:, j].float() * seq[j:j + (b - a)]
            out[a:b] = y.to(out.dtype)
            if keep:
                history[slot, :keep] = seq[seq.shape[0] - keep:].to(history.dtype)

    def decay_logits(self, low, w2t, out):
        self._count("decay_logits")
        out.copy_(torch.tanh(low.float()) @ w2t.float())

    def delta_rule(self, proj, decay_logits, decay_bias, removal_bias, state, o, q_start, state_slots, heads, d,
                   rank, decay_scale, key_eps, max_q_len):
        """proj [T, 5 * heads * d + rank] = r | k | v | gate | removal | low; decay_logits
        [T, heads * d]; state [slots, heads, d, d] (value index first); o [T, heads * d]
        32-bit."""
        self._count("delta_rule")
        W = heads * d
        p = proj.float()
        decay = torch.exp(-decay_scale * torch.sigmoid(decay_logits.float() + decay_bias.float()))
        rate = torch.sigmoid(p[:, 4 * W:5 * W] + removal_bias.float())
        for s in range(state_slots.numel()):
            slot = int(state_slots[s])
            for t in range(int(q_start[s]), int(q_start[s + 1])):
                for h in range(heads):
                    c = slice(h * d, (h + 1) * d)
                    r, k, v = p[t, c], p[t, W + h * d:W + (h + 1) * d], p[t, 2 * W + h * d:2 * W + (h + 1) * d]
                    u = k / torch.sqrt((k * k).sum() + key_eps)
                    S = state[slot, h].t()
                    S = decay[t, c][:, None] * S - torch.outer(rate[t, c] * u, u @ S) + torch.outer(k, v)
                    state[slot, h] = S.t()
                    o[t, c] = S.t() @ r

    def gated_group_norm(self, x, gate, weight, eps, group, out):
        """out = x / rms(x over each run of ``group`` features) * weight * sigmoid(gate)."""
        self._count("gated_group_norm")
        T, W = x.shape
        xf = x.float().view(T, W // group, group)
        y = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
        out.copy_((y.view(T, W) * weight.float() * torch.sigmoid(gate.float())).to(out.dtype))

    def gather_rows(self, x, rows, out):
        self._count("gather_rows")
        out.copy_(x[rows.long()].to(out.dtype))

    def cast(self, x, out):
        out.copy_(x.reshape(out.shape).to(out.dtype))

    def add_into(self, acc, x):
        acc.add_(x.float().reshape(acc.shape))

    def sample(self, logits, temperature, uniform, out):
        self._count("sample")
        for r in range(logits.shape[0]):
            row = logits[r].float()
            T = float(temperature[r]) if temperature is not None else 0.0
            if not T > 0.0:
                best = row.max()
                out[r] = int(torch.nonzero(row == best)[0, 0])
                continue
            p = torch.exp((row - row.max()) / T).double()
            cdf = torch.cumsum(p, 0)
            target = float(uniform[r]) * float(cdf[-1])
            idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
            out[r] = min(idx, row.numel() - 1)
