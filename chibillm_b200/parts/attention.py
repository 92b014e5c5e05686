"""Causal grouped-query attention over the paged cache, as a mixer.

Order of operations (src/qwen/qwen_layer.cc:56-101, 20-52): one product gives
q | k | v (the three matrices are stacked, src/qwen/qwen_weights.cc:27-31);
every q and k head is RMS-normalised over its own features with one weight
shared by all heads; q and k are rotated; k and v are appended to the cache
before the scores are taken, so a token sees itself; softmax in 32-bit over
scale * (q . k); the output projection adds into the residual.

The part takes every size and constant from its spec: head counts, head size,
scale, window, the norm of q and k (or none), the position encoding (or none).
When its run step reads another step's cache, it computes q only and appends
nothing.

Options of the spec beyond that: a soft cap of the scores (c * tanh(s / c)), a
bias by distance taken off the capped score (r1[h] * ln(1 + r2[h] * (i - j)),
two learned numbers per query head, kept in 32-bit), and values tied to the
keys (one product gives q | k, the cache holds keys only and the kernels read
them as values too).

Further options: value heads of another size than query and key heads
(``value_dim``), attention inside blocks of ``chunk`` positions, a layer without
key and value projections that only ever reads another run step's cache
(``own_kv`` False), and a norm of q and k without a weight AFTER the rotation
(``unit_norm_eps``), also with a rotation whose cosines and sines carry an
amplitude.  The last two, and a value size of its own, take the plain order of
kernels: the q | k | v product, one kernel that rotates, normalises and appends,
attention, the output product.

A sink (``sink``: one learned number per query head in the softmax's denominator)
goes to the attention kernels as it is.  Biases on q, k and v, a norm of q and k
over their whole projections (all heads at once) and a sigmoid gate on the
concatenated heads (``biases``, ``whole_norm_eps``, ``output_gate``) take an order
of their own: one product gives q | k | v | gate, one kernel adds the biases,
normalises, rotates if there is a rotation, writes q and appends k and v, attention
follows, one kernel multiplies by sigmoid(gate), then the output product.

Several score maps per head (``query_maps``; two maps joined as a1 - lambda a2:
``differential``), a gate per head (``head_gate``), a bias linear in the distance and
biases together with a per-head norm take one more order: one product gives
q | k | v (| the heads' gates); one kernel adds the biases, normalises every q and k
head with the shared weight, rotates, writes q and appends k and v (the maps of a key
head are key heads of the cache that share one value head); attention follows, 32-bit
where maps are to be subtracted; one kernel joins the maps, normalises and gates; then
the output product.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import (Mixer, PagedKVNeed, Runtime, TensorSpec, make_position, register_mixer)


class PagedAttention(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.position = make_position(spec.position, runtime)
        self.qkv: torch.Tensor = None
        self.o_proj: torch.Tensor = None
        self.q_norm: torch.Tensor = None
        self.k_norm: torch.Tensor = None
        self.distance_r1: torch.Tensor = None
        self.distance_r2: torch.Tensor = None
        if spec.distance_bias not in (None, "log", "linear"):
            raise ValueError(f"distance bias '{spec.distance_bias}' is not supported (None, 'log' or 'linear')")
        self.maps = int(getattr(spec, "query_maps", 1))
        # the order of the module's last paragraph
        self.prepared = (self.maps > 1 or getattr(spec, "head_gate", False) or spec.distance_bias == "linear"
                         or (spec.biases and spec.qk_norm is not None))
        if self.prepared:
            if spec.tied_values or spec.unit_norm_eps is not None or spec.whole_norm_eps is not None \
                    or spec.output_gate or spec.softcap is not None or not spec.own_kv:
                raise ValueError("score maps, a gate per head, a linear distance bias and biases with a per-head "
                                 "norm are not combined with tied values, a norm after the rotation or over the "
                                 "whole projection, a gate per feature, a soft cap or a borrowed cache")
            if getattr(spec, "differential", None) is not None and self.maps != 2:
                raise ValueError("differential attention has two score maps per head")
            if self.maps > 1 and getattr(spec, "differential", None) is None:
                raise ValueError("several score maps need a rule that joins them (differential)")
            if getattr(spec, "head_gate", False) and self.maps == 1:
                raise ValueError("a gate per head is applied where the score maps are joined")
            if self.maps > 1 and spec.biases:
                raise ValueError("several score maps are not combined with biases")
        self.lam = 0.0
        self.slopes: torch.Tensor = None
        self.kv_arrays = 1 if spec.tied_values else 2
        self.value_dim = spec.head_dim if spec.value_dim is None else spec.value_dim
        if spec.tied_values and self.value_dim != spec.head_dim:
            raise ValueError("values tied to the keys have the keys' size")
        if spec.unit_norm_eps is not None and spec.qk_norm is not None:
            raise ValueError("a norm of q and k comes either before the rotation (qk_norm) or after it (unit_norm_eps)")
        if self.prepared:
            self.rotate_then_norm = self.bias_norm_gate = False
            self.bias = self.sink = None
            self.gate_columns = 0
            return
        # the plain order of kernels (see the module's text)
        self.rotate_then_norm = (spec.unit_norm_eps is not None or self.value_dim != spec.head_dim
                                 or getattr(self.position, "amplitude", 1.0) != 1.0)
        # biases, a norm over the whole projections or an output gate: the order of the module's last paragraph
        self.bias_norm_gate = spec.biases or spec.whole_norm_eps is not None or spec.output_gate
        if self.bias_norm_gate:
            if spec.tied_values or spec.qk_norm is not None or spec.unit_norm_eps is not None \
                    or getattr(self.position, "amplitude", 1.0) != 1.0:
                raise ValueError("biases, a norm over the whole projection and an output gate are not combined with "
                                 "tied values, a per-head norm or a rotation with an amplitude")
            self.rotate_then_norm = False
        if self.rotate_then_norm and (spec.tied_values or spec.qk_norm is not None):
            raise ValueError("tied values and a weighted norm before the rotation are not combined with a norm "
                             "after the rotation, an amplitude or a value size of its own")
        self.bias: torch.Tensor = None
        self.sink: torch.Tensor = None
        self.gate_columns = 0

    # ---- weights
    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        qw, kw = s.num_heads * self.maps * s.head_dim, s.num_kv_heads * self.maps * s.head_dim
        out = [TensorSpec(self.names["q_proj"], (qw, s.hidden_size))]
        if s.own_kv:
            out.append(TensorSpec(self.names["k_proj"], (kw, s.hidden_size)))
            if not s.tied_values:
                out.append(TensorSpec(self.names["v_proj"], (s.num_kv_heads * self.value_dim, s.hidden_size)))
        out.append(TensorSpec(self.names["o_proj"], (s.hidden_size, s.num_heads * self.value_dim)))
        if getattr(s, "differential", None) is not None:
            out += [TensorSpec(self.names[r], (s.head_dim,), init=("normal", 0.0, 0.1))
                    for r in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2")]
        if getattr(s, "head_gate", False):
            out.append(TensorSpec(self.names["head_gate"], (s.num_heads, s.hidden_size)))
        if s.distance_bias == "log":
            out += [TensorSpec(self.names["distance_r1"], (s.num_heads,), init=("uniform", 0.0, 2.0)),
                    TensorSpec(self.names["distance_r2"], (s.num_heads,), init=("uniform", 0.1, 0.5))]
        if s.qk_norm is not None:
            out += [TensorSpec(self.names["q_norm"], (s.qk_norm.size,)),
                    TensorSpec(self.names["k_norm"], (s.qk_norm.size,))]
        if s.biases:
            out.append(TensorSpec(self.names["q_bias"], (qw,), init=("normal", 0.0, 0.1)))
            if s.own_kv:
                out += [TensorSpec(self.names["k_bias"], (kw,), init=("normal", 0.0, 0.1)),
                        TensorSpec(self.names["v_bias"], (s.num_kv_heads * self.value_dim,), init=("normal", 0.0, 0.1))]
        if s.whole_norm_eps is not None:
            out.append(TensorSpec(self.names["q_norm"], (qw,)))
            if s.own_kv:
                out.append(TensorSpec(self.names["k_norm"], (kw,)))
        if s.output_gate:
            out.append(TensorSpec(self.names["g_proj"], (s.num_heads * self.value_dim, s.hidden_size)))
        if s.sink:
            out.append(TensorSpec(self.names["sink"], (s.num_heads,), init=("normal", 0.0, 1.0)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        roles = ("q_proj", "k_proj") if self.spec.tied_values else ("q_proj", "k_proj", "v_proj")
        if not self.spec.own_kv:
            roles = ("q_proj",)
        if self.spec.output_gate:
            roles = roles + ("g_proj",)
            self.gate_columns = tensors[self.names["g_proj"]].shape[0]
        if getattr(self.spec, "head_gate", False):
            roles = roles + ("head_gate",)
            self.gate_columns = tensors[self.names["head_gate"]].shape[0]
        if getattr(self.spec, "differential", None) is not None:
            lq1, lk1, lq2, lk2 = (tensors[self.names[r]].float() for r in ("lambda_q1", "lambda_k1", "lambda_q2",
                                                                              "lambda_k2"))
            # one number for the layer, made once in 32-bit
            self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())
                             + torch.tensor(float(self.spec.differential)))
        if self.spec.distance_bias == "linear":
            H = self.spec.num_heads
            self.slopes = torch.tensor([2.0 ** (-float(self.spec.distance_slope_bits) * (h + 1) / H)
                                        for h in range(H)], dtype=torch.float32,
                                       device=tensors[self.names["q_proj"]].device)
        mats = [tensors[self.names[r]] for r in roles]
        if self.maps > 1:
            # Query rows come head by head, a head's maps side by side; a key head of the cache is one map
            # of one key/value head.  The attention kernels give query head i key head i // (heads per key
            # head), so the rows are put in the order (key/value head, map, head of the group).
            s, M = self.spec, self.maps
            G, R, d = s.num_kv_heads, s.num_heads // s.num_kv_heads, s.head_dim
            mats[0] = mats[0].view(G, R, M, d, -1).permute(0, 2, 1, 3, 4).reshape(mats[0].shape)
        self.qkv = torch.cat([m.to(mats[0].dtype) for m in mats], dim=0).contiguous()
        if self.spec.sink:
            self.sink = tensors[self.names["sink"]].float().contiguous()
        if self.spec.biases:
            parts = ("q_bias", "k_bias", "v_bias") if self.spec.own_kv else ("q_bias",)
            self.bias = torch.cat([tensors[self.names[r]].float() for r in parts]).contiguous()
        if self.spec.whole_norm_eps is not None:
            self.q_norm = tensors[self.names["q_norm"]].float().contiguous()
            self.k_norm = tensors[self.names["k_norm"]].float().contiguous() if self.spec.own_kv else None
        if self.spec.distance_bias == "log":
            self.distance_r1 = tensors[self.names["distance_r1"]].float().contiguous()
            self.distance_r2 = tensors[self.names["distance_r2"]].float().contiguous()
        self.o_proj = tensors[self.names["o_proj"]].contiguous()
        if self.spec.qk_norm is not None:
            self.q_norm = tensors[self.names["q_norm"]].contiguous()
            self.k_norm = tensors[self.names["k_norm"]].to(self.q_norm.dtype).contiguous()
            if self.prepared:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    # ---- cache
    accepts_scaled_rows = True       # x goes to the q | k | v product and nowhere else

    def cache_need(self):
        s = self.spec
        kept = s.window if isinstance(s.cache_window, str) else s.cache_window
        return PagedKVNeed(num_kv_heads=s.num_kv_heads * self.maps, head_dim=s.head_dim, window=kept,
                           tied_values=s.tied_values,
                           value_dim=self.value_dim if self.value_dim != s.head_dim else None,
                           value_heads=s.num_kv_heads if self.maps > 1 else None)

    def launch_key(self, ctx):
        if self.position.fused_rotation() is None:
            return None                      # an encoding of its own: nothing is promised
        if self.prepared:
            return ()                        # the plain attention kernel: nothing is decided on the host
        k = self.runtime.kernels
        splits = getattr(k, "decode_attention_splits", None)
        if splits is None:
            return None
        s = self.spec
        return (splits(ctx.num_seqs, s.num_heads, s.num_kv_heads, ctx.max_ctx_len),)

    # ---- run
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache) -> None:
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        qw, kw = nq * d, nkv * d
        writes = cache.writes
        if writes and not s.own_kv:
            raise ValueError("a layer without key and value projections must read another run step's cache")
        if self.prepared:
            return self._prepared_attend(x, residual, ctx, cache)
        if self.bias_norm_gate:
            return self._bias_norm_gate_attend(x, residual, ctx, cache)
        if self.rotate_then_norm:
            return self._rotate_norm_attend(x, residual, ctx, cache)
        width = qw + self.kv_arrays * kw if writes else qw
        modified = s.softcap is not None or s.distance_bias is not None or s.chunk is not None or s.sink
        fused = self.position.fused_rotation()
        if fused is not None and fused[0] is not None and self._heads_from_the_product(x, ctx, cache, fused):
            return self._attend(residual, ctx, cache)
        split = getattr(k, "linear_partial", None)
        pending = None
        if split is not None and fused is not None and d % 4 == 0:
            # the kernels that add these sums up (decode attention; norm + rotation + append) fetch
            # eight splits of a head in one go
            pending = split(x, self.qkv if writes else self.qkv[:qw], max_splits=8)
        if pending is None:
            qkv = ctx.workspace.get("attn.qkv", (T, width), rt.dtype)
            k.linear(x, self.qkv if writes else self.qkv[:qw], qkv)

        q = ctx.workspace.get("attn.q", (T, qw), rt.dtype)
        table = ctx.tables[cache.group]
        norm = s.qk_norm
        q_norm_w = self.q_norm if norm is not None else None
        k_norm_w = self.k_norm if norm is not None else None
        att = ctx.workspace.get("attn.out", (T, qw), rt.dtype)
        from_partial = getattr(k, "attention_decode_from_partial", None)
        if pending is not None and ctx.max_q_len == 1 and from_partial is not None and fused[0] is not None \
                and not modified and not s.tied_values:
            # every sequence brings one token: the attention kernel finishes the product itself
            if from_partial(pending, cache.keys, cache.values, att, table, ctx.q_start, ctx.ctx_len, nq, nkv, d,
                            cache.page_size, s.scale, s.window, ctx.max_ctx_len, q_norm_w, k_norm_w, fused[0],
                            fused[1], norm.eps if norm is not None else 0.0,
                            norm.weight_offset if norm is not None else 0.0, writes, ctx.seq_rows):
                return k.linear(att, self.o_proj, residual, residual=residual, defer=True)
        if fused is None:
            # An encoding the kernels do not know: normalise head by head in
            # place, let the encoding transform q and k, then only copy and append.
            if norm is not None:
                heads = nq + (nkv if writes else 0)
                for h in range(heads):
                    view = qkv[:, h * d:(h + 1) * d]
                    k.rmsnorm(view, self.q_norm if h < nq else self.k_norm, norm.eps,
                              norm.weight_offset, view)
            self.position.apply(qkv[:, :qw], qkv[:, qw:qw + kw] if writes else None, ctx)
            q_norm_w = k_norm_w = None
            fused = (None, 0)
        inv_freq, rotary_dim = fused
        (k.qk_norm_rope_append_partial if pending is not None else k.qk_norm_rope_append)(
            pending if pending is not None else qkv, q, cache.keys if writes else None,
            cache.values if writes and not s.tied_values else None,
            q_norm_w, k_norm_w, inv_freq, rotary_dim, norm.eps if norm is not None else 0.0,
            norm.weight_offset if norm is not None else 0.0,
            ctx.positions, ctx.seq_of_token, table if writes else None, nq, nkv, d, cache.page_size,
            ctx.seq_rows)
        return self._attend(residual, ctx, cache)

    def _rotate_norm_attend(self, x, residual, ctx, cache):
        """The plain order: q | k | v product; per head rotation (with the encoding's
        amplitude), then the norm without a weight; append; attention; output product."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        nq, nkv, d, dv = s.num_heads, s.num_kv_heads, s.head_dim, self.value_dim
        writes = cache.writes
        fused = self.position.fused_rotation()
        if fused is None:
            raise ValueError("a norm after the rotation needs a rotation that the kernels apply themselves")
        inv_freq, rotary_dim = fused
        w = self.qkv if writes else self.qkv[:nq * d]
        qkv = ctx.workspace.get("attn.qkv", (T, w.shape[0]), rt.dtype)
        k.linear(x, w, qkv)
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        k.heads_rotate_append(qkv, q, cache.keys if writes else None, cache.values if writes else None, inv_freq,
                              rotary_dim if inv_freq is not None else 0, getattr(self.position, "amplitude", 1.0),
                              s.unit_norm_eps is not None, s.unit_norm_eps or 0.0, ctx.positions, ctx.seq_of_token,
                              ctx.tables[cache.group] if writes else None, nq, nkv, d, dv, cache.page_size,
                              ctx.seq_rows)
        return self._attend(residual, ctx, cache)

    def _prepared_attend(self, x, residual, ctx, cache):
        """q | k | v (| gates) from one product; biases, per-head norm, rotation and append in one
        kernel; attention with the maps of a head as heads of their own that share the head's
        values; the maps joined, normalised and gated; the output product."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        M = self.maps
        nq, nk, nv, d, dv = s.num_heads * M, s.num_kv_heads * M, s.num_kv_heads, s.head_dim, self.value_dim
        inv_freq, rotary_dim = self.position.fused_rotation() or (None, 0)
        if inv_freq is None and s.position.kind != "none":
            raise ValueError("this order of kernels needs a rotation that the kernels apply")
        proj = ctx.workspace.get("attn.qkv", (T, self.qkv.shape[0]), rt.dtype)
        k.linear(x, self.qkv, proj)
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        norm = s.qk_norm
        table = ctx.tables[cache.group]
        k.heads_prepare_append(proj, q, cache.keys, cache.values, self.bias,
                               self.q_norm if norm is not None else None, self.k_norm if norm is not None else None,
                               norm.eps if norm is not None else 0.0, inv_freq,
                               rotary_dim if inv_freq is not None else 0, ctx.positions, ctx.seq_of_token, table,
                               nq, nk, nv, d, dv, cache.page_size, ctx.seq_rows)
        extra = {}
        if s.chunk is not None:
            extra["chunk"] = s.chunk
        if dv != d:
            extra["value_dim"] = dv
        if s.sink:
            extra["sink"] = self.sink
        if s.distance_bias == "linear":
            extra["distance_bias"] = (self.slopes, None)
        if M > 1:
            extra["kv_share"] = M
        joined = M > 1
        att = ctx.workspace.get("attn.maps" if joined else "attn.out", (T, nq * dv),
                                torch.float32 if joined else rt.dtype)
        k.attention(q, cache.keys, cache.values, att, table, ctx.q_start, ctx.ctx_len, ctx.seq_of_token,
                    ctx.positions, nq, nk, d, cache.page_size, s.scale, s.window, ctx.max_q_len, ctx.max_ctx_len,
                    ctx.min_q_len, ctx.seq_rows, **extra)
        if joined:
            out = ctx.workspace.get("attn.out", (T, s.num_heads * dv), rt.dtype)
            gate = proj[:, proj.shape[1] - self.gate_columns:] if self.gate_columns else None
            k.differential_combine(att, gate, self.lam, s.differential_eps, 1.0 - float(s.differential), out,
                                   s.num_heads, dv, s.num_heads // s.num_kv_heads)
            att = out
        return k.linear(att, self.o_proj, residual, residual=residual, defer=True)

    def _bias_norm_gate_attend(self, x, residual, ctx, cache):
        """q | k | v | gate from one product; biases, the norm over the whole q and k,
        a rotation if the encoding has one, and the append in one kernel; attention;
        the heads times sigmoid(gate); the output product."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        nq, nkv, d, dv = s.num_heads, s.num_kv_heads, s.head_dim, self.value_dim
        writes = cache.writes
        inv_freq, rotary_dim = self.position.fused_rotation() or (None, 0)
        if inv_freq is None and s.position.kind != "none":
            raise ValueError("biases, a whole norm or an output gate need a rotation that the kernels apply")
        proj = ctx.workspace.get("attn.qkv", (T, self.qkv.shape[0]), rt.dtype)
        k.linear(x, self.qkv, proj)
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        k.qkv_bias_norm_append(proj, q, cache.keys if writes else None, cache.values if writes else None, self.bias,
                               self.q_norm, self.k_norm, s.whole_norm_eps, inv_freq,
                               rotary_dim if inv_freq is not None else 0, ctx.positions, ctx.seq_of_token,
                               ctx.tables[cache.group] if writes else None, nq, nkv, d, dv, cache.page_size,
                               ctx.seq_rows)
        gate = proj[:, proj.shape[1] - self.gate_columns:] if self.gate_columns else None
        return self._attend(residual, ctx, cache, gate)

    def _attend(self, residual, ctx, cache, gate=None):
        """Attention over the cache from the step's q, then the output product, left
        for the next norm to add into the residual."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        T = ctx.num_tokens
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        att = ctx.workspace.get("attn.out", (T, nq * self.value_dim), rt.dtype)
        extra = {}
        if s.softcap is not None or s.distance_bias is not None:
            extra = {"softcap": s.softcap, "distance_bias": (self.distance_r1, self.distance_r2)
                     if s.distance_bias is not None else None}
        if s.chunk is not None:
            extra["chunk"] = s.chunk
        if self.value_dim != d:
            extra["value_dim"] = self.value_dim
        if s.sink:
            extra["sink"] = self.sink
        k.attention(q, cache.keys, cache.values, att, ctx.tables[cache.group], ctx.q_start, ctx.ctx_len,
                    ctx.seq_of_token, ctx.positions, nq, nkv, d, cache.page_size, s.scale,
                    s.window, ctx.max_q_len, ctx.max_ctx_len, ctx.min_q_len, ctx.seq_rows, **extra)
        if gate is not None:
            k.sigmoid_gate(att, gate)
        return k.linear(att, self.o_proj, residual, residual=residual, defer=True)

    def _heads_from_the_product(self, x, ctx, cache, fused) -> bool:
        """Many rows on kernels that can do it: the q | k | v product normalises and
        rotates its heads itself and writes q and the cache entries; no q | k | v
        array exists.  The rotation table and the tokens' cache slots are made once
        per step and shared by the layers."""
        s, rt = self.spec, self.runtime
        k = rt.kernels
        takes = getattr(k, "finishes_heads", None)
        T = ctx.num_tokens
        nq, nkv, d = s.num_heads, s.num_kv_heads, s.head_dim
        if takes is None or s.tied_values or not takes(T, d, fused[1], rt.dtype):
            return False
        cos_sin = self.position.step_table(ctx)
        if cos_sin is None:
            return False
        writes = cache.writes
        slots = None
        if writes:
            key = ("cache slots", cache.group, nkv, d, cache.page_size)
            slots = ctx.shared.get(key)
            if slots is None:
                slots = ctx.workspace.get(f"attn.slots.{cache.group}", (T,), torch.int64)
                k.cache_slots(ctx.positions, ctx.seq_of_token, ctx.seq_rows, ctx.tables[cache.group], nkv,
                              cache.page_size, cache.keys.shape[0], d, slots)
                ctx.shared[key] = slots
        norm = s.qk_norm
        q = ctx.workspace.get("attn.q", (T, nq * d), rt.dtype)
        return k.linear_heads(x, self.qkv if writes else self.qkv[:nq * d], q, cache.keys if writes else None,
                              cache.values if writes else None, self.q_norm if norm is not None else None,
                              self.k_norm if norm is not None else None, cos_sin, slots, nq, nkv, d,
                              cache.page_size, norm.eps if norm is not None else 0.0,
                              norm.weight_offset if norm is not None else 0.0)


register_mixer("attention", PagedAttention, replace=True)
