"""Attention over cached latents, as a mixer (LatentAttentionSpec).

Per token the cache holds one row: the rotated key part that all heads share
(r numbers) followed by the normalised latent c (``kv_rank`` numbers); head h's
plain key W_uk[h] c and value W_uv[h] c are never written anywhere.  Because
q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c, a head's query is carried into
the latent's space instead, and because sum_j p_j W_uv[h] c_j = W_uv[h] sum_j p_j c_j
the value up-projection is applied after the weighted sum.  Both up-projections
are folded into their neighbours when the weights are bound:

    Q[h] = [ W_uq[h, rotated rows] ; W_uk[h]^T W_uq[h, plain rows] ]     (r + kv_rank rows)
    O[:, h] = [ 0 (r columns) | W_o[:, h] W_uv[h] ]                      (r + kv_rank columns)

(in 64-bit, rounded once to the weights' type), so the mixer is: one product
x -> c_q | c | k_rot, one kernel (both RMS norms, the rotation of k_rot, the
append), the product Q c_q, the rotation of q's first r features, attention with
ONE key/value head whose values are its keys (r + kv_rank features, window and
sink in the kernel), and the product with O, whose zero columns drop the weighted
sum of the rotated parts.  A layer without a down-projection of its own reads
another run step's cache with its own Q and O.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Mixer, PagedKVNeed, Runtime, TensorSpec, make_position, register_mixer


class LatentAttention(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.rope_dim <= 0 or spec.rope_dim % 2:
            raise ValueError("latent attention needs an even, positive rotated part")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.position = make_position(spec.position, runtime)
        fused = self.position.fused_rotation()
        if fused is None or fused[0] is None or fused[1] != spec.rope_dim or getattr(self.position, "amplitude", 1.0) != 1.0:
            raise ValueError("latent attention needs a plain rotation over the whole rotated part")
        self.key_dim = spec.rope_dim + spec.kv_rank          # a cache row: k_rot | c
        self.down: torch.Tensor = None                        # W_dq ; W_dkv
        self.q_norm: torch.Tensor = None
        self.kv_norm: torch.Tensor = None
        self.q_up: torch.Tensor = None                        # Q of the module's text, [H (r + c), q_rank]
        self.o_proj: torch.Tensor = None                      # O, [hidden, H (r + c)]
        self.sink: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s, n = self.spec, self.names
        out = [TensorSpec(n["q_down"], (s.q_rank, s.hidden_size)), TensorSpec(n["q_latent_norm"], (s.q_rank,)),
               TensorSpec(n["q_up"], (s.num_heads * (s.head_dim + s.rope_dim), s.q_rank))]
        if s.own_kv:
            out += [TensorSpec(n["kv_down"], (s.kv_rank + s.rope_dim, s.hidden_size)),
                    TensorSpec(n["kv_latent_norm"], (s.kv_rank,))]
        out += [TensorSpec(n["k_up"], (s.num_heads * s.head_dim, s.kv_rank)),
                TensorSpec(n["v_up"], (s.num_heads * s.value_dim, s.kv_rank)),
                TensorSpec(n["o_proj"], (s.hidden_size, s.num_heads * s.value_dim))]
        if s.sink:
            out.append(TensorSpec(n["sink"], (s.num_heads,), init=("normal", 0.0, 1.0)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s, n = self.spec, self.names
        H, d, r, e, c = s.num_heads, s.head_dim, s.rope_dim, s.value_dim, s.kv_rank
        w_dq = tensors[n["q_down"]]
        kind = w_dq.dtype
        mats = [w_dq] + ([tensors[n["kv_down"]].to(kind)] if s.own_kv else [])
        self.down = torch.cat(mats, dim=0).contiguous()
        self.q_norm = tensors[n["q_latent_norm"]].float().contiguous()
        self.kv_norm = tensors[n["kv_latent_norm"]].float().contiguous() if s.own_kv else None
        w_uq = tensors[n["q_up"]].double().view(H, d + r, s.q_rank)
        w_uk = tensors[n["k_up"]].double().view(H, d, c)
        w_uv = tensors[n["v_up"]].double().view(H, e, c)
        w_o = tensors[n["o_proj"]].double().view(s.hidden_size, H, e)
        carried = torch.einsum("hdc,hdq->hcq", w_uk, w_uq[:, :d, :])                   # W_uk[h]^T W_uq[h, plain]
        self.q_up = torch.cat([w_uq[:, d:, :], carried], dim=1).reshape(H * (r + c), s.q_rank).to(kind).contiguous()
        back = torch.einsum("nhe,hec->nhc", w_o, w_uv)                                # W_o[:, h] W_uv[h]
        zeros = torch.zeros(s.hidden_size, H, r, dtype=back.dtype, device=back.device)
        self.o_proj = torch.cat([zeros, back], dim=2).reshape(s.hidden_size, H * (r + c)).to(kind).contiguous()
        if s.sink:
            self.sink = tensors[n["sink"]].float().contiguous()

    def cache_need(self):
        s = self.spec
        kept = s.window if isinstance(s.cache_window, str) else s.cache_window
        return PagedKVNeed(num_kv_heads=1, head_dim=self.key_dim, window=kept, tied_values=True)

    def launch_key(self, ctx):
        splits = getattr(self.runtime.kernels, "decode_attention_splits", None)
        if splits is None:
            return None
        return (splits(ctx.num_seqs, self.spec.num_heads, 1, ctx.max_ctx_len),)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache):
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        H, r, kd = s.num_heads, s.rope_dim, self.key_dim
        writes = cache.writes
        if writes and not s.own_kv:
            raise ValueError("a layer without a key/value down-projection must read another run step's cache")
        inv_freq, _ = self.position.fused_rotation()
        down = self.down if writes else self.down[:s.q_rank]
        proj = ctx.workspace.get("latent.down", (T, down.shape[0]), rt.dtype)
        k.linear(x, down, proj)
        cq = ctx.workspace.get("latent.cq", (T, s.q_rank), rt.dtype)
        k.latent_prepare(proj, cq, cache.keys if writes else None, self.q_norm, self.kv_norm if writes else None,
                         s.norm_eps, inv_freq, s.q_rank, s.kv_rank, r, ctx.positions, ctx.seq_of_token,
                         ctx.tables[cache.group] if writes else None, cache.page_size, ctx.seq_rows)
        q_raw = ctx.workspace.get("latent.q_raw", (T, H * kd), rt.dtype)
        k.linear(cq, self.q_up, q_raw)
        q = ctx.workspace.get("attn.q", (T, H * kd), rt.dtype)
        k.heads_rotate_append(q_raw, q, None, None, inv_freq, r, 1.0, False, 0.0, ctx.positions, ctx.seq_of_token,
                              None, H, 1, kd, kd, cache.page_size, ctx.seq_rows)
        att = ctx.workspace.get("attn.out", (T, H * kd), rt.dtype)
        extra = {"sink": self.sink} if s.sink else {}
        k.attention(q, cache.keys, cache.values, att, ctx.tables[cache.group], ctx.q_start, ctx.ctx_len,
                    ctx.seq_of_token, ctx.positions, H, 1, kd, cache.page_size, s.scale, s.window, ctx.max_q_len,
                    ctx.max_ctx_len, ctx.min_q_len, ctx.seq_rows, **extra)
        return k.linear(att, self.o_proj, residual, residual=residual, defer=True)


register_mixer("latent_attention", LatentAttention, replace=True)
