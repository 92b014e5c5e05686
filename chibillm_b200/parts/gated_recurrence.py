"""A gated linear recurrence as a mixer (GatedRecurrenceSpec): linear attention in
which the forget gate also decides what is written.

One product gives q | f | v for all heads.  A first kernel makes the recurrence's
inputs in 32-bit: silu(q), the gate f = l + (1 - l) * sigmoid(f + b) with its
lower bound l per channel, and v.  The recurrence kernel then runs, per head,

    S <- diag(f) S + (1 - f) v^T,   o = S^T q

over the step's tokens of every sequence, from the state that the request's slot
holds to the state it leaves there (32-bit, [heads, key channel, value channel]).
Each head's o is divided by its root mean square and multiplied by a weight that
the heads share; the output product adds into the residual.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FixedStateNeed, Mixer, Runtime, TensorSpec, register_mixer


class GatedRecurrence(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.stacked: torch.Tensor = None        # q | f | v
        self.gate_bias: torch.Tensor = None
        self.gate_floor: torch.Tensor = None
        self.norm_weight: torch.Tensor = None
        self.o_proj: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s, n = self.spec, self.names
        kw, vw = s.num_heads * s.head_dim, s.num_heads * s.value_dim
        return [TensorSpec(n["q_proj"], (kw, s.hidden_size)), TensorSpec(n["f_proj"], (kw, s.hidden_size)),
                TensorSpec(n["f_bias"], (kw,), init=("uniform", -1.0, 3.0)),
                TensorSpec(n["gate_floor"], (kw,), init=("uniform", 0.0, 0.9)),
                TensorSpec(n["v_proj"], (vw, s.hidden_size)), TensorSpec(n["out_norm"], (s.value_dim,)),
                TensorSpec(n["o_proj"], (s.hidden_size, vw))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        mats = [tensors[n[r]] for r in ("q_proj", "f_proj", "v_proj")]
        self.stacked = torch.cat([m.to(mats[0].dtype) for m in mats], dim=0).contiguous()
        self.gate_bias = tensors[n["f_bias"]].float().contiguous()
        self.gate_floor = tensors[n["gate_floor"]].float().contiguous()
        self.norm_weight = tensors[n["out_norm"]].float().contiguous()
        self.o_proj = tensors[n["o_proj"]].contiguous()

    accepts_scaled_rows = True       # x goes to the stacked product and nowhere else

    def cache_need(self):
        s = self.spec
        return FixedStateNeed((("state", (s.num_heads, s.head_dim, s.value_dim), torch.float32),))

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache):
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        kw, vw = s.num_heads * s.head_dim, s.num_heads * s.value_dim
        proj = ctx.workspace.get("recurrence.proj", (T, 2 * kw + vw), rt.dtype)
        k.linear(x, self.stacked, proj)
        qfv = ctx.workspace.get("recurrence.qfv", (T, 2 * kw + vw), torch.float32)
        k.recurrence_gates(proj, self.gate_bias, self.gate_floor, qfv, kw)
        o = ctx.workspace.get("recurrence.o", (T, vw), torch.float32)
        k.gated_recurrence(qfv, cache.arrays["state"], o, ctx.q_start, ctx.state_slots, s.num_heads, s.head_dim,
                           s.value_dim, ctx.max_q_len)
        normed = ctx.workspace.get("recurrence.normed", (T, vw), rt.dtype)
        k.rmsnorm(o.view(-1, s.value_dim), self.norm_weight, s.norm_eps, 0.0, normed.view(-1, s.value_dim))
        return k.linear(normed, self.o_proj, residual, residual=residual, defer=True)


register_mixer("gated_recurrence", GatedRecurrence, replace=True)
