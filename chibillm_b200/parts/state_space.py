"""A selective state-space mixer with a scalar decay per head (StateSpaceSpec).

One product gives z | x | B | C | dt.  x | B | C pass a causal convolution per channel
with a bias and silu; its last taps - 1 inputs are kept per request in the activations'
type, as they were read.  The scan kernel then runs, per head,

    step = softplus(dt + dt_bias)
    S <- exp(-exp(A_log) * step) S + step * B x^T,    y = S^T C + D x

over the step's tokens of every sequence, from the state that the request's slot holds
to the state it leaves there (32-bit, [heads, value column, state row]); step sizes,
decays and the state never leave 32-bit.  y * silu(z) is normalised in equal parts with
a weight, and the output product adds into the residual.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FixedStateNeed, Mixer, Runtime, TensorSpec, register_mixer


class StateSpace(Mixer):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.num_heads % spec.groups != 0:
            raise ValueError("state_space: num_heads must be a multiple of groups")
        if (spec.num_heads * spec.value_dim) % spec.norm_groups != 0:
            raise ValueError("state_space: the inner width must divide into norm_groups equal parts")
        if spec.conv_taps < 1:
            raise ValueError("state_space: the convolution needs at least one tap")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.inner = spec.num_heads * spec.value_dim
        self.channels = self.inner + 2 * spec.groups * spec.state_size
        self.in_proj: torch.Tensor = None
        self.conv: torch.Tensor = None
        self.conv_t: torch.Tensor = None
        self.conv_bias: torch.Tensor = None
        self.dt_bias: torch.Tensor = None
        self.a_log: torch.Tensor = None
        self.skip: torch.Tensor = None
        self.norm_weight: torch.Tensor = None
        self.o_proj: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s, n = self.spec, self.names
        H = s.num_heads
        return [TensorSpec(n["in_proj"], (2 * self.inner + 2 * s.groups * s.state_size + H, s.hidden_size)),
                TensorSpec(n["conv"], (self.channels, s.conv_taps), init=("normal", 0.0, 0.3)),
                TensorSpec(n["conv_bias"], (self.channels,), init=("normal", 0.0, 0.1)),
                TensorSpec(n["dt_bias"], (H,), init=("uniform", -3.0, 0.0)),
                TensorSpec(n["a_log"], (H,), init=("uniform", -1.0, 1.5)),
                TensorSpec(n["skip"], (H,)),
                TensorSpec(n["out_norm"], (self.inner,)),
                TensorSpec(n["o_proj"], (s.hidden_size, self.inner))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.in_proj = tensors[n["in_proj"]].contiguous()
        self.conv = tensors[n["conv"]].float().contiguous()
        self.conv_t = self.conv.t().contiguous()
        self.conv_bias = tensors[n["conv_bias"]].float().contiguous()
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.a_log = tensors[n["a_log"]].float().contiguous()
        self.skip = tensors[n["skip"]].float().contiguous()
        self.norm_weight = tensors[n["out_norm"]].float().contiguous()
        self.o_proj = tensors[n["o_proj"]].contiguous()

    def cache_need(self):
        s = self.spec
        return FixedStateNeed((("state", (s.num_heads, s.value_dim, s.state_size), torch.float32),
                               ("history", (max(s.conv_taps - 1, 1), self.channels), None)))

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, cache):
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        inner, C, H = self.inner, self.channels, s.num_heads
        proj = ctx.workspace.get("state_space.proj", (T, inner + C + H), rt.dtype)
        k.linear(x, self.in_proj, proj)
        xbc = ctx.workspace.get("state_space.xbc", (T, C), rt.dtype)
        k.causal_conv(proj[:, inner:inner + C], self.conv, self.conv_bias, cache.arrays["history"], xbc,
                      ctx.q_start, ctx.state_slots, ctx.max_q_len, activation="silu", weight_t=self.conv_t)
        y = ctx.workspace.get("state_space.y", (T, inner), torch.float32)
        k.state_space_scan(xbc, proj[:, inner + C:], self.dt_bias, self.a_log, self.skip, cache.arrays["state"], y,
                           ctx.q_start, ctx.state_slots, H, s.groups, s.value_dim, s.state_size)
        normed = ctx.workspace.get("state_space.normed", (T, inner), rt.dtype)
        k.gated_group_rms(y, proj[:, :inner], self.norm_weight, s.norm_eps, s.norm_groups, normed)
        return k.linear(normed, self.o_proj, residual, residual=residual, defer=True)


register_mixer("state_space", StateSpace, replace=True)
