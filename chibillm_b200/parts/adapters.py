"""Adapters: parts outside the blocks.

"scale": multiplies its argument by a constant (``params``: "factor"); as an
input adapter it scales the embeddings, as a logit adapter the logits.

"softcap": replaces x by cap * tanh(x / cap) (``params``: "cap"); as a logit
adapter it bounds the logits.

"reentry_mix": a stream adapter for a group of layers that runs several times.
Before each pass the residual x is replaced by W [x; x0] + step[turn], where x0
is the residual as the input adapters left it, W is [hidden, 2 * hidden] (x's
columns first) and step holds one vector per pass (tensor roles "mix", "step").
The product takes its inputs in the activations' type; the sum is 32-bit.

"reentry_add": the same place, without a matrix: before every pass but the first the
embedding output x0 is added to x, and before every pass the pass's vector step[turn]
(tensor role "step"; ``params``: "hidden_size", "turns").

"bigram": an input adapter that adds a row of a table chosen by the token and the
token before it, row = (previous * mul_prev + token * mul_cur) mod buckets, and the
table's last row (number ``buckets``) for a sequence's first token (tensor role
"table"; ``params``: "hidden_size", "buckets", "mul_prev", "mul_cur").  The token
before a step's first is part of the request's state: the adapter declares a cache
need of one integer per request.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import Adapter, FixedStateNeed, Runtime, TensorSpec, register_adapter


class Scale(Adapter):
    def __init__(self, spec, runtime: Runtime):
        self.factor = float(spec.constants()["factor"])
        self.runtime = runtime

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, ctx, turn: int = 0) -> None:
        if self.factor != 1.0:
            self.runtime.kernels.scale(x, self.factor)


class SoftCap(Adapter):
    def __init__(self, spec, runtime: Runtime):
        self.cap = float(spec.constants()["cap"])
        if not self.cap > 0:
            raise ValueError("softcap: the cap must be positive")
        self.runtime = runtime

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, ctx, turn: int = 0) -> None:
        self.runtime.kernels.softcap(x, self.cap)


class ReentryMix(Adapter):
    needs_embedding_output = True

    def __init__(self, spec, runtime: Runtime):
        self.names = spec.names()
        c = spec.constants()
        self.hidden, self.turns = int(c["hidden_size"]), int(c["turns"])
        self.runtime = runtime
        self.mix: torch.Tensor = None
        self.step: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.names["mix"], (self.hidden, 2 * self.hidden)),
                TensorSpec(self.names["step"], (self.turns, self.hidden), init=("normal", 0.0, 0.1))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.mix = tensors[self.names["mix"]].contiguous()
        self.step = tensors[self.names["step"]].float().contiguous()

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, ctx, turn: int = 0) -> None:
        rt = self.runtime
        k = rt.kernels
        T, D = x.shape
        both = ctx.workspace.get("reentry.both", (T, 2 * D), rt.dtype)
        if ctx.shared.get("reentry.filled") is not both:
            # x0 is the same in every pass of a step: its half is filled once
            k.cast_rows(ctx.shared["embedding output"], both[:, D:])
            ctx.shared["reentry.filled"] = both
        k.cast_rows(x, both[:, :D])
        k.linear(both, self.mix, x)
        k.add_row_vector(x, self.step[turn])


class ReentryAdd(Adapter):
    needs_embedding_output = True

    def __init__(self, spec, runtime: Runtime):
        self.names = spec.names()
        c = spec.constants()
        self.hidden, self.turns = int(c["hidden_size"]), int(c["turns"])
        self.runtime = runtime
        self.step: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.names["step"], (self.turns, self.hidden), init=("normal", 0.0, 0.1))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.step = tensors[self.names["step"]].float().contiguous()

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, ctx, turn: int = 0) -> None:
        self.runtime.kernels.stream_enter(x, ctx.shared["embedding output"] if turn > 0 else None, self.step[turn])


class Bigram(Adapter):
    def __init__(self, spec, runtime: Runtime):
        self.names = spec.names()
        c = spec.constants()
        self.hidden, self.buckets = int(c["hidden_size"]), int(c["buckets"])
        self.mul_prev, self.mul_cur = int(c["mul_prev"]), int(c["mul_cur"])
        if self.buckets < 1:
            raise ValueError("bigram: the table needs at least one bucket")
        self.runtime = runtime
        self.table: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.names["table"], (self.buckets + 1, self.hidden), init=("normal", 0.0, 0.02))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.names["table"]].contiguous()

    def cache_need(self):
        return FixedStateNeed((("last_token", (1,), torch.int32),))

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, ctx, turn: int = 0, cache=None) -> None:
        self.runtime.kernels.bigram_embed(x, self.table, cache.arrays["last_token"], ctx.tokens, ctx.positions,
                                          ctx.seq_of_token, ctx.q_start, ctx.state_slots, self.mul_prev,
                                          self.mul_cur)


register_adapter("reentry_add", ReentryAdd, replace=True)
register_adapter("bigram", Bigram, replace=True)
register_adapter("scale", Scale, replace=True)
register_adapter("softcap", SoftCap, replace=True)
register_adapter("reentry_mix", ReentryMix, replace=True)
