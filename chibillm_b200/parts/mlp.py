"""Dense gated feed-forward (SwiGLU): residual += down(silu(gate(x)) * up(x))
(src/tensor/functions.cc:220-253).  gate and up are stacked into one matrix so
one product yields both (src/qwen/qwen_weights.cc:13-16).  With another gate
activation (the tanh form of gelu) or with biases on the three products the
gate | up product is followed by one kernel that adds the biases, activates
and multiplies.

"table_experts": small gated feed-forwards without biases, chosen per token
from a table by the token's id; the output is the mean of the chosen experts'.
All experts' matrices are stacked, the (token, choice) pairs are sorted by
expert on the device, and two products over tiles of one expert's rows do the
work; nothing is read on the host, so a decode step can be captured.

"routed_experts": small feed-forwards without a gate, down(act(up(x))), chosen per
token by a router: the ``top`` largest of z = W_router x (32-bit), weighted by the
softmax over the chosen logits.  One kernel picks and weighs, the pairs are sorted
by expert on the device by the kernel that sorts a table's choices, and the same
two products over tiles of one expert's rows do the work.  Options: gated experts;
scores from a softmax over all router outputs, chosen by score plus a correction
within the best groups of outputs and weighted by the plain score times a constant;
experts without tensors that return their input (their pairs are sorted into a bucket
of their own whose rows are copies of the tokens' inputs, so the same combination
weighs them); one more gated expert that every token uses."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import FeedForward, Runtime, TensorSpec, register_feed_forward


class GatedMLP(FeedForward):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.activation not in ("silu", "gelu_tanh", "swish_clamped"):
            raise ValueError(f"activation '{spec.activation}' is not supported by gated_mlp")
        if spec.activation == "swish_clamped" and (spec.biases or not spec.limit > 0):
            raise ValueError("gated_mlp: the clamped gate has a positive limit and no biases")
        self.spec = spec
        self.plain_swiglu = spec.activation == "silu" and not spec.biases
        self.bias_gate_up: torch.Tensor = None
        self.bias_down: torch.Tensor = None
        self.names = names
        self.runtime = runtime
        self.gate_up: torch.Tensor = None
        self.gate_up_interleaved: torch.Tensor = None
        self.down: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(self.names["gate_proj"], (s.intermediate_size, s.hidden_size)),
               TensorSpec(self.names["up_proj"], (s.intermediate_size, s.hidden_size)),
               TensorSpec(self.names["down_proj"], (s.hidden_size, s.intermediate_size))]
        if s.biases:
            out += [TensorSpec(self.names["gate_bias"], (s.intermediate_size,), init=("normal", 0.0, 0.1)),
                    TensorSpec(self.names["up_bias"], (s.intermediate_size,), init=("normal", 0.0, 0.1)),
                    TensorSpec(self.names["down_bias"], (s.hidden_size,), init=("normal", 0.0, 0.1))]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors[self.names["gate_proj"]], tensors[self.names["up_proj"]]
        if gate.dtype != up.dtype:
            up = up.to(gate.dtype)
        if self.spec.biases:
            self.bias_gate_up = torch.cat([tensors[self.names["gate_bias"]].to(gate.dtype),
                                           tensors[self.names["up_bias"]].to(gate.dtype)]).contiguous()
            self.bias_down = tensors[self.names["down_bias"]].float().contiguous()
        interleave = getattr(self.runtime.kernels, "interleave_gate_up", None) if self.plain_swiglu else None
        self.gate_up_interleaved = interleave(gate, up) if interleave is not None else None
        # one of the two layouts is kept: blocks of 64 gate rows and their 64 up rows for the kernel
        # that applies SwiGLU itself, else gate rows followed by up rows
        self.gate_up = None if self.gate_up_interleaved is not None else torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.names["down_proj"]].contiguous()

    accepts_scaled_rows = True       # x goes to the gate | up product and nowhere else

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        k = self.runtime.kernels
        T = x.shape[0]
        inter = self.spec.intermediate_size
        act = ctx.workspace.get("mlp.act", (T, inter), self.runtime.dtype)
        if not self.plain_swiglu:
            gate_up = ctx.workspace.get("mlp.gate_up", (T, 2 * inter), self.runtime.dtype)
            k.linear(x, self.gate_up, gate_up)
            if self.spec.activation == "swish_clamped":
                k.clamped_swish_gate(gate_up, act, self.spec.limit, self.spec.gate_slope)
            else:
                k.gated_activation(gate_up, self.bias_gate_up, act, self.spec.activation)
            if self.bias_down is not None:
                k.add_row_vector(residual, self.bias_down)
            return k.linear(act, self.down, residual, residual=residual, defer=True)
        if self.gate_up_interleaved is not None:
            if not k.linear_swiglu(x, self.gate_up_interleaved, act):
                raise RuntimeError("gated_mlp: the fused kernel refused a shape it was prepared for")
            return k.linear(act, self.down, residual, residual=residual, defer=True)
        split = getattr(k, "linear_partial", None)
        pending = split(x, self.gate_up) if split is not None else None
        if pending is not None:
            k.reduce_swiglu(pending, act)            # adds the partial sums and applies SwiGLU
        else:
            gate_up = ctx.workspace.get("mlp.gate_up", (T, 2 * inter), self.runtime.dtype)
            k.linear(x, self.gate_up, gate_up)
            k.swiglu(gate_up, act)
        return k.linear(act, self.down, residual, residual=residual, defer=True)


class DenseMLP(FeedForward):
    """Dense feed-forward without a gate: residual += down(act(up(x))).  The
    activation is applied to the 32-bit sums of the first product (by the kernel
    that adds up a split product, or in place on the product's output)."""

    ACTIVATIONS = ("gelu", "gelu_tanh", "silu", "relu")

    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.activation not in self.ACTIVATIONS:
            raise ValueError(f"activation '{spec.activation}' is not supported by mlp; known: {self.ACTIVATIONS}")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.up: torch.Tensor = None
        self.down: torch.Tensor = None

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        return [TensorSpec(self.names["up_proj"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(self.names["down_proj"], (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up = tensors[self.names["up_proj"]].contiguous()
        self.down = tensors[self.names["down_proj"]].contiguous()

    accepts_scaled_rows = True       # x goes to the up product and nowhere else

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        k = self.runtime.kernels
        T = x.shape[0]
        act = ctx.workspace.get("mlp.act", (T, self.spec.intermediate_size), self.runtime.dtype)
        fused = getattr(k, "linear_activation", None)
        if fused is None or not fused(x, self.up, act, self.spec.activation):
            k.linear(x, self.up, act)
            k.activation(act, self.spec.activation)
        return k.linear(act, self.down, residual, residual=residual, defer=True)


class TableExperts(FeedForward):
    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation '{spec.activation}' is not supported by table_experts")
        if not (0 < spec.top <= spec.num_experts):
            raise ValueError("table_experts: 0 < top <= num_experts is required")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.table: torch.Tensor = None
        # [experts, 2 ff, hidden]: an expert's gate rows, then its up rows -- or, for kernels that
        # want it so, blocks of 16 gate rows each followed by its 16 up rows (``interleaved``)
        self.gate_up: torch.Tensor = None
        self.interleaved = False
        self.down: torch.Tensor = None          # [experts, hidden, ff]

    def _name(self, role: str, e: int) -> str:
        return self.names[role].replace("{e}", str(e))

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(self.names["expert_table"], (s.vocab_size, s.top), kind="int",
                          init=("distinct", 0, s.num_experts))]
        for e in range(s.num_experts):
            out += [TensorSpec(self._name("expert_gate", e), (s.intermediate_size, s.hidden_size)),
                    TensorSpec(self._name("expert_up", e), (s.intermediate_size, s.hidden_size)),
                    TensorSpec(self._name("expert_down", e), (s.hidden_size, s.intermediate_size))]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.table = tensors[self.names["expert_table"]].to(torch.int32).contiguous()
        self.table_host = self.table.to("cpu", torch.int64)
        if self.table.numel() and (int(self.table.min()) < 0 or int(self.table.max()) >= s.num_experts):
            raise ValueError(f"{self.names['expert_table']}: an entry names an expert outside 0..{s.num_experts - 1}")
        first = tensors[self._name("expert_gate", 0)]
        self.gate_up = torch.empty((s.num_experts, 2 * s.intermediate_size, s.hidden_size), dtype=first.dtype,
                                   device=first.device)
        self.down = torch.empty((s.num_experts, s.hidden_size, s.intermediate_size), dtype=first.dtype,
                                device=first.device)
        fast = getattr(self.runtime.kernels, "expert_tensor_cores", None)
        self.interleaved = fast is not None and fast(first.dtype, s.hidden_size, s.intermediate_size)
        for e in range(s.num_experts):
            gate, up = tensors[self._name("expert_gate", e)], tensors[self._name("expert_up", e)]
            if self.interleaved:
                self.gate_up[e] = self.runtime.kernels.interleave_expert_gate_up(gate, up)
            else:
                self.gate_up[e, :s.intermediate_size] = gate
                self.gate_up[e, s.intermediate_size:] = up
            self.down[e] = tensors[self._name("expert_down", e)]

    def launch_key(self, ctx):
        return ()

    # Experts whose sizes the tcgen05 kernel of the routed rows does not take (no multiples of 64): a prompt
    # step whose token ids the host knows, of so many (token, choice) pairs and of so many multiplications
    # per expert on average, is sorted by expert on the host, and every expert's rows go through the kernels'
    # ordinary matrix products (2 E launches instead of 2: smaller experts lose more to the launches than the
    # faster product gains; measured against the mma.sync kernel at 8 experts and 4,096 pairs: width 1,024,
    # ff 1,536: 2.1 -> 3.6 ms a prompt step; width 2,048, ff 3,072: 4.5 -> 3.7; width 4,096, ff 6,144:
    # 13.0 -> 6.8; the tcgen05 kernel takes 1.6, 2.7 and 6.6 and is used wherever it can be)
    MANY_PAIRS = 512
    MUCH_WORK = 1 << 31

    def _forward_expert_by_expert(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T, top, E, F, D = x.shape[0], s.top, s.num_experts, s.intermediate_size, s.hidden_size
        pairs = T * top
        chosen = self.table_host[ctx.tokens_host.long()].reshape(-1)            # expert of pair t * top + choice
        order = torch.argsort(chosen, stable=True).to(torch.int32)             # pairs, sorted by expert
        counts = torch.bincount(chosen, minlength=E).tolist()
        plan = torch.empty(E + 1 + 3 * pairs, dtype=torch.int32)
        plan[0] = 0
        plan[1:E + 1] = torch.cumsum(torch.tensor(counts), 0).to(torch.int32)
        plan[E + 1:E + 1 + pairs] = order
        plan[E + 1 + pairs + order.long()] = torch.arange(pairs, dtype=torch.int32)   # row of every pair
        plan[E + 1 + 2 * pairs:] = order // top                                 # token of every sorted row
        route = ctx.workspace.get("experts.plan", (E + 1 + 3 * pairs,), torch.int32)
        route.copy_(plan)
        rows = route[E + 1 + 2 * pairs:]
        xs = ctx.workspace.get("experts.sorted", (pairs, D), rt.dtype)
        k.gather_rows(x, rows, xs)
        gate_up = ctx.workspace.get("experts.gate_up", (pairs, 2 * F), rt.dtype)
        act = ctx.workspace.get("experts.act", (pairs, F), rt.dtype)
        y = ctx.workspace.get("experts.out", (pairs, D), torch.float32)
        at = 0
        for e, n in enumerate(counts):
            if n:
                k.linear(xs[at:at + n], self.gate_up[e], gate_up[at:at + n])
            at += n
        k.gated_activation(gate_up, None, act, s.activation, **({"interleaved": True} if self.interleaved else {}))
        at = 0
        for e, n in enumerate(counts):
            if n:
                k.linear(act[at:at + n], self.down[e], y[at:at + n])
            at += n
        k.combine_experts(y, route, residual, top, E, 1.0 / top)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        s, k = self.spec, self.runtime.kernels
        T = x.shape[0]
        pairs = T * s.top
        if pairs >= self.MANY_PAIRS and ctx.max_q_len > 1 and getattr(ctx, "tokens_host", None) is not None \
                and pairs * s.intermediate_size * s.hidden_size >= self.MUCH_WORK * s.num_experts \
                and getattr(k, "combine_experts", None) is not None \
                and not (hasattr(k, "experts_on_tcgen05")
                         and k.experts_on_tcgen05(self.runtime.dtype, s.hidden_size, s.intermediate_size)):
            return self._forward_expert_by_expert(x, residual, ctx)
        route = ctx.workspace.get("experts.route", (k.route_words(pairs, s.num_experts),), torch.int32)
        act = ctx.workspace.get("experts.act", (pairs, s.intermediate_size), self.runtime.dtype)
        y = ctx.workspace.get("experts.out", (pairs, s.hidden_size), torch.float32)
        extra = {}
        if self.interleaved:
            extra = {"interleaved": True,
                     "sorted_x": ctx.workspace.get("experts.sorted", (pairs, s.hidden_size), self.runtime.dtype)}
        k.routed_experts(x, ctx.tokens, self.table, self.gate_up, self.down, residual, route, act, y,
                         s.activation, 1.0 / s.top, **extra)
        return None


class RoutedExperts(FeedForward):
    ACTIVATIONS = ("relu2", "relu", "silu", "gelu", "gelu_tanh")

    def __init__(self, spec, names: Dict[str, str], runtime: Runtime):
        if spec.activation not in self.ACTIVATIONS:
            raise ValueError(f"activation '{spec.activation}' is not supported by routed_experts")
        self.outputs = spec.num_experts + spec.identity_experts
        if not (0 < spec.top <= self.outputs):
            raise ValueError("routed_experts: 0 < top <= num_experts (+ identity_experts) is required")
        if spec.scores not in ("softmax_top", "softmax_all"):
            raise ValueError(f"routed_experts: scores '{spec.scores}' is not supported")
        if spec.scores == "softmax_top" and (spec.correction or spec.group_count != 1 or spec.identity_experts
                                             or spec.weight_scale != 1.0):
            raise ValueError("routed_experts: corrections, groups, identity experts and a weight scale belong "
                             "to scores 'softmax_all'")
        if self.outputs % spec.group_count != 0 or not (0 < spec.group_keep <= spec.group_count) \
                or spec.top > (self.outputs // spec.group_count) * spec.group_keep:
            raise ValueError("routed_experts: the router's outputs must form equal groups whose kept ones hold "
                             "at least top outputs")
        self.spec = spec
        self.names = names
        self.runtime = runtime
        self.router: torch.Tensor = None        # [outputs, hidden]
        self.correction: torch.Tensor = None    # [outputs], 32-bit
        self.up: torch.Tensor = None            # [experts, ff, hidden]; gated: [experts, 2 ff, hidden]
        self.down: torch.Tensor = None          # [experts, hidden, ff]
        self.interleaved = False
        self.shared = None
        if spec.shared_size:
            from ..config.spec import GatedMLPSpec
            self.shared = GatedMLP(GatedMLPSpec(kind="gated_mlp", hidden_size=spec.hidden_size,
                                                intermediate_size=spec.shared_size, activation=spec.activation),
                                   {"gate_proj": names["shared_gate"], "up_proj": names["shared_up"],
                                    "down_proj": names["shared_down"]}, runtime)

    def _name(self, role: str, e: int) -> str:
        return self.names[role].replace("{e}", str(e))

    def expected_tensors(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(self.names["router"], (self.outputs, s.hidden_size), init=("normal", 0.0, 0.5))]
        if s.correction:
            out.append(TensorSpec(self.names["correction"], (self.outputs,), init=("normal", 0.0, 0.02)))
        for e in range(s.num_experts):
            if s.gated:
                out.append(TensorSpec(self._name("expert_gate", e), (s.intermediate_size, s.hidden_size)))
            out += [TensorSpec(self._name("expert_up", e), (s.intermediate_size, s.hidden_size)),
                    TensorSpec(self._name("expert_down", e), (s.hidden_size, s.intermediate_size))]
        if self.shared is not None:
            out += self.shared.expected_tensors()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.router = tensors[self.names["router"]].contiguous()
        if s.correction:
            self.correction = tensors[self.names["correction"]].float().contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)
        first = tensors[self._name("expert_up", 0)]
        # experts that return their input: one more bucket of the route, behind the experts with tensors; the
        # stacked matrices get a stand-in of zeros there, so that every expert number of the route is in bounds
        E = s.num_experts + (1 if s.identity_experts else 0)
        F, D = s.intermediate_size, s.hidden_size
        fast = getattr(self.runtime.kernels, "expert_tensor_cores", None)
        self.interleaved = bool(s.gated and fast is not None and fast(first.dtype, D, F))
        self.up = torch.zeros((E, (2 if s.gated else 1) * F, D), dtype=first.dtype, device=first.device)
        self.down = torch.zeros((E, D, F), dtype=first.dtype, device=first.device)
        for e in range(s.num_experts):
            up = tensors[self._name("expert_up", e)]
            if not s.gated:
                self.up[e] = up
            elif self.interleaved:
                self.up[e] = self.runtime.kernels.interleave_expert_gate_up(tensors[self._name("expert_gate", e)], up)
            else:
                self.up[e, :F] = tensors[self._name("expert_gate", e)]
                self.up[e, F:] = up
            self.down[e] = tensors[self._name("expert_down", e)]

    def launch_key(self, ctx):
        return ()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        s, rt = self.spec, self.runtime
        k = rt.kernels
        T = x.shape[0]
        pairs = T * s.top
        logits = ctx.workspace.get("router.logits", (T, self.outputs), torch.float32)
        k.linear(x, self.router, logits)
        chosen = ctx.workspace.get("router.chosen", (T, s.top), torch.int32)
        share = ctx.workspace.get("router.share", (T, s.top), torch.float32)
        buckets = self.up.shape[0]
        extra = {}
        if s.scores == "softmax_all":
            k.router_choose(logits, self.correction, chosen, share, s.group_count, s.group_keep, s.weight_scale,
                            last_choice=buckets - 1)
            extra = {"gated": s.gated, "interleaved": self.interleaved, "identity": s.identity_experts}
        else:
            k.router_top(logits, chosen, share)
            if s.gated:
                extra = {"gated": True, "interleaved": self.interleaved}
        route = ctx.workspace.get("experts.route", (k.route_words(pairs, buckets),), torch.int32)
        act = ctx.workspace.get("experts.act", (pairs, s.intermediate_size), rt.dtype)
        y = ctx.workspace.get("experts.out", (pairs, s.hidden_size), torch.float32)
        sorted_x = ctx.workspace.get("experts.sorted", (pairs, s.hidden_size), rt.dtype)
        k.chosen_experts(x, chosen, share, self.up, self.down, residual, route, act, y, s.activation, sorted_x,
                         **extra)
        if self.shared is not None:
            return self.shared.forward(x, residual, ctx)
        return None


register_feed_forward("gated_mlp", GatedMLP, replace=True)
register_feed_forward("routed_experts", RoutedExperts, replace=True)
register_feed_forward("table_experts", TableExperts, replace=True)
register_feed_forward("mlp", DenseMLP, replace=True)
