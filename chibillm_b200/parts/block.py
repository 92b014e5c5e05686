"""Block arrangements.  "prenorm": residual += mixer(norm(residual)), then
residual += feed_forward(norm(residual)); the residual itself is never
normalised in place (src/qwen/qwen_layer.cc:124-146).  Two options of the
layer's spec: a short convolution over time between the first norm and the
mixer (it keeps its last inputs per request, so the block then has two cache
needs), and no feed-forward at all.  With ``layer_scale`` each sublayer's result is
multiplied feature by feature by a learned vector before it joins the residual: the
sublayer then adds into a 32-bit array of its own, and one kernel adds vector * array
to the residual and writes the next norm's output (the block leaves that kernel
pending, as it leaves a product pending otherwise).

"parallel": one norm whose output both branches read,
residual += scale * (mixer(norm(residual)) + feed_forward(norm(residual))), then an
optional per-layer token input (parts/token_input.py).  The branches add into a
32-bit array of their own; one kernel at the layer's end adds it to the residual
with the scale, applies the token input and, when the next block's norm asks for
it, writes that norm's output too (the block leaves that kernel pending, as a
product is left pending by the other arrangement).

"postnorm": the sublayers read the residual itself and the norms sit on their
outputs, residual += norm(mixer(residual)), then residual += norm(ff(residual)),
then the optional token input.  With ``token_shift`` the mixer reads every token
moved towards the one before it, h + (h' - h) * w; the last token's h is kept per
request (a second cache need of the block, 32-bit), so a portion of a prompt goes
on where the one before stopped."""
from __future__ import annotations

from typing import Dict, List

import torch

from .base import (Block, FixedStateNeed, Runtime, TensorSpec, make_feed_forward, make_mixer, make_norm,
                   register_block)
from .short_conv import ShortConv
from .token_input import TokenInput


class ScaledSum:
    """What a sublayer with a scale per feature leaves pending: its sum, still to be multiplied
    by the vector and added to the residual; the norm that follows can be done on the way."""

    def __init__(self, kernels, delta: torch.Tensor, vec: torch.Tensor):
        self.kernels, self.delta, self.vec = kernels, delta, vec

    def add_into(self, residual: torch.Tensor) -> None:
        self.kernels.scaled_add_norm(residual, self.delta, self.vec)

    def finish_with_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                         out: torch.Tensor, scaled_ok: bool):
        self.kernels.scaled_add_norm(residual, self.delta, self.vec, norm=(weight, eps, offset, out))
        return out


class PreNormBlock(Block):
    def __init__(self, layer, runtime: Runtime):
        self.layer = layer
        self.runtime = runtime
        names = {role: layer.weight_prefix + name for role, name in layer.names().items()}
        self.mixer_norm = make_norm(layer.mixer_norm, names["mixer_norm"], runtime)
        self.mixer = make_mixer(layer.mixer, names, runtime)
        self.mixer_conv = None if layer.mixer_conv is None else ShortConv(layer.mixer_conv, names["mixer_conv"], runtime)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = make_norm(layer.feed_forward_norm, names["feed_forward_norm"], runtime)
            self.feed_forward = make_feed_forward(layer.feed_forward, names, runtime)
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer_conv, self.mixer, self.feed_forward_norm,
                                        self.feed_forward) if p is not None)
        self.scale_names = None
        self.mixer_scale: torch.Tensor = None
        self.feed_forward_scale: torch.Tensor = None
        if getattr(layer, "layer_scale", False):
            self.scale_names = (names["mixer_scale"],
                                names["feed_forward_scale"] if self.feed_forward is not None else None)

    def expected_tensors(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for p in self._parts:
            out.extend(p.expected_tensors())
        if self.scale_names is not None:
            out += [TensorSpec(n, (self.layer.mixer_norm.size,)) for n in self.scale_names if n is not None]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.bind(tensors)
        if self.scale_names is not None:
            self.mixer_scale = tensors[self.scale_names[0]].float().contiguous()
            if self.scale_names[1] is not None:
                self.feed_forward_scale = tensors[self.scale_names[1]].float().contiguous()

    def _scaled(self, run, vec: torch.Tensor, residual: torch.Tensor, ctx, tag: str) -> ScaledSum:
        """Runs a sublayer into a 32-bit array of its own; what joins the residual is vec * that."""
        k = self.runtime.kernels
        delta = ctx.workspace.get("block.delta." + tag, tuple(residual.shape), torch.float32)
        k.zero(delta)
        left = run(delta)
        if left is not None:
            left.add_into(delta)
        return ScaledSum(k, delta, vec)

    def cache_need(self):
        if self.mixer_conv is None:
            return self.mixer.cache_need()
        return (self.mixer.cache_need(), self.mixer_conv.cache_need())

    def launch_key(self, ctx):
        keys = [p.launch_key(ctx) for p in (self.mixer_conv, self.mixer, self.feed_forward) if p is not None]
        return None if any(k is None for k in keys) else tuple(keys)

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        x = ctx.workspace.get("block.normed", tuple(residual.shape), self.runtime.dtype)
        conv = self.mixer_conv
        normed = self.mixer_norm.forward_fused(residual, pending, x,
                                               conv is None and self.mixer.accepts_scaled_rows)
        normed = x if normed is None else normed
        if conv is not None:
            cache, conv_state = cache
            mixed = ctx.workspace.get("block.conv", tuple(residual.shape), self.runtime.dtype)
            conv.forward(normed, mixed, ctx, conv_state)
            normed = mixed
        if self.scale_names is not None:
            pending = self._scaled(lambda acc: self.mixer.forward(normed, acc, ctx, cache), self.mixer_scale,
                                   residual, ctx, "mixer")
        else:
            pending = self.mixer.forward(normed, residual, ctx, cache)
        if self.feed_forward is None:
            return pending
        normed = self.feed_forward_norm.forward_fused(residual, pending, x, self.feed_forward.accepts_scaled_rows)
        normed = x if normed is None else normed
        if self.scale_names is not None:
            return self._scaled(lambda acc: self.feed_forward.forward(normed, acc, ctx), self.feed_forward_scale,
                                residual, ctx, "ff")
        return self.feed_forward.forward(normed, residual, ctx)


class LayerEnd:
    """What a parallel block leaves pending: the branches' sum, still to be added
    to the residual with the block's scale, and the token input after it."""

    def __init__(self, block: "ParallelBlock", delta: torch.Tensor, ctx):
        self.block, self.delta, self.ctx = block, delta, ctx

    def _run(self, residual: torch.Tensor, norm) -> None:
        b = self.block
        k = b.runtime.kernels
        scale = b.layer.residual_scale
        ti = b.token_input
        if ti is None:
            k.layer_end(residual, self.delta, scale, norm=norm)
            return
        side = ti.kernel_arguments(self.ctx)
        if ti.wants_products(residual.shape[0]):
            # the token input reads the residual after the block's update, so that comes first
            x = self.ctx.workspace.get("token_input.x", tuple(residual.shape), b.runtime.dtype)
            k.layer_end(residual, self.delta, scale, copy_out=x)
            y = ti.products(x, self.ctx)
            k.layer_end(residual, None, scale, side=side, y_in=y, norm=norm)
        else:
            k.layer_end(residual, self.delta, scale, side=side, norm=norm)

    def add_into(self, residual: torch.Tensor) -> None:
        self._run(residual, None)

    def finish_with_norm(self, residual: torch.Tensor, weight: torch.Tensor, eps: float, offset: float,
                         out: torch.Tensor, scaled_ok: bool):
        ti = self.block.token_input
        if ti is not None and (weight.dtype != ti.norm.dtype or float(eps) != float(ti.spec.eps)):
            self._run(residual, None)
            self.block.runtime.kernels.rmsnorm(residual, weight, eps, offset, out)
            return out
        self._run(residual, (weight, eps, offset, out))
        return out


class ParallelBlock(Block):
    def __init__(self, layer, runtime: Runtime):
        if layer.mixer_conv is not None or layer.feed_forward_norm is not None:
            raise ValueError("the parallel arrangement has one norm and no convolution")
        self.layer = layer
        self.runtime = runtime
        names = {role: layer.weight_prefix + name for role, name in layer.names().items()}
        self.mixer_norm = make_norm(layer.mixer_norm, names["mixer_norm"], runtime)
        self.mixer = make_mixer(layer.mixer, names, runtime)
        self.feed_forward = None if layer.feed_forward is None else make_feed_forward(layer.feed_forward, names, runtime)
        self.token_input = None if layer.token_input is None else TokenInput(layer.token_input, names, runtime)
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward, self.token_input)
                            if p is not None)

    def expected_tensors(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for p in self._parts:
            out.extend(p.expected_tensors())
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.bind(tensors)

    def launch_key(self, ctx):
        keys = [p.launch_key(ctx) for p in (self.mixer, self.feed_forward, self.token_input) if p is not None]
        return None if any(k is None for k in keys) else tuple(keys)

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        rt = self.runtime
        k = rt.kernels
        x = ctx.workspace.get("block.normed", tuple(residual.shape), rt.dtype)
        normed = self.mixer_norm.forward_fused(residual, pending, x, False)
        normed = x if normed is None else normed
        delta = ctx.workspace.get("block.delta", tuple(residual.shape), torch.float32)
        k.zero(delta)
        left = self.mixer.forward(normed, delta, ctx, cache)
        if left is not None:
            left.add_into(delta)          # before the feed-forward starts split products of its own
        if self.feed_forward is not None:
            left = self.feed_forward.forward(normed, delta, ctx)
            if left is not None:
                left.add_into(delta)
        return LayerEnd(self, delta, ctx)


class PostNormBlock(Block):
    def __init__(self, layer, runtime: Runtime):
        if layer.mixer_conv is not None:
            raise ValueError("the postnorm arrangement has no convolution")
        self.layer = layer
        self.runtime = runtime
        names = {role: layer.weight_prefix + name for role, name in layer.names().items()}
        self.hidden = layer.mixer_norm.size
        self.mixer_norm = make_norm(layer.mixer_norm, names["mixer_norm"], runtime)
        self.mixer = make_mixer(layer.mixer, names, runtime)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = make_norm(layer.feed_forward_norm, names["feed_forward_norm"], runtime)
            self.feed_forward = make_feed_forward(layer.feed_forward, names, runtime)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "add_to"):
                raise ValueError(f"norm kind '{norm.spec.kind}' cannot add its output to the residual")
        self.token_input = None if layer.token_input is None else TokenInput(layer.token_input, names, runtime)
        self.shift_name = names["token_shift"] if layer.token_shift else None
        self.shift: torch.Tensor = None
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward,
                                        self.token_input) if p is not None)

    def expected_tensors(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for p in self._parts:
            out.extend(p.expected_tensors())
        if self.shift_name is not None:
            out.append(TensorSpec(self.shift_name, (self.hidden,), init=("uniform", 0.0, 1.0)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.bind(tensors)
        if self.shift_name is not None:
            self.shift = tensors[self.shift_name].float().contiguous()

    def cache_need(self):
        if self.shift_name is None:
            return self.mixer.cache_need()
        return (self.mixer.cache_need(), FixedStateNeed((("last_input", (self.hidden,), torch.float32),)))

    def launch_key(self, ctx):
        keys = [p.launch_key(ctx) for p in (self.mixer, self.feed_forward, self.token_input) if p is not None]
        return None if any(k is None for k in keys) else tuple(keys)

    def forward(self, residual: torch.Tensor, ctx, cache, pending=None):
        rt = self.runtime
        k = rt.kernels
        if pending is not None:
            pending.add_into(residual)
        shape = tuple(residual.shape)
        h = ctx.workspace.get("block.normed", shape, rt.dtype)
        if self.shift_name is not None:
            cache, kept = cache
            k.token_shift(residual, self.shift, kept.arrays["last_input"], ctx.q_start, ctx.seq_of_token,
                          ctx.state_slots, h)
        else:
            k.cast(residual, h)
        delta = ctx.workspace.get("block.delta", shape, torch.float32)
        k.zero(delta)
        left = self.mixer.forward(h, delta, ctx, cache)
        if left is not None:
            left.add_into(delta)
        ti = self.token_input
        products = ti is not None and ti.wants_products(shape[0])
        # the residual in the activations' type, for whoever reads it next
        x = ctx.workspace.get("block.x", shape, rt.dtype)
        ff = self.feed_forward
        self.mixer_norm.add_to(delta, residual, copy_out=x if (ff is not None or products) else None)
        if ff is not None:
            k.zero(delta)
            left = ff.forward(x, delta, ctx)
            if left is not None:
                left.add_into(delta)
            self.feed_forward_norm.add_to(delta, residual, copy_out=x if products else None)
        if ti is not None:
            side = ti.kernel_arguments(ctx)
            if products:
                k.layer_end(residual, None, 1.0, side=side, y_in=ti.products(x, ctx))
            else:
                k.layer_end(residual, None, 1.0, side=side)
        return None


register_block("prenorm", PreNormBlock, replace=True)
register_block("postnorm", PostNormBlock, replace=True)
register_block("parallel", ParallelBlock, replace=True)
