"""Pitudra: the typed configuration and its translation into parts.

A Pitudra config.json names the architecture under "architecture" and gives
every size and constant in nested objects:

* "vocab", "width"; "norm": {"eps"}; "token_side": {"dim"};
* "layers": one object per layer with "type", "mixer" and "mlp".
  - type "latent_attention": "heads", "dim" (a head's plain query/key size),
    "rot_dim" (its rotated part), "vdim", "q_rank", "kv_rank", "scale",
    "mask": {"size"} (a sliding window), "rot": {"base", "dims"}, and optionally
    "kv_from": j (the layer has no key/value down-projection and reads layer j's
    cached latents with up-projections of its own);
  - type "hgrn2": "heads", "dim", "vdim";
  - type "attention": "heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}.
  "mlp" is null or {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}.

Absent optional objects ("token_side", a mixer's "mask", "vdim", "kv_heads")
switch their mechanism off or fall back to the plain value.

What the design fixes: the norms are layer norms with weight and bias and sit on
the sublayers' outputs (x + norm(mixer(x)), x + norm(ff(x))); every mixer reads
its input shifted towards the token before; attention has a sink per head in the
softmax's denominator; plain attention has biases on q, k and v, a norm over the
whole q and k projections, no rotation and a sigmoid gate on its output; experts
are down(relu(up x)^2) chosen by a router, weighted by the softmax over the chosen
logits; the token input is gated with the tanh form of gelu.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, KeyReader, object_at as _object
from .spec import (AttentionSpec, GatedRecurrenceSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                   PositionSpec, RoutedExpertsSpec, RunStep, TokenInputSpec)

ARCHITECTURE = "Pitudra"
SIDE_TABLE = "side.embed"
MIXERS = ("latent_attention", "hgrn2", "attention")


@dataclass(frozen=True)
class PitudraLayer:
    kind: str                      # one of MIXERS
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0              # attention
    scale: float = 0.0             # both kinds of attention
    window: Optional[int] = None
    rot_dim: int = 0               # latent attention from here on
    q_rank: int = 0
    kv_rank: int = 0
    rot_base: float = 0.0
    kv_from: Optional[int] = None
    ff: int = 0                    # 0: no feed-forward
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class PitudraConfig:
    vocab: int
    width: int
    eps: float
    side_dim: Optional[int]
    layers: Tuple[PitudraLayer, ...]

    @classmethod
    def from_dict(cls, obj: dict) -> "PitudraConfig":
        r = KeyReader(obj)
        vocab, width = r.positive_int("vocab"), r.positive_int("width")
        eps = KeyReader(_object(r, "norm")).positive_float("eps")
        side_dim = KeyReader(_object(r, "token_side")).positive_int("dim") if r.has("token_side") else None
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("invalid_field", "key 'layers' must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw)
            kind = lr.require_value("type", MIXERS)
            m = KeyReader(_object(lr, "mixer"))
            heads, dim = m.positive_int("heads"), m.positive_int("dim")
            vdim = m.positive_int("vdim", dim)
            window = KeyReader(_object(m, "mask")).positive_int("size") if m.has("mask") else None
            fields = dict(kind=kind, heads=heads, dim=dim, vdim=vdim)
            if kind == "attention":
                kv_heads = m.positive_int("kv_heads", heads)
                if heads % kv_heads != 0:
                    raise ConfigError("invalid_geometry",
                                      f"layer {i}: heads {heads} is not a multiple of kv_heads {kv_heads}")
                fields.update(kv_heads=kv_heads, scale=m.positive_float("scale"), window=window)
            elif kind == "latent_attention":
                rot_dim = m.positive_int("rot_dim")
                rr = KeyReader(_object(m, "rot"))
                dims = rr.positive_int("dims")
                if dims != rot_dim or dims % 2:
                    raise ConfigError("invalid_geometry", f"layer {i}: rot.dims {dims} must be even and equal "
                                                          f"rot_dim {rot_dim}")
                fields.update(scale=m.positive_float("scale"), window=window, rot_dim=rot_dim,
                              q_rank=m.positive_int("q_rank"), kv_rank=m.positive_int("kv_rank"),
                              rot_base=rr.positive_float("base"))
                if m.has("kv_from"):
                    j = m.raw("kv_from")
                    if isinstance(j, bool) or not isinstance(j, int) or not (0 <= j < i):
                        raise ConfigError("invalid_field", f"layer {i}: 'kv_from' must name an earlier layer")
                    src = layers[j]
                    if src.kind != "latent_attention" or src.kv_from is not None:
                        raise ConfigError("invalid_field", f"layer {i}: 'kv_from' names layer {j}, which keeps no "
                                                           f"latents of its own")
                    if (src.kv_rank, src.rot_dim, src.rot_base) != (fields["kv_rank"], rot_dim, fields["rot_base"]):
                        raise ConfigError("invalid_geometry", f"layer {i}: its kv_rank, rot_dim and rotation must "
                                                              f"equal those of layer {j}, whose cache it reads")
                    fields["kv_from"] = j
            if lr.has("mlp"):
                mlp = KeyReader(_object(lr, "mlp"))
                mlp.require_value("kind", ("moe",))
                router = KeyReader(_object(mlp, "router"))
                fields.update(ff=KeyReader(_object(mlp, "expert")).positive_int("ff"),
                              experts=router.positive_int("experts"), top=router.positive_int("top"))
                if fields["top"] > fields["experts"]:
                    raise ConfigError("invalid_geometry", f"layer {i}: top {fields['top']} exceeds experts "
                                                          f"{fields['experts']}")
            layers.append(PitudraLayer(**fields))
        return cls(vocab, width, eps, side_dim, tuple(layers))

    def kept_window(self, i: int):
        """How long layer i's cache keeps a key: the longest window among the layer and
        its readers (None: everything), so that no reader meets a page that is gone."""
        j = self.layers[i].kv_from if self.layers[i].kv_from is not None else i
        windows = [l.window for n, l in enumerate(self.layers) if n == j or l.kv_from == j]
        return None if any(w is None for w in windows) else max(windows)

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = NormSpec("layernorm", D, self.eps)
        n = len(self.layers)
        layers, order = [], []
        for i, l in enumerate(self.layers):
            names = [("mixer_norm", "norm1"), ("token_shift", "shift"), ("o_proj", "mix.o")]
            if l.kind == "latent_attention":
                position = PositionSpec(kind="rope", head_dim=l.rot_dim, rotary_dim=l.rot_dim, theta=l.rot_base)
                mixer = LatentAttentionSpec(kind="latent_attention", hidden_size=D, num_heads=l.heads, head_dim=l.dim,
                                            rope_dim=l.rot_dim, value_dim=l.vdim, q_rank=l.q_rank, kv_rank=l.kv_rank,
                                            scale=l.scale, norm_eps=self.eps, window=l.window, sink=True,
                                            own_kv=l.kv_from is None, position=position,
                                            cache_window=self.kept_window(i))
                names += [("q_down", "mix.dq"), ("q_latent_norm", "mix.dq.norm"), ("q_up", "mix.uq"),
                          ("kv_down", "mix.dkv"), ("kv_latent_norm", "mix.dkv.norm"), ("k_up", "mix.uk"),
                          ("v_up", "mix.uv"), ("sink", "mix.sink")]
            elif l.kind == "hgrn2":
                mixer = GatedRecurrenceSpec(kind="gated_recurrence", hidden_size=D, num_heads=l.heads, head_dim=l.dim,
                                            value_dim=l.vdim, norm_eps=self.eps)
                names += [("q_proj", "mix.q"), ("f_proj", "mix.f"), ("f_bias", "mix.f.b"), ("gate_floor", "mix.lower"),
                          ("v_proj", "mix.v"), ("out_norm", "mix.norm")]
            else:
                mixer = AttentionSpec(kind="attention", hidden_size=D, num_heads=l.heads, num_kv_heads=l.kv_heads,
                                      head_dim=l.dim, scale=l.scale, window=l.window,
                                      position=PositionSpec(kind="none", head_dim=l.dim), value_dim=l.vdim, sink=True,
                                      biases=True, whole_norm_eps=self.eps, output_gate=True)
                names += [("q_proj", "mix.q"), ("k_proj", "mix.k"), ("v_proj", "mix.v"), ("q_bias", "mix.q.b"),
                          ("k_bias", "mix.k.b"), ("v_bias", "mix.v.b"), ("q_norm", "mix.q.norm"),
                          ("k_norm", "mix.k.norm"), ("sink", "mix.sink"), ("g_proj", "mix.g")]
            ff = None
            if l.ff:
                ff = RoutedExpertsSpec(kind="routed_experts", hidden_size=D, intermediate_size=l.ff,
                                       num_experts=l.experts, top=l.top, activation="relu2")
                names += [("feed_forward_norm", "norm2"), ("router", "mlp.router"), ("expert_up", "mlp.e{e}.up"),
                          ("expert_down", "mlp.e{e}.down")]
            token_input = None
            if self.side_dim is not None:
                token_input = TokenInputSpec(hidden_size=D, dim=self.side_dim, offset=i * self.side_dim,
                                             table_name=SIDE_TABLE, table_width=n * self.side_dim,
                                             vocab_size=self.vocab, activation="gelu_tanh", eps=self.eps)
                names += [("token_gate", "side.gate"), ("token_proj", "side.proj"), ("token_norm", "side.norm")]
            layers.append(LayerSpec(arrangement="postnorm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, weight_prefix=f"l{i}.",
                                    weight_names=tuple(names), token_input=token_input, token_shift=True))
            order.append(RunStep(layer=i, cache_of=l.kv_from))
        shared = ()
        if self.side_dim is not None:
            shared = ((SIDE_TABLE, (self.vocab, n * self.side_dim), "float"),)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=D, max_positions=0,
            layers=tuple(layers), run_order=tuple(order), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", tie_output_to_embedding=False, shared_tensors=shared)
