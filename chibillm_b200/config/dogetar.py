"""Dogetar: the typed configuration and its translation into parts.

A Dogetar config.json names the architecture under "architecture" and gives every
size and constant in nested objects:

* "vocab", "width"; "norm": {"eps"}; "logit_softcap" (optional);
* "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}} (optional);
* "loop": {"start", "stop", "times"} (optional): layers start .. stop - 1 run "times" times;
* "layers": one object per layer with "type", "mixer" and "mlp" (null: none).
  - type "attention_2": "heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"} (a sliding
    window), "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}};
  - type "attention": the same keys without "scaling", "mask" a block size, plus "diff";
  - type "parallel": "left" (an attention: "heads", "kv_heads", "dim", "vdim", "scale", "mask" a
    block size), "right" (a state-space mixer: "heads", "vdim", "state", "groups", "conv",
    "norm_groups"), "left_scale", "right_scale".
  "mlp": {"kind": "dense", "ff", "limit"} or {"kind": "moe", "expert": {"ff"}, "router":
  {"experts", "top", "identity", "scale", "groups": {"count", "keep"}}, "shared": {"ff"}}.

Absent optional objects ("mask", "rot", "scaling", "vdim", "kv_heads", "groups", "identity",
"shared", "bigram", "loop", "logit_softcap") switch their mechanism off or fall back to the plain
value.

What the design fixes: RMS norms before the sublayers; a learned scale per feature on each
sublayer's result; "attention_2" has biases on q, k, v and a weighted RMS norm per q and k head
before the rotation; "attention" has two score maps per head joined as a1 - lambda a2, a unit
norm over the joined head and a sigmoid gate per head; the left branch of "parallel" has no
rotation, a bias of slope 2^(-8 (h + 1) / H) per unit of distance and a sink; the dense
feed-forward is min(g, L) sigmoid(1.702 min(g, L)) (clamp(u) + 1); the routed experts are
silu-gated, chosen by softmax score plus a correction within the best groups.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, KeyReader, finite_number, object_at as _object
from .spec import (AdapterSpec, AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, ParallelMixersSpec,
                   PositionSpec, RoutedExpertsSpec, RunStep, StateSpaceSpec)

ARCHITECTURE = "Dogetar"
MIXERS = ("attention", "attention_2", "parallel")
GATE_SLOPE = 1.702
SLOPE_BITS = 8.0


def _non_negative_int(reader: KeyReader, key: str) -> int:
    v = reader.raw(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError("invalid_field", f"key '{key}' must be a non-negative integer, got {v!r}")
    return v


@dataclass(frozen=True)
class DogetarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: Optional[int] = None
    rot_dims: int = 0                       # 0: no rotation
    rot_base: float = 0.0
    rot_bands: Optional[Tuple[float, float, float, float]] = None
    diff: Optional[float] = None


@dataclass(frozen=True)
class DogetarStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class DogetarMLP:
    kind: str                               # "dense" | "moe"
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    identity: int = 0
    scale: float = 1.0
    group_count: int = 1
    group_keep: int = 1
    shared_ff: int = 0


@dataclass(frozen=True)
class DogetarLayer:
    kind: str                               # one of MIXERS
    attention: Optional[DogetarAttention]
    state_space: Optional[DogetarStateSpace] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[DogetarMLP] = None


def _read_attention(m: KeyReader, where: str, rotation: bool, diff: bool) -> DogetarAttention:
    heads, dim = m.positive_int("heads"), m.positive_int("dim")
    kv_heads = m.positive_int("kv_heads", heads)
    if heads % kv_heads != 0:
        raise ConfigError("invalid_geometry", f"{where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    fields = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=m.positive_int("vdim", dim),
                  scale=m.positive_float("scale"),
                  mask=KeyReader(_object(m, "mask")).positive_int("size") if m.has("mask") else None)
    if rotation and m.has("rot"):
        rr = KeyReader(_object(m, "rot"))
        dims = rr.positive_int("dims")
        if dims % 2 or dims > dim:
            raise ConfigError("invalid_geometry", f"{where}: rot.dims {dims} must be even and at most dim {dim}")
        fields.update(rot_dims=dims, rot_base=rr.positive_float("base"))
        if rr.has("scaling"):
            sc = KeyReader(_object(rr, "scaling"))
            bands = (sc.positive_float("factor"), sc.positive_float("low"), sc.positive_float("high"),
                     sc.positive_float("original"))
            if bands[2] == bands[1]:
                raise ConfigError("invalid_field", f"{where}: rot.scaling needs high != low")
            fields["rot_bands"] = bands
    if diff:
        fields["diff"] = finite_number(m, "diff")
    return DogetarAttention(**fields)


def _read_mlp(raw, where: str) -> DogetarMLP:
    mlp = KeyReader(raw)
    kind = mlp.require_value("kind", ("dense", "moe"))
    if kind == "dense":
        return DogetarMLP(kind=kind, ff=mlp.positive_int("ff"), limit=mlp.positive_float("limit"))
    router = KeyReader(_object(mlp, "router"))
    experts, top = router.positive_int("experts"), router.positive_int("top")
    identity = _non_negative_int(router, "identity") if router.has("identity") else 0
    count = keep = 1
    if router.has("groups"):
        g = KeyReader(_object(router, "groups"))
        count, keep = g.positive_int("count"), g.positive_int("keep")
    outputs = experts + identity
    if outputs % count != 0 or keep > count:
        raise ConfigError("invalid_geometry", f"{where}: {outputs} router outputs do not form {count} equal groups "
                                              f"of which {keep} are kept")
    if top > (outputs // count) * keep:
        raise ConfigError("invalid_geometry", f"{where}: top {top} exceeds the outputs of the kept groups")
    return DogetarMLP(kind=kind, ff=KeyReader(_object(mlp, "expert")).positive_int("ff"), experts=experts, top=top,
                      identity=identity, scale=router.positive_float("scale", 1.0), group_count=count,
                      group_keep=keep,
                      shared_ff=KeyReader(_object(mlp, "shared")).positive_int("ff") if mlp.has("shared") else 0)


@dataclass(frozen=True)
class DogetarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[DogetarLayer, ...]
    bigram: Optional[Tuple[int, int, int]] = None          # buckets, mul_prev, mul_cur
    loop: Optional[Tuple[int, int, int]] = None            # start, stop, times
    logit_softcap: Optional[float] = None

    @classmethod
    def from_dict(cls, obj: dict) -> "DogetarConfig":
        r = KeyReader(obj)
        vocab, width = r.positive_int("vocab"), r.positive_int("width")
        eps = KeyReader(_object(r, "norm")).positive_float("eps")
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("invalid_field", "key 'layers' must be a non-empty list")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw)
            kind = lr.require_value("type", MIXERS)
            m = KeyReader(_object(lr, "mixer"))
            where = f"layer {i}"
            if kind == "parallel":
                right = KeyReader(_object(m, "right"))
                ss = DogetarStateSpace(heads=right.positive_int("heads"), vdim=right.positive_int("vdim"),
                                       state=right.positive_int("state"), groups=right.positive_int("groups", 1),
                                       conv=right.positive_int("conv"), norm_groups=right.positive_int("norm_groups", 1))
                if ss.heads % ss.groups != 0 or (ss.heads * ss.vdim) % ss.norm_groups != 0:
                    raise ConfigError("invalid_geometry", f"{where}: heads {ss.heads} must be a multiple of groups "
                                                          f"{ss.groups}, and heads * vdim of norm_groups {ss.norm_groups}")
                fields = dict(attention=_read_attention(KeyReader(_object(m, "left")), where + " (left)", False, False),
                              state_space=ss, left_scale=finite_number(m, "left_scale") if m.has("left_scale") else 1.0,
                              right_scale=finite_number(m, "right_scale") if m.has("right_scale") else 1.0)
            else:
                fields = dict(attention=_read_attention(m, where, True, kind == "attention"))
            mlp = _read_mlp(_object(lr, "mlp"), where) if lr.has("mlp") else None
            layers.append(DogetarLayer(kind=kind, mlp=mlp, **fields))
        bigram = None
        if r.has("embedding") and KeyReader(_object(r, "embedding")).has("bigram"):
            b = KeyReader(_object(KeyReader(_object(r, "embedding")), "bigram"))
            bigram = (b.positive_int("buckets"), _non_negative_int(b, "mul_prev"), _non_negative_int(b, "mul_cur"))
        loop = None
        if r.has("loop"):
            lp = KeyReader(_object(r, "loop"))
            start, stop, times = _non_negative_int(lp, "start"), lp.positive_int("stop"), lp.positive_int("times")
            if not (start < stop <= len(layers)):
                raise ConfigError("invalid_field", f"loop: start {start} < stop {stop} <= {len(layers)} layers is required")
            loop = (start, stop, times)
        cap = r.positive_float("logit_softcap") if r.has("logit_softcap") else None
        return cls(vocab, width, eps, tuple(layers), bigram, loop, cap)

    # ---- translation
    def _attention_spec(self, a: DogetarAttention, kind: str, prefix: str, names: list) -> AttentionSpec:
        D = self.width
        position = PositionSpec(kind="none", head_dim=a.dim)
        if a.rot_dims:
            position = PositionSpec(kind="rope", head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base,
                                    wavelength_bands=a.rot_bands)
        common = dict(kind="attention", hidden_size=D, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim,
                      scale=a.scale, position=position, value_dim=a.vdim)
        names += [(prefix + "q_proj", "mix." + prefix + "q"), (prefix + "k_proj", "mix." + prefix + "k"),
                  (prefix + "v_proj", "mix." + prefix + "v"), (prefix + "o_proj", "mix." + prefix + "o")]
        if kind == "attention_2":
            names += [("q_bias", "mix.q.b"), ("k_bias", "mix.k.b"), ("v_bias", "mix.v.b"),
                      ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm")]
            return AttentionSpec(window=a.mask, biases=True, qk_norm=NormSpec("rmsnorm", a.dim, self.eps), **common)
        if kind == "attention":
            names += [("lambda_q1", "mix.lq1"), ("lambda_k1", "mix.lk1"), ("lambda_q2", "mix.lq2"),
                      ("lambda_k2", "mix.lk2"), ("head_gate", "mix.g")]
            return AttentionSpec(chunk=a.mask, query_maps=2, differential=a.diff, differential_eps=self.eps,
                                 head_gate=True, **common)
        names.append((prefix + "sink", "mix." + prefix + "sink"))
        return AttentionSpec(chunk=a.mask, distance_bias="linear", distance_slope_bits=SLOPE_BITS, sink=True, **common)

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = NormSpec("rmsnorm", D, self.eps)
        layers = []
        for i, l in enumerate(self.layers):
            names = [("mixer_norm", "norm1"), ("mixer_scale", "ls1")]
            if l.kind == "parallel":
                left = self._attention_spec(l.attention, "left", "left.", names)
                s = l.state_space
                right = StateSpaceSpec(kind="state_space", hidden_size=D, num_heads=s.heads, value_dim=s.vdim,
                                       state_size=s.state, groups=s.groups, conv_taps=s.conv,
                                       norm_groups=s.norm_groups, norm_eps=self.eps)
                names += [("right." + role, "mix.right." + name) for role, name in (
                    ("in_proj", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"),
                    ("a_log", "A_log"), ("skip", "D"), ("out_norm", "norm"), ("o_proj", "o"))]
                mixer = ParallelMixersSpec(kind="parallel_mixers", left=left, right=right, left_scale=l.left_scale,
                                           right_scale=l.right_scale)
            else:
                mixer = self._attention_spec(l.attention, l.kind, "", names)
            ff = None
            if l.mlp is not None:
                names += [("feed_forward_norm", "norm2"), ("feed_forward_scale", "ls2")]
                if l.mlp.kind == "dense":
                    ff = GatedMLPSpec(kind="gated_mlp", hidden_size=D, intermediate_size=l.mlp.ff,
                                      activation="swish_clamped", limit=l.mlp.limit, gate_slope=GATE_SLOPE)
                    names += [("gate_proj", "mlp.gate"), ("up_proj", "mlp.up"), ("down_proj", "mlp.down")]
                else:
                    m = l.mlp
                    ff = RoutedExpertsSpec(kind="routed_experts", hidden_size=D, intermediate_size=m.ff,
                                           num_experts=m.experts, top=m.top, activation="silu", gated=True,
                                           scores="softmax_all", correction=True, group_count=m.group_count,
                                           group_keep=m.group_keep, identity_experts=m.identity,
                                           weight_scale=m.scale, shared_size=m.shared_ff)
                    names += [("router", "mlp.router"), ("correction", "mlp.correction"),
                              ("expert_gate", "mlp.e{e}.gate"), ("expert_up", "mlp.e{e}.up"),
                              ("expert_down", "mlp.e{e}.down"), ("shared_gate", "mlp.shared.gate"),
                              ("shared_up", "mlp.shared.up"), ("shared_down", "mlp.shared.down")]
            layers.append(LayerSpec(arrangement="prenorm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, weight_prefix=f"l{i}.",
                                    weight_names=tuple(names), layer_scale=True))
        n = len(layers)
        stream = ()
        if self.loop is None:
            order = [RunStep(layer=i) for i in range(n)]
        else:
            start, stop, times = self.loop
            stream = (AdapterSpec(kind="reentry_add", weight_names=(("step", "loop.step"),),
                                  params=(("hidden_size", D), ("turns", times))),)
            order = [RunStep(layer=i) for i in range(start)]
            for t in range(times):
                order += [RunStep(layer=i, enter=0 if i == start else None, turn=t) for i in range(start, stop)]
            order += [RunStep(layer=i) for i in range(stop, n)]
        inputs = ()
        if self.bigram is not None:
            buckets, mul_prev, mul_cur = self.bigram
            inputs = (AdapterSpec(kind="bigram", weight_names=(("table", "bigram"),),
                                  params=(("hidden_size", D), ("buckets", buckets), ("mul_prev", mul_prev),
                                          ("mul_cur", mul_cur))),)
        logits = ()
        if self.logit_softcap is not None:
            logits = (AdapterSpec(kind="softcap", params=(("cap", self.logit_softcap),)),)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=D, max_positions=0,
            layers=tuple(layers), run_order=tuple(order), final_norm=norm, embedding_name="embed",
            final_norm_name="final.norm", output_name="head", tie_output_to_embedding=False,
            input_adapters=inputs, logit_adapters=logits, stream_adapters=stream)
