"""Architecture-neutral description of a decoder: parts, layers and run order.

A configuration class (one per architecture) turns the keys of its own
``config.json`` into a :class:`ModelSpec`.  Everything below the configuration
(weights loader, parts, cache manager, step function) reads only the spec, so
no part knows which model it is in.

Every size and constant is a field of a spec; nothing here has a default that
stands for a model's value.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last ``size`` features.

    ``kind`` names a registered norm part ("rmsnorm"; "layernorm": the mean is
    taken off first, the variance is the mean of the squared deviations, and a
    bias, the tensor of the weight's name with ``bias_suffix`` added, follows the
    weight).  ``weight_offset`` is added to the stored weight before use (0 for
    plain RMSNorm, 1 for the zero-centred variant).
    """

    kind: str
    size: int
    eps: float
    weight_offset: float = 0.0
    bias_suffix: str = ".b"


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer.

    ``kind`` "rope": split-half rotation of the first ``rotary_dim`` features
    of every head with ``inv_freq[j] = theta ** (-2j / rotary_dim)``.
    ``kind`` "none": nothing is applied.

    ``scaling_factor`` s > 0 stretches the slow frequencies for contexts longer
    than ``original_positions`` (the YaRN rule): with
    turn(t) = rotary_dim * ln(original_positions / (2 pi t)) / (2 ln theta),
    lo = max(floor(turn(fast_turns)), 0), hi = min(ceil(turn(slow_turns)), rotary_dim - 1)
    and ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1), frequency j becomes
    inv_freq[j] * (ramp_j / s + 1 - ramp_j), and cosines and sines are multiplied by
    ``amplitude_slope`` * ln(s) + 1.  0 switches it off.

    ``wavelength_bands`` (factor, low, high, original), None = off: frequencies are divided by
    ``factor`` according to their wavelength l = 2 pi / f.  l < original / high keeps f;
    l > original / low gives f / factor; between the two, with
    s = (original / l - low) / (high - low), the frequency is (1 - s) * f / factor + s * f.
    """

    kind: str
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 0.0
    scaling_factor: float = 0.0
    original_positions: int = 0
    fast_turns: float = 0.0
    slow_turns: float = 0.0
    amplitude_slope: float = 0.0
    wavelength_bands: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class MixerSpec:
    """Base of all token mixers; ``kind`` names a registered mixer part."""

    kind: str


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    """Causal grouped-query attention over a paged key/value cache.

    ``window`` None means every earlier key is visible; an integer W means the
    W most recent keys, the query's own included.  ``scale`` multiplies the
    scores after the dot product.  ``softcap`` c (None: off) then replaces a
    score s by c * tanh(s / c).  ``distance_bias`` "log" then takes
    r1[h] * ln(1 + r2[h] * (i - j)) off the score of query i and key j, with two
    learned numbers per query head (tensor roles "distance_r1", "distance_r2").
    ``tied_values``: the values are the keys as projected; there is no value
    projection and the cache holds keys only.
    ``value_dim`` (None: ``head_dim``): the size of a value head where it differs
    from that of a query or key head.  ``chunk`` C: position i sees j <= i only
    if floor(i / C) = floor(j / C), blocks counted from the sequence's start.
    ``unit_norm_eps`` (None: off): after the rotation every q and k head is
    divided by its root mean square (this eps inside the root), without a
    weight; ``qk_norm`` by contrast comes before the rotation and has weights.
    ``own_kv`` False: the layer has no key and value projections at all and runs
    only as a reader of another run step's cache (``RunStep.cache_of``).
    ``sink``: a learned number per query head (tensor role "sink") joins the
    softmax's denominator as exp(sink), unscaled, without a key or a value.
    ``biases``: the q, k and v projections add a vector each (roles "q_bias",
    "k_bias", "v_bias").  ``whole_norm_eps`` (None: off): q and k are divided by
    the root mean square of their WHOLE projection (all heads at once, this eps
    inside the root) and multiplied by weights of that size (roles "q_norm",
    "k_norm"), before any rotation.  ``output_gate``: the concatenated heads are
    multiplied by sigmoid(Wg x) (role "g_proj") before the output projection.
    ``cache_window``: how long the cache keeps a key where that is not ``window``
    (a layer whose cache a layer with a longer window reads); "same" = ``window``.

    ``distance_bias`` "linear": slope[h] * (i - j) is taken off the score, with
    slope[h] = 2 ** (-``distance_slope_bits`` * (h + 1) / num_heads); no tensors.
    ``query_maps`` M > 1: every query head has M score maps (q has num_heads * M * head_dim
    rows, k num_kv_heads * M * head_dim, a head's maps side by side), each an attention of its
    own over the head's one value.  ``differential`` c (with two maps): the maps' outputs
    a1, a2 are joined as o = a1 - lambda * a2 with
    lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + c (four vectors of head_dim numbers,
    roles "lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"), o is divided by its root mean
    square over the head's values (``differential_eps`` inside the root, no weight) and
    multiplied by 1 - c.  ``head_gate``: head h's output is multiplied by sigmoid(Wg x)[h], one
    number per head (role "head_gate", [num_heads, hidden]), before the output projection.
    ``biases`` together with ``qk_norm``: the biases are added first, then every q and k head is
    normalised with the shared weight, then rotated.
    """

    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec(kind="none")
    softcap: Optional[float] = None
    distance_bias: Optional[str] = None
    tied_values: bool = False
    value_dim: Optional[int] = None
    chunk: Optional[int] = None
    unit_norm_eps: Optional[float] = None
    own_kv: bool = True
    sink: bool = False
    biases: bool = False
    whole_norm_eps: Optional[float] = None
    output_gate: bool = False
    cache_window: object = "same"
    distance_slope_bits: float = 8.0
    query_maps: int = 1
    differential: Optional[float] = None
    differential_eps: float = 0.0
    head_gate: bool = False


@dataclass(frozen=True)
class StateSpaceSpec(MixerSpec):
    """A selective state-space mixer with a scalar decay per head.  With inner =
    ``num_heads`` * ``value_dim``, N = ``state_size`` and G = ``groups``, the input projection
    (role "in_proj") gives z [inner] | x [inner] | B [G N] | C [G N] | dt [num_heads].  x | B | C
    pass a causal convolution per channel (``conv_taps`` taps, role "conv" [channels, taps] with
    the current token's tap last, bias role "conv_bias") and silu.  Per head h of group
    floor(h / (num_heads / G)), with step = softplus(dt + dt_bias) (no clamp):

        S <- exp(-exp(A_log[h]) * step) S + step * B x^T      (S is N by value_dim, 32-bit)
        y  = S^T C + D[h] x

    y * silu(z) is divided, in ``norm_groups`` equal parts, by each part's root mean square
    (``norm_eps`` inside the root) and multiplied by a weight (role "out_norm"), then projected
    (role "o_proj").  The state and the convolution's last ``conv_taps`` - 1 inputs are kept
    per request (roles "dt_bias", "a_log", "skip" name the per-head vectors)."""

    hidden_size: int = 0
    num_heads: int = 0
    value_dim: int = 0
    state_size: int = 0
    groups: int = 1
    conv_taps: int = 1
    norm_groups: int = 1
    norm_eps: float = 0.0


@dataclass(frozen=True)
class ParallelMixersSpec(MixerSpec):
    """Two mixers side by side that read the same input; the result is
    ``left_scale`` * left + ``right_scale`` * right.  The tensor roles of the two are those of
    their kinds with "left." / "right." in front."""

    left: MixerSpec = None
    right: MixerSpec = None
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass(frozen=True)
class LatentAttentionSpec(MixerSpec):
    """Attention whose keys and values are made from one cached latent per token.

    c_q = RMSNorm(W_dq x) (``q_rank`` features, weight role "q_latent_norm"),
    q = W_uq c_q: per head ``head_dim`` plain features followed by ``rope_dim``
    rotated ones.  W_dkv x has ``kv_rank`` + ``rope_dim`` rows: the first,
    RMS-normalised (role "kv_latent_norm"), are the latent c; the last, rotated,
    are one key part that all heads share.  Head h's plain key is W_uk[h] c, its
    value W_uv[h] c (``value_dim`` features); score = (q_plain . k_plain +
    q_rot . k_rot) * ``scale``.  The cache holds c and the rotated part only
    (one row of ``kv_rank`` + ``rope_dim`` numbers per token).  ``window``,
    ``sink``, ``own_kv`` and ``cache_window`` as for AttentionSpec (a layer
    without W_dkv reads another step's cache with W_uk and W_uv of its own).
    ``position`` rotates the ``rope_dim`` part (its ``head_dim`` is ``rope_dim``).
    """

    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    value_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 0.0
    norm_eps: float = 0.0
    window: Optional[int] = None
    sink: bool = False
    own_kv: bool = True
    position: PositionSpec = PositionSpec(kind="none")
    cache_window: object = "same"


@dataclass(frozen=True)
class GatedRecurrenceSpec(MixerSpec):
    """Linear attention whose forget gate also sets what is written: per head a
    state S [``head_dim``, ``value_dim``] (32-bit, zero at a sequence's start),

        q = silu(Wq x),  v = Wv x,  f = l + (1 - l) * sigmoid(Wf x + bf)
        S <- diag(f) S + (1 - f) v^T,   o = S^T q

    with a lower bound l per gate channel (role "gate_floor").  Each head's o is
    divided by its root mean square (``norm_eps`` inside the root) and multiplied by
    a weight of ``value_dim`` numbers that the heads share (role "out_norm"), then
    projected back to ``hidden_size``.
    """

    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    norm_eps: float = 0.0


@dataclass(frozen=True)
class DeltaRuleSpec(MixerSpec):
    """Linear recurrence with a state matrix per head (``head_dim`` key rows by
    ``head_dim`` value columns, 32-bit, zero at a sequence's start).  With r, k, v
    projections of the input, a decay per key channel
    w = exp(-``decay_scale`` * sigmoid(W2 tanh(W1 x) + w0)) (W1 of low rank), a
    removal rate per key channel a = sigmoid(Wa x + ba) and the unit key
    u = k / sqrt(sum(k^2) + ``key_eps``):

        S <- diag(w) S - (a * u) (u^T S) + k v^T      (both products read the old S)
        o  = S^T r

    Each head's o is divided by its root mean square (``norm_eps`` inside the
    root), multiplied by a weight over all heads and by sigmoid(Wg x), and
    projected back to ``hidden_size``.
    """

    hidden_size: int = 0
    num_heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0
    decay_scale: float = 0.0
    key_eps: float = 0.0
    norm_eps: float = 0.0


@dataclass(frozen=True)
class ShortConvSpec:
    """A causal convolution over time on each channel, added to its input:
    y_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j), zeros before the sequence's
    start.  The last ``taps`` - 1 inputs are part of a request's state."""

    size: int
    taps: int


@dataclass(frozen=True)
class FeedForwardSpec:
    """Base of all feed-forward parts; ``kind`` names a registered part."""

    kind: str


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x)); ``activation`` "silu"
    or "gelu_tanh".  ``biases``: every one of the three products adds a vector
    (tensor roles "gate_bias", "up_bias", "down_bias").  ``activation`` "swish_clamped":
    g = min(gate(x), ``limit``), u = clamp(up(x), -``limit``, ``limit``) and the product is
    down(g * sigmoid(``gate_slope`` * g) * (u + 1))."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"
    biases: bool = False
    limit: float = 0.0
    gate_slope: float = 1.702


@dataclass(frozen=True)
class TableExpertsSpec(FeedForwardSpec):
    """``num_experts`` small gated feed-forwards without biases, of which every
    token uses ``top``: an integer table [vocab_size, top] (tensor role
    "expert_table"; the entries of a row differ) names them by the token's id, and
    the output is the mean of theirs.  Tensor roles of expert e: "expert_gate",
    "expert_up", "expert_down", each a name with ``{e}`` where the number goes."""

    hidden_size: int = 0
    intermediate_size: int = 0
    num_experts: int = 0
    top: int = 0
    vocab_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class RoutedExpertsSpec(FeedForwardSpec):
    """``num_experts`` small feed-forwards without gate or biases, down(act(up(x))),
    of which every token uses ``top``: those with the largest router logits
    (z = W_router x in 32-bit; role "router"), weighted by the softmax over the
    chosen logits only.  ``activation``: "relu2" (the square of relu), "relu",
    "silu", "gelu" or "gelu_tanh".  Tensor roles of expert e: "expert_up",
    "expert_down", each a name with ``{e}`` where the number goes.

    ``gated``: an expert is down(act(gate(x)) * up(x)) (role "expert_gate" too).
    ``scores`` "softmax_all": the router has ``num_experts`` + ``identity_experts`` outputs,
    s = softmax over all of them, the choice goes by s + a correction per output (role
    "correction", if ``correction``) and the weights are the chosen outputs' s (without the
    correction) times ``weight_scale``, not renormalised.  ``group_count`` / ``group_keep``:
    the outputs form ``group_count`` equal groups of neighbours, a group's score is its largest
    choice score, and only outputs of the ``group_keep`` best groups can be chosen.  The last
    ``identity_experts`` outputs name experts without tensors that return their input.
    ``shared_size`` > 0: one more gated expert of that inner size (roles "shared_gate",
    "shared_up", "shared_down") runs for every token with weight one."""

    hidden_size: int = 0
    intermediate_size: int = 0
    num_experts: int = 0
    top: int = 0
    activation: str = "relu2"
    gated: bool = False
    scores: str = "softmax_top"
    correction: bool = False
    group_count: int = 1
    group_keep: int = 1
    identity_experts: int = 0
    weight_scale: float = 1.0
    shared_size: int = 0


@dataclass(frozen=True)
class TokenInputSpec:
    """A per-layer input from the token's id at the end of a block.  A table shared
    by all layers (``table_name`` [vocab_size, table_width]) holds ``dim`` features
    per layer, this layer's from column ``offset`` on.  With x the residual:
    g = act(G x) * e[token]; y = P g; x += residual_scale * y / rms(y) * w
    (tensor roles "token_gate" [dim, hidden], "token_proj" [hidden, dim],
    "token_norm" [hidden]; ``eps`` inside the root)."""

    hidden_size: int
    dim: int
    offset: int
    table_name: str
    table_width: int
    vocab_size: int
    activation: str
    eps: float


@dataclass(frozen=True)
class DenseMLPSpec(FeedForwardSpec):
    """Dense feed-forward without a gate: down(act(up(x))).  ``activation``:
    "gelu" (exact, with erf), "gelu_tanh", "silu" or "relu"."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "gelu"


@dataclass(frozen=True)
class LayerSpec:
    """One block: how mixer, feed-forward and norms are arranged.

    ``arrangement`` names a registered block ("prenorm": x + mixer(norm(x)),
    then x + ff(norm(x)); "postnorm": the norms sit on the sublayers' outputs,
    x + norm(mixer(x)), then x + norm(ff(x))).  ``token_shift`` (arrangement
    "postnorm"): the mixer reads h + (h' - h) * w with h' the token before (zeros
    before the first; tensor role "token_shift"), and the last h is part of a
    request's state.  ``weight_prefix`` is the checkpoint prefix of the
    block's tensors.  ``weight_names`` maps the part-local tensor roles to
    checkpoint names under that prefix.  ``feed_forward`` (with its norm) may be
    None: the block then ends after the mixer.  ``mixer_conv``: a short
    convolution between the mixer's norm and the mixer (tensor role
    "mixer_conv").
    """

    arrangement: str
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    feed_forward_norm: Optional[NormSpec]
    weight_prefix: str
    weight_names: Tuple[Tuple[str, str], ...] = ()
    mixer_conv: Optional[ShortConvSpec] = None
    # arrangement "parallel": one norm, x += residual_scale * (mixer(norm(x)) + ff(norm(x)))
    residual_scale: float = 1.0
    token_input: Optional[TokenInputSpec] = None
    token_shift: bool = False
    # arrangement "prenorm": the mixer's and the feed-forward's results are multiplied feature by feature
    # by a learned vector each (roles "mixer_scale", "feed_forward_scale") before they join the residual
    layer_scale: bool = False

    def names(self) -> dict:
        return dict(self.weight_names)


@dataclass(frozen=True)
class RunStep:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice: its
    weights are shared, every run has a cache of its own).  ``cache_of`` names
    an earlier run step whose cache this step reads instead of writing one.
    ``enter`` indexes ``ModelSpec.stream_adapters``: that adapter transforms the
    residual stream right before this step, with ``turn`` as its argument (the
    number of the pass that begins here, for a group of layers that runs
    several times).
    """

    layer: int
    cache_of: Optional[int] = None
    enter: Optional[int] = None
    turn: int = 0


@dataclass(frozen=True)
class AdapterSpec:
    """A part at one of the decoder's ends: after the token embedding (it
    changes the residual stream in place: a learned or absolute position table,
    a scale of the embeddings) or on the logits of the wanted rows (a soft cap,
    a bias).  ``kind`` names a registered adapter part; ``weight_names`` maps
    its tensor roles to checkpoint names; ``params`` are its constants."""

    kind: str
    weight_names: Tuple[Tuple[str, str], ...] = ()
    params: Tuple[Tuple[str, float], ...] = ()

    def names(self) -> dict:
        return dict(self.weight_names)

    def constants(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class ModelSpec:
    """A whole decoder: embedding, what follows it at once, layers, run order,
    final norm, output, what is done to the logits."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int                                # 0: no limit of the model's own (the cache pool bounds a request)
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunStep, ...]
    final_norm: NormSpec
    embedding_name: str
    final_norm_name: str
    output_name: str
    tie_output_to_embedding: bool
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    extra: dict = field(default_factory=dict, compare=False)
    input_adapters: Tuple[AdapterSpec, ...] = ()      # run on the residual right after the embedding
    logit_adapters: Tuple[AdapterSpec, ...] = ()      # run on the 32-bit logits of the wanted rows
    stream_adapters: Tuple[AdapterSpec, ...] = ()     # run on the residual where a run step's ``enter`` names them
    # tensors that several parts read and none owns: (name, shape, "float" | "int"); every part finds
    # them in the dict it is bound with
    shared_tensors: Tuple[Tuple[str, Tuple[int, ...], str], ...] = ()
