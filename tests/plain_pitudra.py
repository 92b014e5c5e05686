"""A plain, slow restatement of the Pitudra design: whole sequences, no cache,
one function per mechanism, on the CPU.  It shares no code with the package: it
takes the parsed config.json and a dict of tensors by their checkpoint names and
returns logits (and, if asked, the residual stream after every layer).
``dtype`` torch.float64 gives the yardstick for both engine types.

Notation: T tokens, D width, H query heads, G key/value heads, d the size of an
unrotated query or key head, r the size of the rotated part, e a value head's
size, c the rank of the key/value latent.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w + b


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """h [T, D]: every token moves towards its predecessor (zeros before the first) by ``mix``."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mix


def rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, n]: feature i of the first ``dims`` turns with feature i + dims / 2."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(torch.float64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] True where query i sees key j: j <= i and, with a window, i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size is not None:
        seen = seen & (i - j < size)
    return seen


def softmax_with_sink(scores: torch.Tensor, sink: Optional[torch.Tensor], seen: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T]; ``sink`` [H] joins the denominator as one more, valueless column."""
    scores = scores.masked_fill(~seen[None], float("-inf"))
    if sink is None:
        return torch.softmax(scores, dim=-1)
    H, T, _ = scores.shape
    wide = torch.cat([scores, sink[:, None, None].expand(H, T, 1)], dim=-1)
    return torch.softmax(wide, dim=-1)[..., :T]


def latent_cache(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, positions: torch.Tensor, eps: float):
    """What a latent-attention layer with a projection of its own keeps per token:
    the normalised latent [T, c] and the rotated shared key part [T, r]."""
    c, r = m["kv_rank"], m["rot_dim"]
    both = h @ w[p + "dkv"].T
    latent = unit_rms(both[:, :c], eps) * w[p + "dkv.norm"]
    shared = rotate(both[:, None, c:c + r], positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))[:, 0]
    return latent, shared


def latent_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, positions: torch.Tensor, eps: float,
                     kept) -> torch.Tensor:
    T = h.shape[0]
    H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    latent, shared = kept
    cq = unit_rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    q_plain = q[..., :d]
    q_turned = rotate(q[..., d:], positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    k_plain = (latent @ w[p + "uk"].T).view(T, H, d)
    v = (latent @ w[p + "uv"].T).view(T, H, e)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_turned, shared)
    scores = scores * float(m["scale"])
    size = m["mask"]["size"] if m.get("mask") else None
    prob = softmax_with_sink(scores, w.get(p + "sink"), window_mask(T, size))
    out = torch.einsum("hij,jhe->ihe", prob, v).reshape(T, H * e)
    return out @ w[p + "o"].T


def gated_recurrence(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float,
                     margins: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One state matrix [d, e] per head; the forget gate f also sets how much is written (1 - f).
    ``margins`` [T]: the first token's output is v times the ONE number sum_d (1 - f_d) q_d, whose
    sign alone survives the norm; position 0 takes that number's size relative to the sum of its
    terms' sizes (the least over heads) if that is smaller than what is there."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, e)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).view(T, H, d)
    state = torch.zeros(H, d, e, dtype=h.dtype)
    out = torch.zeros(T, H, e, dtype=h.dtype)
    for t in range(T):
        state = f[t][:, :, None] * state + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", state, q[t])
    if margins is not None:
        terms = (1.0 - f[0]) * q[0]
        rel = (terms.sum(dim=-1).abs() / terms.abs().sum(dim=-1).clamp_min(1e-300)).min()
        margins[0] = torch.minimum(margins[0], rel.to(margins.dtype))
    out = unit_rms(out, eps) * w[p + "norm"]
    return out.reshape(T, H * e) @ w[p + "o"].T


def gated_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, e)
    q = (unit_rms(q, eps) * w[p + "q.norm"]).view(T, H, d)            # over all heads at once
    k = (unit_rms(k, eps) * w[p + "k.norm"]).view(T, G, d)
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    size = m["mask"]["size"] if m.get("mask") else None
    prob = softmax_with_sink(scores, w.get(p + "sink"), window_mask(T, size))
    out = torch.einsum("hij,jhe->ihe", prob, v).reshape(T, H * e)
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def routed_experts(w: Dict[str, torch.Tensor], p: str, mlp: dict, x: torch.Tensor,
                   margins: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``margins`` [T]: takes, where smaller, the gap between the last chosen logit and the best one
    left out, relative to the largest |logit| of the token (how close the choice was)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = x @ w[p + "router"].T
    best, chosen = torch.topk(logits, top, dim=-1)
    if margins is not None and top < E:
        ordered = torch.sort(logits, dim=-1, descending=True).values
        gap = (ordered[:, top - 1] - ordered[:, top]) / logits.abs().max(dim=-1).values.clamp_min(1e-300)
        margins.copy_(torch.minimum(margins, gap.to(margins.dtype)))
    share = torch.softmax(best, dim=-1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for s in range(top):
            n = int(chosen[t, s])
            inner = torch.relu(w[f"{p}e{n}.up"] @ x[t]) ** 2
            out[t] += share[t, s] * (w[f"{p}e{n}.down"] @ inner)
    return out


def token_input(w: Dict[str, torch.Tensor], p: str, x: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, layer: int,
                dim: int, eps: float) -> torch.Tensor:
    e = table[ids][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return unit_rms(y, eps) * w[p + "norm"]


def forward(config: dict, weights: Dict[str, torch.Tensor], token_ids: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None, margins: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``margins`` (float64 [T], filled with inf by the caller) takes per position the closest of the
    design's two kinds of close call (see ``routed_experts`` and ``gated_recurrence``): where it is small,
    an implementation that rounds differently may rightly decide the other way."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    ids = torch.tensor(token_ids, dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    side = (config.get("token_side") or {}).get("dim")
    x = w["embed"][ids]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = token_shift(x, w[p + "shift"]) if p + "shift" in w else x
        if layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_cache(w, p + "mix.", m, h, positions, eps)
            y = latent_attention(w, p + "mix.", m, h, positions, eps, kept[m["kv_from"] if m.get("kv_from") is not None else i])
        elif layer["type"] == "hgrn2":
            y = gated_recurrence(w, p + "mix.", m, h, eps, margins)
        elif layer["type"] == "attention":
            y = gated_attention(w, p + "mix.", m, h, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + layer_norm(y, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer.get("mlp") is not None:
            y = routed_experts(w, p + "mlp.", layer["mlp"], x, margins)
            x = x + layer_norm(y, w[p + "norm2"], w[p + "norm2.b"], eps)
        if side:
            x = x + token_input(w, p + "side.", x, ids, w["side.embed"], i, side, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].T
