"""Dogetar, written out plainly: whole sequences, no cache, one function per mechanism.

Everything here is torch on the CPU in the type of the tensors it is given (float64 in the tests).
It shares no code with the package: the tests compare the engine with it.

`config` is the design's nested config.json as a dict, `w` a dict of tensors by name.
"""
import math

import torch


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ---------------------------------------------------------------- embedding

def bigram_rows(tokens, cfg):
    """Row of the bigram table for every token of one sequence."""
    n = cfg["buckets"]
    rows = [n]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * cfg["mul_prev"] + b * cfg["mul_cur"]) % n)
    return rows


def embed(tokens, config, w):
    x = w["embed"][tokens]
    bg = (config.get("embedding") or {}).get("bigram")
    if bg:
        x = x + w["bigram"][torch.tensor(bigram_rows([int(t) for t in tokens], bg))]
    return x


# ---------------------------------------------------------------- positions and masks

def rotary_frequencies(rot):
    d = rot["dims"]
    f = [rot["base"] ** (-2.0 * i / d) for i in range(d // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for x in f:
            wave = 2 * math.pi / x
            if wave < sc["original"] / sc["high"]:
                out.append(x)
            elif wave > sc["original"] / sc["low"]:
                out.append(x / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * x / sc["factor"] + s * x)
        f = out
    return f


def rotate(x, rot):
    """x: [T, heads, dim]; pairs (i, i + dims / 2) of the first dims features, position = row."""
    if not rot:
        return x
    d = rot["dims"]
    f = torch.tensor(rotary_frequencies(rot), dtype=x.dtype)
    a = torch.arange(x.shape[0], dtype=x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :d // 2], x[..., d // 2:d]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., d:]], -1)


def visible(T, window=None, chunk=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window:
        m &= (i - j) < window
    if chunk:
        m &= (i // chunk) == (j // chunk)
    return m


def softmax_attention(q, k, v, scale, mask, bias=None, sink=None):
    """q: [T, H, d], k: [T, G, d], v: [T, G, e]; bias: [H, T, T] taken off the scores; sink: [H]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if bias is not None:
            s = s - bias[h]
        s = s.masked_fill(~mask, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out.append((e / den) @ v[:, g])
    return torch.stack(out, 1)


# ---------------------------------------------------------------- mixers

def mixer_attention_2(h, m, w, p, eps):
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, e)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    mask = visible(T, window=(m.get("mask") or {}).get("size"))
    o = softmax_attention(q, k, v, m["scale"], mask)
    return o.reshape(T, H * e) @ w[p + "o"].T


def differential_lambda(m, w, p):
    return (torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum())
            + m["diff"])


def mixer_attention(h, m, w, p, eps):
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).view(T, H * 2, d)
    k = (h @ w[p + "k"].T).view(T, G * 2, d)
    v = (h @ w[p + "v"].T).view(T, G, e)
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    q, k = q.view(T, H, 2, d), k.view(T, G, 2, d)
    mask = visible(T, chunk=(m.get("mask") or {}).get("size"))
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], mask)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], mask)
    o = a1 - differential_lambda(m, w, p) * a2
    o = rms_unit(o, eps) * (1 - m["diff"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * e) @ w[p + "o"].T


def distance_slopes(H, dtype):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def mixer_biased_sink_attention(h, m, w, p):
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, e)
    i = torch.arange(T, dtype=h.dtype)
    bias = distance_slopes(H, h.dtype)[:, None, None] * (i[:, None] - i[None, :])[None]
    mask = visible(T, chunk=(m.get("mask") or {}).get("size"))
    o = softmax_attention(q, k, v, m["scale"], mask, bias=bias, sink=w[p + "sink"])
    return o.reshape(T, H * e) @ w[p + "o"].T


def causal_conv(x, weight, bias):
    """x: [T, C], weight: [C, taps] (last column is the current token's), zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    pad = torch.cat([x.new_zeros(taps - 1, C), x], 0)
    out = bias.expand(T, C).clone()
    for j in range(taps):
        out = out + pad[j:j + T] * weight[:, j]
    return out


def state_space_scan(x, B, C, dt, A_log, D):
    """x: [T, H, e], B, C: [T, G, N], dt: [T, H] (after softplus).  Returns y [T, H, e] and the last states."""
    T, H, e = x.shape
    G, N = B.shape[1], B.shape[2]
    S = x.new_zeros(H, N, e)
    ys = []
    for t in range(T):
        y = []
        for h in range(H):
            g = h // (H // G)
            S[h] = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y.append(S[h].T @ C[t, g] + D[h] * x[t, h])
        ys.append(torch.stack(y))
    return torch.stack(ys), S


def mixer_state_space(h, m, w, p, eps):
    T = h.shape[0]
    H, e, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
    inner = H * e
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, e)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y, _ = state_space_scan(x, B, C, dt, w[p + "A_log"], w[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def mixer_parallel(h, m, w, p, eps):
    left = mixer_biased_sink_attention(h, m["left"], w, p + "left.")
    right = mixer_state_space(h, m["right"], w, p + "right.", eps)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2, "parallel": mixer_parallel}


# ---------------------------------------------------------------- feed-forward

def dense_ff(h, mlp, w, p):
    lim = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=lim)
    u = torch.clamp(h @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def expert_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def _closest_call(sorted_scores, k, largest):
    """Gap between the k-th and the (k + 1)-th of scores sorted downwards, as a fraction of ``largest``."""
    if sorted_scores.shape[-1] <= k:
        return torch.full(sorted_scores.shape[:-1], float("inf"), dtype=sorted_scores.dtype)
    gap = sorted_scores[..., k - 1] - sorted_scores[..., k]
    return torch.where(torch.isfinite(gap), gap / largest, torch.full_like(gap, float("inf")))


def route(h, mlp, w, p, margins=None):
    """For every token the chosen outputs of the router and their weights.  ``margins`` [T] is
    lowered to the smallest gap that decided a choice (between groups or between outputs), as a
    fraction of the token's largest score."""
    r = mlp["router"]
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    largest = s.max(-1).values
    gr = r.get("groups")
    if gr and gr["count"] > 1 and gr["keep"] < gr["count"]:
        per = n // gr["count"]
        best = choice.view(-1, gr["count"], per).max(-1).values
        kept = best.topk(gr["keep"], -1).indices
        if margins is not None:
            margins.copy_(torch.minimum(margins, _closest_call(best.sort(-1, descending=True).values, gr["keep"],
                                                               largest).to(margins.dtype)))
        allow = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allow.repeat_interleave(per, 1), float("-inf"))
    chosen = choice.topk(r["top"], -1).indices
    if margins is not None:
        margins.copy_(torch.minimum(margins, _closest_call(choice.sort(-1, descending=True).values, r["top"],
                                                           largest).to(margins.dtype)))
    return chosen, s.gather(1, chosen) * r.get("scale", 1.0)


def moe_ff(h, mlp, w, p, margins=None):
    r = mlp["router"]
    chosen, weight = route(h, mlp, w, p, margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weight[t]):
            if e >= r["experts"]:
                out[t] += c * h[t]
            else:
                out[t] += c * expert_ff(h[t:t + 1], w, "%se%d." % (p, e))[0]
    if mlp.get("shared"):
        out = out + expert_ff(h, w, p + "shared.")
    return out


def feed_forward(h, mlp, w, p, margins=None):
    return dense_ff(h, mlp, w, p) if mlp["kind"] == "dense" else moe_ff(h, mlp, w, p, margins)


# ---------------------------------------------------------------- the model

def run_order(config):
    """(layer, pass number or None, first of its pass) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def forward(tokens, config, w, layers_out=None, margins=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``, a list, takes the residual stream
    after every layer run; ``margins`` [T] the routers' closest calls (see ``route``)."""
    eps = config["norm"]["eps"]
    x0 = embed(tokens, config, w)
    x = x0.clone()
    for i, turn, first in run_order(config):
        if first:
            if turn > 0:
                x = x + x0
            x = x + w["loop.step"][turn]
        layer = config["layers"][i]
        p = "l%d." % i
        h = rms_norm(x, w[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, layer["mixer"], w, p + "mix.", eps)
        x = x + y * w[p + "ls1"] if (p + "ls1") in w else x + y
        if layer.get("mlp"):
            h = rms_norm(x, w[p + "norm2"], eps)
            y = feed_forward(h, layer["mlp"], w, p + "mlp.", margins)
            x = x + y * w[p + "ls2"] if (p + "ls2") in w else x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
