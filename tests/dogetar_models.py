"""Small Dogetar configurations and random weights for the tests.

The configurations differ from one another in every size and option: width and vocabulary
(also odd ones), the order of the three kinds of layer, head counts and groups (one, several
and as many key heads as query heads), key sizes that are and are not multiples of 16, value
sizes equal to the key size and not, partly and fully rotated heads and none, wavelength bands,
windows and blocks shorter and longer than a page and absent, state sizes and group counts of
the state-space branch, one to five taps, dense and routed feed-forwards and none, routers with
and without groups, identity experts and a shared expert, with and without the bigram table,
the loop (from the first layer and from a later one) and the logit cap.
The weights are made here, with torch's generator, and written with the ``safetensors``
library; nothing of the package takes part.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, identity=None, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _attention(heads, kv_heads, dim, vdim, mask, scale):
    m = {"heads": heads, "dim": dim, "scale": scale if scale is not None else 1.5 / math.sqrt(dim)}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if vdim is not None:
        m["vdim"] = vdim
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


def windowed(heads, kv_heads, dim, vdim=None, window=None, rot=None, base=10000.0, bands=None, scale=None, mlp=None):
    m = _attention(heads, kv_heads, dim, vdim, window, scale)
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if bands:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def differential(heads, kv_heads, dim, vdim=None, chunk=None, rot=None, base=10000.0, diff=0.4, scale=None, mlp=None):
    m = _attention(heads, kv_heads, dim, vdim, chunk, scale)
    m["diff"] = diff
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def parallel(left, right, left_scale=None, right_scale=None, mlp=None):
    """left: (heads, kv_heads, dim, vdim, chunk); right: dict of the state-space branch's sizes."""
    m = {"left": _attention(*left, None), "right": right}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return {"type": "parallel", "mixer": m, "mlp": mlp}


CONFIGS: Dict[str, dict] = {
    # starts with the parallel layer; the loop starts at the first layer; a block shorter than two pages of 16;
    # half of a head rotated; wavelength bands that touch all three cases
    "G1": {"architecture": "Dogetar", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
           "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}},
           "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [parallel((4, 2, 16, 8, 24), {"heads": 4, "vdim": 12, "state": 8, "groups": 2, "conv": 3,
                                                   "norm_groups": 1}, 0.7, 1.1,
                               mlp=moe(24, 6, 2, identity=2, groups=(2, 1), scale=1.5, shared=16)),
                      differential(4, 2, 8, 16, chunk=20, rot=4, base=1000.0, diff=0.3, mlp=dense(40, 2.0)),
                      windowed(6, 3, 12, 12, window=13, rot=12, base=500.0, bands=(8.0, 1.0, 4.0, 64.0),
                               mlp=moe(20, 5, 3))]},
    # nothing optional: no bigram, no loop, no cap, no masks, no rotation, absent kv_heads / vdim / groups /
    # identity / shared / scales; a layer without a feed-forward; one tap; top = 1; as many key heads as heads
    "G2": {"architecture": "Dogetar", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
           "layers": [windowed(3, None, 16),
                      differential(2, None, 12, mlp=moe(16, 4, 1, identity=2, groups=(3, 2))),
                      parallel((3, 1, 8, None, None), {"heads": 3, "vdim": 10, "state": 5, "conv": 1, "norm_groups": 3},
                               mlp=dense(24, 0.75))]},
    # sizes that the tensor-core kernels take: heads of 64 with values of 64, experts of multiples of 64, state 64;
    # the loop from a later layer, three passes; a window and blocks longer than a page
    "G3": {"architecture": "Dogetar", "vocab": 512, "width": 256, "norm": {"eps": 2e-5}, "logit_softcap": 30.0,
           "embedding": {"bigram": {"buckets": 257, "mul_prev": 1000003, "mul_cur": 13}},
           "loop": {"start": 1, "stop": 3, "times": 3},
           "layers": [windowed(4, 1, 64, 64, window=40, rot=32, base=50000.0, bands=(4.0, 1.0, 2.0, 32.0),
                               mlp=dense(128, 1.0)),
                      parallel((4, 4, 64, 64, 64), {"heads": 4, "vdim": 64, "state": 64, "groups": 1, "conv": 4,
                                                    "norm_groups": 2}, 0.9, 0.8,
                               mlp=moe(128, 7, 2, identity=1, groups=(4, 2), scale=2.0, shared=64)),
                      differential(4, 2, 32, 64, chunk=64, rot=32, base=50000.0, diff=0.5, mlp=moe(64, 8, 2, shared=128)),
                      differential(2, 1, 64, 128, chunk=48, rot=16, diff=0.2, mlp=dense(192, 3.0))]},
    # odd sizes throughout; three heads to a key head in the differential layer; a block of 7 positions and a
    # window of one; five taps; three groups of the state-space branch; more identity experts than one
    "G4": {"architecture": "Dogetar", "vocab": 131, "width": 72, "norm": {"eps": 3e-6}, "logit_softcap": 9.0,
           "embedding": {"bigram": {"buckets": 13, "mul_prev": 7, "mul_cur": 3}},
           "loop": {"start": 1, "stop": 2, "times": 2},
           "layers": [differential(6, 2, 10, 14, chunk=7, rot=6, base=300.0, diff=0.6, mlp=moe(24, 5, 4, identity=3,
                                                                                           groups=(4, 3), scale=0.5)),
                      parallel((5, 5, 6, 9, 17), {"heads": 6, "vdim": 7, "state": 9, "groups": 3, "conv": 5,
                                                  "norm_groups": 2}, 1.2, 0.6, mlp=moe(40, 3, 2, shared=24)),
                      windowed(2, 1, 20, 4, window=1, rot=20, base=77.0),
                      windowed(4, 2, 6, 10, window=16, rot=2, base=77.0, bands=(2.0, 0.5, 8.0, 16.0), mlp=dense(56, 1.25))]},
}


def get(name: str) -> dict:
    return json.loads(json.dumps(CONFIGS[name]))


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, V = config["width"], config["vocab"]

    def normal(*shape, std):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / math.sqrt(inp))

    def around_one(n):
        return (0.7 + 0.6 * torch.rand(n, generator=g)).to(dtype)

    def between(n, lo, hi):
        return (lo + (hi - lo) * torch.rand(n, generator=g)).to(dtype)

    w = {"embed": normal(V, D, std=1.0), "final.norm": around_one(D), "head": matrix(V, D)}
    bg = (config.get("embedding") or {}).get("bigram")
    if bg:
        w["bigram"] = normal(bg["buckets"] + 1, D, std=0.7)
    if config.get("loop"):
        w["loop.step"] = normal(config["loop"]["times"], D, std=0.3)

    def attention_tensors(p, m, maps):
        H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
        e = m.get("vdim", d)
        w[p + "q"] = matrix(H * maps * d, D)
        w[p + "k"] = matrix(G * maps * d, D)
        w[p + "v"] = matrix(G * e, D)
        w[p + "o"] = matrix(D, H * e)
        return H, G, d, e

    for i, l in enumerate(config["layers"]):
        p = f"l{i}."
        m = l["mixer"]
        w[p + "norm1"] = around_one(D)
        w[p + "ls1"] = between(D, 0.3, 1.0)
        if l["type"] == "attention_2":
            H, G, d, e = attention_tensors(p + "mix.", m, 1)
            w[p + "mix.q.b"] = normal(H * d, std=0.3)
            w[p + "mix.k.b"] = normal(G * d, std=0.3)
            w[p + "mix.v.b"] = normal(G * e, std=0.3)
            w[p + "mix.q.norm"] = around_one(d)
            w[p + "mix.k.norm"] = around_one(d)
        elif l["type"] == "attention":
            H, G, d, e = attention_tensors(p + "mix.", m, 2)
            for name in ("lq1", "lk1", "lq2", "lk2"):
                w[p + "mix." + name] = normal(d, std=0.4)
            w[p + "mix.g"] = matrix(H, D, gain=2.0)
        else:
            H, G, d, e = attention_tensors(p + "mix.left.", m["left"], 1)
            w[p + "mix.left.sink"] = normal(H, std=1.5)
            r = m["right"]
            Hs, es, N, Gs = r["heads"], r["vdim"], r["state"], r.get("groups", 1)
            inner, ch = Hs * es, Hs * es + 2 * Gs * N
            w[p + "mix.right.in"] = matrix(2 * inner + 2 * Gs * N + Hs, D)
            w[p + "mix.right.conv"] = normal(ch, r["conv"], std=0.5)
            w[p + "mix.right.conv.b"] = normal(ch, std=0.2)
            w[p + "mix.right.dt_bias"] = between(Hs, -2.0, 0.5)
            w[p + "mix.right.A_log"] = between(Hs, -2.0, 1.0)
            w[p + "mix.right.D"] = around_one(Hs)
            w[p + "mix.right.norm"] = around_one(inner)
            w[p + "mix.right.o"] = matrix(D, inner)
        mlp = l.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"] = around_one(D)
        w[p + "ls2"] = between(D, 0.3, 1.0)
        if mlp["kind"] == "dense":
            w[p + "mlp.gate"] = matrix(mlp["ff"], D, gain=1.5)
            w[p + "mlp.up"] = matrix(mlp["ff"], D, gain=1.5)
            w[p + "mlp.down"] = matrix(D, mlp["ff"])
            continue
        r = mlp["router"]
        outputs = r["experts"] + r.get("identity", 0)
        w[p + "mlp.router"] = matrix(outputs, D, gain=1.5)
        w[p + "mlp.correction"] = normal(outputs, std=0.05)
        for n in list(range(r["experts"])) + (["shared"] if mlp.get("shared") else []):
            q = f"{p}mlp.e{n}." if n != "shared" else p + "mlp.shared."
            ff = mlp["expert"]["ff"] if n != "shared" else mlp["shared"]["ff"]
            w[q + "gate"] = matrix(ff, D)
            w[q + "up"] = matrix(ff, D)
            w[q + "down"] = matrix(D, ff, gain=2.0)
    return w


def write_model(config: dict, folder: str, seed: int, dtype=torch.bfloat16, weights: Optional[dict] = None) -> str:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    weights = random_weights(config, seed, dtype) if weights is None else weights
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def plain_logits(config: dict, seed: int, requests: Dict[str, List[int]], dtype=torch.float64, stored=torch.bfloat16,
                 weights: Optional[dict] = None, margins: Optional[dict] = None) -> Dict[str, torch.Tensor]:
    """The plain implementation on the weights that ``write_model`` stores.  ``margins``, a dict, takes
    per request how close each position's closest call of a router was (``plain_dogetar.route``)."""
    import plain_dogetar

    w = random_weights(config, seed, stored) if weights is None else weights
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    out = {}
    for rid, ids in requests.items():
        m = None
        if margins is not None:
            m = margins[rid] = torch.full((len(ids),), float("inf"), dtype=torch.float64)
        out[rid] = plain_dogetar.forward(torch.tensor(ids), config, w, margins=m).float()
    return out


def safe_prefix(margins: torch.Tensor, least: float) -> int:
    """How many leading positions of a request have no close call nearer than ``least``; a close
    call's effect reaches later positions, never earlier ones."""
    close = torch.nonzero(margins < least)
    return int(close[0, 0]) if close.numel() else int(margins.numel())


# Below these margins (a gap between two choice scores, as a fraction of the larger score) a run may
# rightly choose otherwise than the plain implementation in 64-bit: bfloat16 rounds the router's input
# to 8 bits, 32-bit runs differ by the order of their sums.
LEAST_MARGIN = {"float32": 1e-4, "bfloat16": 6e-2}


def cut_to_safe(got: Dict[str, torch.Tensor], ref: Dict[str, torch.Tensor], margins: Dict[str, torch.Tensor],
                dtype: str, most_lost: float = 0.6):
    """Both sets of logits cut to each request's positions before its first close call (requests
    with none left are dropped); at most ``most_lost`` of all positions may go that way."""
    a, b, kept, total = {}, {}, 0, 0
    for rid, r in ref.items():
        n = safe_prefix(margins[rid], LEAST_MARGIN[dtype])
        total += r.shape[0]
        kept += n
        assert got[rid].shape == r.shape, f"{rid}: shape {tuple(got[rid].shape)} vs {tuple(r.shape)}"
        if n:
            a[rid], b[rid] = got[rid][:n], r[:n]
    assert kept >= (1.0 - most_lost) * total, f"only {kept} of {total} positions are free of close calls"
    return a, b


def decisive(weights: Dict[str, torch.Tensor], seed: int = 0) -> Dict[str, torch.Tensor]:
    """The same weights with every router's corrections two units apart (in a random order): which outputs a
    token gets is then decided by the corrections alone, so that a run in bfloat16 cannot rightly choose
    otherwise than the plain implementation; the weights of the chosen outputs still come from the scores."""
    g = torch.Generator().manual_seed(seed)
    out = dict(weights)
    for name, t in weights.items():
        if name.endswith(".correction"):
            out[name] = (2.0 * torch.randperm(t.numel(), generator=g).to(torch.float32)).to(t.dtype)
    return out
