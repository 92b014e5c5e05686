"""Small Pitudra configurations and random weights for the tests.

The configurations differ from one another in every size and option: width and
vocabulary (also odd ones), the order and number of the three kinds of layer,
head counts and groups, key sizes that are and are not multiples of 16, value
sizes equal to the key size and not, latents smaller and larger than a head,
rotated parts of 4 to 16 features, windows from one position to longer than any
test prompt and none at all, readers of another layer's latents with a window
shorter and longer than their source's, layers without a feed-forward, one to
three choices out of 3 to 9 experts, with and without the token input.
The scales and the weights' sizes keep attention scores and router logits within a few units, as a
trained model's are: scores of 15 or more make single rows of a bfloat16 run depend on the rounding
of one score (the tests of the kernels alone use such scores on purpose, in both types).
The weights are made here, with torch's generator, and written with the
``safetensors`` library; nothing of the package takes part.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window=None, base=10000.0, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else 0.5 / math.sqrt(dim + rot_dim)}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def recurrent(heads, dim, vdim, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim=None, window=None, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim,
         "scale": scale if scale is not None else 1.5 / math.sqrt(dim)}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


CONFIGS: Dict[str, dict] = {
    # all three kinds; the last layer reads the first one's latents with a LONGER window and other heads
    "P1": {"architecture": "Pitudra", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 12},
           "layers": [latent(3, 16, 8, 24, 40, 24, window=20, base=1000.0, mlp=moe(40, 5, 2)),
                      recurrent(2, 24, 16, mlp=moe(24, 3, 3)),
                      attention(4, 2, 16, vdim=8, window=13, mlp=moe(32, 4, 1)),
                      latent(2, 8, 8, 16, 24, 24, window=33, base=1000.0, kv_from=0, mlp=moe(40, 5, 2))]},
    # no token input, no windows at all, a layer without a feed-forward, as many key heads as query heads
    "P2": {"architecture": "Pitudra", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
           "layers": [recurrent(3, 8, 8, mlp=moe(16, 3, 1)),
                      attention(2, 2, 24),
                      latent(2, 24, 4, 8, 16, 44, mlp=moe(20, 4, 2))]},
    # sizes that the tensor-core kernels take: key rows of 64 features, heads of 64, experts of multiples of 64;
    # a reader right after its source with a SHORTER window; windows shorter and longer than a page
    "P3": {"architecture": "Pitudra", "vocab": 512, "width": 256, "norm": {"eps": 2e-5}, "token_side": {"dim": 16},
           "layers": [attention(4, 1, 64, window=40, mlp=moe(64, 8, 2)),
                      latent(4, 32, 16, 32, 64, 48, window=70, base=50000.0, mlp=moe(128, 8, 2)),
                      latent(2, 64, 16, 64, 32, 48, window=9, base=50000.0, kv_from=1, mlp=moe(64, 6, 3)),
                      recurrent(4, 32, 64, mlp=moe(64, 8, 2))]},
    # sizes that are no power of two anywhere; a window shorter than a page; seven experts, three choices
    "P4": {"architecture": "Pitudra", "vocab": 257, "width": 160, "norm": {"eps": 3e-6}, "token_side": {"dim": 11},
           "layers": [recurrent(3, 40, 24, mlp=moe(56, 7, 3)),
                      latent(5, 12, 6, 20, 36, 26, window=5, base=300.0, mlp=moe(24, 9, 2)),
                      attention(6, 3, 24, vdim=40, window=37)]},
    # one head everywhere; a window of one position (a token sees only itself and the sink); a recurrent
    # head of 130 key channels
    "P5": {"architecture": "Pitudra", "vocab": 89, "width": 40, "norm": {"eps": 1e-5}, "token_side": {"dim": 14},
           "layers": [recurrent(1, 130, 8, mlp=moe(16, 3, 2)),
                      attention(1, 1, 40, vdim=8, window=1),
                      latent(1, 8, 16, 8, 8, 16, window=64, mlp=moe(16, 3, 2))]},
    # odd sizes throughout: a cache row of 33 numbers, heads of 20 and 12, a recurrent head of 7 x 5; plain
    # attention first; two recurrent layers in a row; two readers of one source; a window of exactly one
    # page of 16 and one of a page and a position; a single expert
    "P6": {"architecture": "Pitudra", "vocab": 131, "width": 72, "norm": {"eps": 1e-5}, "token_side": {"dim": 13},
           "layers": [attention(6, 2, 20, vdim=12, window=16, mlp=moe(40, 6, 2)),
                      latent(3, 10, 6, 14, 22, 27, window=17, base=777.0, mlp=moe(24, 1, 1)),
                      recurrent(5, 7, 5, mlp=moe(8, 2, 2)),
                      recurrent(2, 33, 18),
                      latent(2, 6, 6, 9, 11, 27, window=16, base=777.0, kv_from=1, mlp=moe(40, 6, 5)),
                      latent(4, 4, 6, 5, 30, 27, base=777.0, kv_from=1)]},
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

    layers = config["layers"]
    w = {"embed": normal(V, D, std=1.0), "final.norm": around_one(D), "final.norm.b": normal(D, std=0.1),
         "head": matrix(V, D)}
    side = (config.get("token_side") or {}).get("dim")
    if side:
        w["side.embed"] = normal(V, len(layers) * side, std=1.0)
    for i, l in enumerate(layers):
        p = f"l{i}."
        m = l["mixer"]
        H, d, e = m["heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = around_one(D)
        w[p + "norm1.b"] = normal(D, std=0.1)
        w[p + "shift"] = torch.rand(D, generator=g).to(dtype)
        if l["type"] == "latent_attention":
            r, c, qr = m["rot_dim"], m["kv_rank"], m["q_rank"]
            w[p + "mix.dq"] = matrix(qr, D)
            w[p + "mix.dq.norm"] = around_one(qr)
            w[p + "mix.uq"] = matrix(H * (d + r), qr, gain=2.0)
            if "kv_from" not in m:
                w[p + "mix.dkv"] = matrix(c + r, D, gain=2.0)
                w[p + "mix.dkv.norm"] = around_one(c)
            w[p + "mix.uk"] = matrix(H * d, c, gain=2.0)
            w[p + "mix.uv"] = matrix(H * e, c)
            w[p + "mix.sink"] = normal(H, std=1.5)
            w[p + "mix.o"] = matrix(D, H * e)
        elif l["type"] == "hgrn2":
            w[p + "mix.q"] = matrix(H * d, D)
            w[p + "mix.f"] = matrix(H * d, D, gain=2.0)
            w[p + "mix.f.b"] = normal(H * d, std=1.0)
            w[p + "mix.lower"] = (0.9 * torch.rand(H * d, generator=g)).to(dtype)
            w[p + "mix.v"] = matrix(H * e, D)
            w[p + "mix.norm"] = around_one(e)
            w[p + "mix.o"] = matrix(D, H * e)
        else:
            G = m["kv_heads"]
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * e)):
                w[p + "mix." + name] = matrix(rows, D)
                w[p + "mix." + name + ".b"] = normal(rows, std=0.3)
            w[p + "mix.q.norm"] = around_one(H * d)
            w[p + "mix.k.norm"] = around_one(G * d)
            w[p + "mix.sink"] = normal(H, std=1.5)
            w[p + "mix.g"] = matrix(H * e, D, gain=2.0)
            w[p + "mix.o"] = matrix(D, H * e)
        mlp = l["mlp"]
        if mlp is not None:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            w[p + "norm2"] = around_one(D)
            w[p + "norm2.b"] = normal(D, std=0.1)
            w[p + "mlp.router"] = matrix(E, D, gain=1.5)
            for n in range(E):
                w[f"{p}mlp.e{n}.up"] = matrix(ff, D)
                w[f"{p}mlp.e{n}.down"] = matrix(D, ff, gain=2.0)
        if side:
            w[p + "side.gate"] = matrix(side, D)
            w[p + "side.proj"] = matrix(D, side)
            w[p + "side.norm"] = (0.5 + torch.rand(D, generator=g)).to(dtype)
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
    """The plain implementation on the weights that ``write_model`` stores.  ``margins``, a dict,
    takes per request how close each position's closest call was (see ``plain_pitudra.forward``)."""
    import plain_pitudra

    w = random_weights(config, seed, stored) if weights is None else weights
    out = {}
    for rid, ids in requests.items():
        m = None
        if margins is not None:
            m = margins[rid] = torch.full((len(ids),), float("inf"), dtype=torch.float64)
        out[rid] = plain_pitudra.forward(config, w, ids, dtype, margins=m).float()
    return out


def all_experts(config: dict) -> dict:
    """The same model with every expert chosen by every token: nothing is decided by a comparison
    of router logits, so that a run in bfloat16 cannot rightly choose other experts than the
    plain implementation (the weights do not depend on ``top``)."""
    cfg = json.loads(json.dumps(config))
    for l in cfg["layers"]:
        if l.get("mlp") is not None:
            l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return cfg


def safe_prefix(margins: torch.Tensor, least: float) -> int:
    """How many leading positions of a request have no close call nearer than ``least``; a close
    call's effect reaches later positions, never earlier ones."""
    close = torch.nonzero(margins < least)
    return int(close[0, 0]) if close.numel() else int(margins.numel())


# Below these margins a run may rightly decide otherwise than the plain implementation in 64-bit:
# bfloat16 rounds the router's input to 8 bits, 32-bit runs differ by the order of their sums.
LEAST_MARGIN = {"float32": 1e-5, "bfloat16": 2e-2}


def cut_to_safe(got: Dict[str, torch.Tensor], ref: Dict[str, torch.Tensor], margins: Dict[str, torch.Tensor],
                dtype: str, most_lost: float = 0.4):
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
