"""Pitudra on the GPU against the plain implementation of the design
(tests/plain_pitudra.py): each mechanism's kernels alone -- the norm on a sublayer's
output, the token shift, attention with a window and a sink (keys made to stand out
just inside and just outside the window, at page borders, far back), the latent
rows, the whole-width norm of q and k, the gated recurrence, the router and its
experts -- then whole models through the step function: whole prompts, the last
tokens one by one, portions down to two tokens, mixed batches with reused pages and
slots, long decoding; then greedy generation through the package's entry point and
the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import pitudra_models
import plain_pitudra as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def kernels():
    from chibillm_b200.kernels.ops import CudaKernels
    return CudaKernels(torch.device(DEV))


def close(got, ref, tol, what):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    worst = float((got - ref).abs().max())
    scale = float(ref.abs().max())
    assert worst <= tol * max(scale, 1e-30), f"{what}: max |diff| {worst:.3e} > {tol:.1e} * {scale:.3e}"


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ the norm on a sublayer's output, the token shift
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,n", [(1, 40), (37, 64), (5, 1000), (300, 257)])
def test_norm_of_a_sublayer_output(kernels, dtype, T, n):
    g = torch.Generator().manual_seed(T + n)
    dt = DTYPES[dtype]
    y = torch.randn(T, n, generator=g) * 3 + 1.5
    w, b = (0.5 + torch.rand(n, generator=g)).to(dt), torch.randn(n, generator=g).to(dt)
    x0 = torch.randn(T, n, generator=g)
    ref = plain.layer_norm(y.double(), w.double(), b.double(), 1e-5)
    res = x0.clone().to(DEV)
    out = torch.empty(T, n, dtype=dt, device=DEV)
    kernels.norm_rows(y.to(DEV), w.to(DEV), b.to(DEV), 1e-5, 0.0, True, residual=res, out=out)
    close(res, x0.double() + ref, 2e-6, "x + layer norm(y)")
    assert torch.equal(out, res.to(dt))
    alone = torch.empty(T, n, dtype=torch.float32, device=DEV)
    kernels.norm_rows(y.to(DEV), w.to(DEV), b.to(DEV), 1e-5, 0.0, True, out=alone)
    close(alone, ref, 2e-6, "layer norm alone")
    kernels.norm_rows(y.to(DEV), w.to(DEV), None, 1e-5, 0.0, False, out=alone)
    close(alone, plain.unit_rms(y.double(), 1e-5) * w.double(), 2e-6, "rms norm with a plain weight")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_shift_across_steps_and_slots(kernels, dtype):
    """Two sequences in one step (a portion and a single token), then the other way round: the
    token before a step's first one comes from the sequence's slot, a new sequence starts from
    zeros, and the slot is left with the step's last input in 32-bit."""
    g = torch.Generator().manual_seed(1)
    n, dt = 70, DTYPES[dtype]
    a, b = torch.randn(9, n, generator=g), torch.randn(6, n, generator=g)
    mix = torch.rand(n, generator=g)
    mix[0], mix[1] = 0.0, 1.0
    ref_a, ref_b = plain.token_shift(a.double(), mix.double()), plain.token_shift(b.double(), mix.double())
    state = torch.full((4, n), float("nan"), device=DEV)
    state[3].zero_()                                        # a's slot, b's is 1
    state[1].zero_()
    slots = i32([3, 1])
    steps = [((0, 5), (0, 1)), ((5, 6), (1, 4)), ((6, 9), (4, 6))]
    got_a, got_b = torch.zeros(9, n), torch.zeros(6, n)
    for (a0, a1), (b0, b1) in steps:
        x = torch.cat([a[a0:a1], b[b0:b1]]).to(DEV)
        na, nb = a1 - a0, b1 - b0
        out = torch.empty(na + nb, n, dtype=dt, device=DEV)
        kernels.token_shift(x, mix.to(DEV), state, i32([0, na, na + nb]), i32([0] * na + [1] * nb), slots, out)
        got_a[a0:a1], got_b[b0:b1] = out[:na].float().cpu(), out[na:].float().cpu()
        assert torch.equal(state[3].cpu(), a[a1 - 1]) and torch.equal(state[1].cpu(), b[b1 - 1])
    tol = 1e-6 if dtype == "float32" else 1e-2
    close(got_a, ref_a, tol, "token shift, first sequence")
    close(got_b, ref_b, tol, "token shift, second sequence")
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all()


# ------------------------------------------------------------------ attention with a window and a sink
def run_attention(kernels, q, k, v, sink, scale, window, dtype, page_size, portions):
    """One sequence's rows through the attention kernel in portions.  k [T, G, d] and v [T, G, e]
    (None: the values are the keys, one array) are put into pages in a scrambled order as they
    arrive, the sequence sits on row 1 of the table.  Returns [T, H, e]."""
    dt = DTYPES[dtype]
    T, H, d = q.shape
    G = k.shape[1]
    e = d if v is None else v.shape[2]
    pages = (T + page_size - 1) // page_size + 3
    keys = torch.full((pages, G, page_size, d), float("nan"), dtype=dt, device=DEV)
    values = keys if v is None else torch.full((pages, G, page_size, e), float("nan"), dtype=dt, device=DEV)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(5))
    table = torch.full((2, pages), -1, dtype=torch.int32, device=DEV)
    table[1] = order.to(torch.int32).to(DEV)
    rows = i32([1])
    out_all = torch.zeros(T, H, e)
    for a, b in portions:
        n = b - a
        idx = torch.arange(a, b)
        page, slot = order[idx // page_size].to(DEV), (idx % page_size).to(DEV)
        keys[page, :, slot, :] = k[a:b].to(dt).to(DEV)
        if v is not None:
            values[page, :, slot, :] = v[a:b].to(dt).to(DEV)
        positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
        out = torch.empty(n, H * e, dtype=dt, device=DEV)
        kernels.attention(q[a:b].reshape(n, H * d).to(dt).to(DEV).contiguous(), keys, values, out, table, i32([0, n]),
                          i32([b]), torch.zeros(n, dtype=torch.int32, device=DEV), positions, H, G, d, page_size, scale,
                          window, n, b, n, rows, value_dim=e if e != d else None,
                          sink=None if sink is None else sink.float().to(DEV))
        out_all[a:b] = out.float().cpu().view(n, H, e)
    kernels.check_error_word()
    return out_all


def attention_reference(q, k, v, sink, scale, window):
    T, H, d = q.shape
    G = k.shape[1]
    v = k if v is None else v
    kk, vv = k.double().repeat_interleave(H // G, dim=1), v.double().repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q.double(), kk) * scale
    prob = plain.softmax_with_sink(scores, None if sink is None else sink.double(), plain.window_mask(T, window))
    return torch.einsum("hij,jhe->ihe", prob, vv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e,window", [
    (4, 2, 16, 16, 7), (3, 1, 48, 32, 40), (8, 1, 64, 64, 100), (2, 2, 128, 128, 33), (5, 1, 80, None, 130),
    (2, 1, 40, None, 9), (1, 1, 24, 72, 1), (6, 3, 32, 32, None), (4, 1, 256, None, 150), (2, 1, 272, None, 64), (1, 1, 576, None, 200),
    (3, 1, 96, None, 50), (2, 2, 112, 112, 20), (2, 1, 160, None, 70), (2, 1, 208, None, 31)])
def test_attention_with_a_window_and_a_sink(kernels, dtype, H, G, d, e, window):
    """Head sizes that the tensor-core kernels take (multiples of 16 up to 256 with values as wide
    as keys; 64 and 128: tcgen05 for prompt portions) and that they do not; values tied to the keys
    (e None); with a sink and without: whole, in portions that cut pages and windows, token by token."""
    g = torch.Generator().manual_seed(d + (e or 0))
    T, page_size = 300, 8
    dt = DTYPES[dtype]
    q = torch.randn(T, H, d, generator=g).to(dt)
    k = torch.randn(T, G, d, generator=g).to(dt)
    v = None if e is None else torch.randn(T, G, e, generator=g).to(dt)
    sink = torch.randn(H, generator=g) * 2 + 1.0
    scale = 5.0 / math.sqrt(d)
    tol = 2e-5 if dtype == "float32" else 2e-2
    cuts = [(0, 61), (61, 63), (63, 64), (64, 199), (199, 201), (201, 260)] + [(i, i + 1) for i in range(260, T)]
    for s in (sink, None):
        ref = attention_reference(q, k, v, s, scale, window)
        whole = run_attention(kernels, q, k, v, s, scale, window, dtype, page_size, [(0, T)])
        close(whole, ref, tol, f"attention whole, sink {s is not None}")
        cut_up = run_attention(kernels, q, k, v, s, scale, window, dtype, page_size, cuts)
        close(cut_up, ref, tol, f"attention in portions and single tokens, sink {s is not None}")
    # the sink takes weight: with it the rows are shorter
    with_sink = attention_reference(q, k, v, sink, scale, window)
    assert float((with_sink - ref).abs().max()) > 0.05 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,tied", [(64, False), (80, True), (40, False)])
def test_attention_sees_its_window_and_the_sink(kernels, dtype, d, tied):
    """Keys are made to stand out: the oldest one inside the window (the first position of a
    page), the newest one outside it (the last position of the page before) and one far back.
    With a window the first takes the weight and the others are not seen; without one all
    three share it.  The sink is made as heavy as a marked key: it takes its share and no more.
    In a prompt and for tokens decoded alone, through the split-key kernel's long context."""
    H, G = 2, 1
    T, page_size, window = 1409, 16, 177
    g = torch.Generator().manual_seed(3)
    q = torch.randn(T, H, d, generator=g) * 0.3
    k = torch.randn(T, G, d, generator=g) * 0.3
    v = None if tied else torch.randn(T, G, d, generator=g)
    direction = torch.randn(d, generator=g)
    direction /= direction.norm()
    last = T - 1                                   # the decoded query
    inside, outside, far = last - window + 1, last - window, 37
    assert inside % page_size == 0
    mid = 900                                      # a query inside the prompt: its window's edge is no page border
    for j in (inside, outside, far, mid - window + 1, mid - window):
        k[j] = 8 * direction
    for t in (last, mid):
        q[t] = 8 * direction
    dt = DTYPES[dtype]
    q, k = q.to(dt), k.to(dt)
    v = None if v is None else v.to(dt)
    scale = 0.5                                    # a marked pair scores 32, any other about 0
    sink = torch.tensor([32.0, -5.0])              # head 0: as heavy as one marked key; head 1: nearly nothing
    ref = attention_reference(q, k, v, sink, scale, window)
    vals = (k if v is None else v).double()
    # head 0 of the decoded query: half the marked key inside the window, half nothing
    assert float((ref[last, 0] - vals[inside, 0] / 2).abs().max()) < 0.1 * float(vals[inside, 0].abs().max())
    assert float((ref[last, 1] - vals[inside, 0]).abs().max()) < 0.02 * float(vals[inside, 0].abs().max())
    tol = 2e-5 if dtype == "float32" else 2e-2
    cuts = [(0, mid - 3), (mid - 3, mid + 2), (mid + 2, last - 1), (last - 1, last), (last, T)]
    got = run_attention(kernels, q, k, v, sink, scale, window, dtype, page_size, cuts)
    for t, what in ((last, "decoded token"), (mid, "inside a prompt portion"), (last - 1, "decoded token before")):
        close(got[t], ref[t], tol, f"marked keys, {what}")
    close(got, ref, tol, "marked keys, all rows")
    # without a window the far key and the one just outside are seen again
    free = attention_reference(q, k, v, sink, scale, None)
    got = run_attention(kernels, q, k, v, sink, scale, None, dtype, page_size, [(0, last), (last, T)])
    close(got, free, tol, "marked keys, no window")
    assert float((free[last] - ref[last]).abs().max()) > 0.1


# ------------------------------------------------------------------ what the two kinds of attention put into the cache
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("q_rank,kv_rank,rot", [(40, 24, 8), (96, 48, 16), (17, 130, 4), (256, 192, 64)])
def test_latent_rows(kernels, dtype, q_rank, kv_rank, rot):
    """c_q | c | k_rot -> the normalised query latent, and the cache row k_rot (rotated) | c
    (normalised) at the token's place; positions that start in the middle of a page."""
    g = torch.Generator().manual_seed(q_rank)
    dt = DTYPES[dtype]
    T, page_size, first, eps, base = 29, 8, 13, 1e-5, 1000.0
    proj = (torch.randn(T, q_rank + kv_rank + rot, generator=g) * 2).to(dt)
    qn, kn = 0.5 + torch.rand(q_rank, generator=g), 0.5 + torch.rand(kv_rank, generator=g)
    pos = torch.arange(first, first + T)
    ref_cq = plain.unit_rms(proj[:, :q_rank].double(), eps) * qn.double()
    ref_c = plain.unit_rms(proj[:, q_rank:q_rank + kv_rank].double(), eps) * kn.double()
    ref_k = plain.rotate(proj[:, None, q_rank + kv_rank:].double(), pos, base, rot)[:, 0]
    pages = (first + T + page_size - 1) // page_size + 2
    cache = torch.full((pages, 1, page_size, rot + kv_rank), float("nan"), dtype=dt, device=DEV)
    order = torch.randperm(pages, generator=g)
    table = torch.full((3, pages), -1, dtype=torch.int32, device=DEV)
    table[2] = order.to(torch.int32).to(DEV)
    inv_freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    cq = torch.empty(T, q_rank, dtype=dt, device=DEV)
    kernels.latent_prepare(proj.to(DEV), cq, cache, qn.to(DEV), kn.to(DEV), eps, inv_freq, q_rank, kv_rank, rot,
                           pos.to(torch.int32).to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), table, page_size,
                           i32([2]))
    held = cache[order[pos // page_size].to(DEV), 0, (pos % page_size).to(DEV)].float().cpu()
    tol = 2e-6 if dtype == "float32" else 1e-2
    close(cq, ref_cq, tol, "query latent")
    close(held[:, rot:], ref_c, tol, "cached latent")
    close(held[:, :rot], ref_k, tol, "cached rotated key part")
    # a layer without a cache of its own: the query latent only
    cq2 = torch.empty(T, q_rank, dtype=dt, device=DEV)
    kernels.latent_prepare(proj[:, :q_rank].contiguous().to(DEV), cq2, None, qn.to(DEV), None, eps, inv_freq, q_rank,
                           kv_rank, rot, pos.to(torch.int32).to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV),
                           None, page_size, i32([2]))
    assert torch.equal(cq2, cq)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e", [(4, 2, 16, 8), (8, 1, 64, 64), (3, 3, 24, 40), (1, 1, 130, 6)])
def test_biases_and_the_norm_over_all_heads(kernels, dtype, H, G, d, e):
    g = torch.Generator().manual_seed(H * d)
    dt = DTYPES[dtype]
    T, page_size, first, eps = 21, 4, 6, 1e-5
    width = H * d + G * d + G * e
    proj = (torch.randn(T, width + 5, generator=g) * 2).to(dt)          # more columns follow (the gate's)
    bias = torch.randn(width, generator=g)
    qn, kn = 0.5 + torch.rand(H * d, generator=g), 0.5 + torch.rand(G * d, generator=g)
    pos = torch.arange(first, first + T)
    x = proj[:, :width].double() + bias.double()
    ref_q = plain.unit_rms(x[:, :H * d], eps) * qn.double()
    ref_k = (plain.unit_rms(x[:, H * d:H * d + G * d], eps) * kn.double()).view(T, G, d)
    ref_v = x[:, H * d + G * d:].view(T, G, e)
    pages = (first + T + page_size - 1) // page_size + 2
    keys = torch.full((pages, G, page_size, d), float("nan"), dtype=dt, device=DEV)
    values = torch.full((pages, G, page_size, e), float("nan"), dtype=dt, device=DEV)
    order = torch.randperm(pages, generator=g)
    table = order.to(torch.int32).to(DEV).view(1, pages)
    q = torch.empty(T, H * d, dtype=dt, device=DEV)
    kernels.qkv_bias_norm_append(proj.to(DEV), q, keys, values, bias.to(DEV), qn.to(DEV), kn.to(DEV), eps, None, 0,
                                 pos.to(torch.int32).to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), table,
                                 H, G, d, e, page_size, None)
    page, slot = order[pos // page_size].to(DEV), (pos % page_size).to(DEV)
    tol = 2e-6 if dtype == "float32" else 1e-2
    close(q, ref_q, tol, "q")
    close(keys[page, :, slot], ref_k, tol, "cached keys")
    close(values[page, :, slot], ref_v, tol, "cached values")
    gate = (torch.randn(T, H * e, generator=g) * 3).to(dt)
    att = torch.randn(T, H * e, generator=g).to(dt)
    out = att.clone().to(DEV)
    kernels.sigmoid_gate(out, gate.to(DEV))
    close(out, att.double() * torch.sigmoid(gate.double()), tol, "output gate")


# ------------------------------------------------------------------ the gated recurrence
def recurrence_reference(proj, bias, floor, H, d, e):
    """proj [T, 2 H d + H e] -> o [T, H, e] and the last state [H, d, e], in 64-bit."""
    T = proj.shape[0]
    kw = H * d
    q = plain.silu(proj[:, :kw].double()).view(T, H, d)
    f = (floor.double() + (1 - floor.double()) * torch.sigmoid(proj[:, kw:2 * kw].double() + bias.double())).view(T, H, d)
    v = proj[:, 2 * kw:].double().view(T, H, e)
    state = torch.zeros(H, d, e, dtype=torch.float64)
    out = torch.zeros(T, H, e, dtype=torch.float64)
    for t in range(T):
        state = f[t][:, :, None] * state + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", state, q[t])
    return out, state


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d,e", [(2, 24, 16), (1, 130, 8), (4, 32, 64), (3, 64, 128), (6, 48, 32), (2, 200, 20), (1, 7, 5)])
def test_gated_recurrence(kernels, dtype, H, d, e):
    """A long sequence in portions of every kind beside a second sequence that is decoded token by
    token; slots that were used before (their state set to zero by hand, as the manager does) and
    channels whose gate is 1 (they keep their state) or 0 (they take the new value whole)."""
    g = torch.Generator().manual_seed(d + e)
    dt = DTYPES[dtype]
    Ta, Tb = 700, 40
    kw = H * d
    width = 2 * kw + H * e
    pa = torch.randn(Ta, width, generator=g).to(dt)
    pb = torch.randn(Tb, width, generator=g).to(dt)
    bias = torch.randn(kw, generator=g)
    floor = 0.9 * torch.rand(kw, generator=g)
    floor[0] = 1.0                                 # this channel never forgets and never writes
    bias[1], floor[1] = -80.0, 0.0                 # this one holds the last value only
    ref_a, state_a = recurrence_reference(pa, bias, floor, H, d, e)
    ref_b, state_b = recurrence_reference(pb, bias, floor, H, d, e)
    state = torch.full((3, H, d, e), float("nan"), device=DEV)
    state[2].zero_()
    state[0].zero_()
    slots = i32([2, 0])
    cuts_a = [0, 300, 302, 303, 431, 433, 500]
    cuts_a += list(range(cuts_a[-1] + 5, Ta + 1, 5))
    got_a, got_b = torch.zeros(Ta, H, e), torch.zeros(Tb, H, e)
    b_at = 0
    for i in range(len(cuts_a) - 1):
        a0, a1 = cuts_a[i], cuts_a[i + 1]
        nb = 1 if b_at < Tb else 0
        proj = torch.cat([pa[a0:a1], pb[b_at:b_at + nb]]).to(DEV)
        n = proj.shape[0]
        qfv = torch.empty(n, width, dtype=torch.float32, device=DEV)
        kernels.recurrence_gates(proj, bias.to(DEV), floor.to(DEV), qfv, kw)
        o = torch.empty(n, H * e, dtype=torch.float32, device=DEV)
        q_start = i32([0, a1 - a0, n]) if nb else i32([0, a1 - a0])
        kernels.gated_recurrence(qfv, state, o, q_start, slots[:2 if nb else 1], H, d, e, a1 - a0)
        got_a[a0:a1] = o[:a1 - a0].cpu().view(-1, H, e)
        if nb:
            got_b[b_at] = o[a1 - a0:].cpu().view(H, e)
            b_at += 1
    assert b_at == Tb
    # the reference starts from the rounded inputs too; the recurrence itself is 32-bit in both types
    close(got_a, ref_a, 2e-5, "recurrence, portions")
    close(got_b, ref_b, 2e-5, "recurrence, token by token beside the portions")
    close(state[2], state_a, 2e-5, "state after the long sequence")
    close(state[0], state_b, 2e-5, "state after the decoded sequence")
    assert torch.isnan(state[1]).all()
    assert float(state_a[0, 0].abs().max()) == 0.0 and torch.equal(state[2, 0, 0].cpu(), torch.zeros(e))
    close(state[2, 0, 1], pa[-1, 2 * kw:2 * kw + e].double(), 1e-6, "a channel that holds the last value")


# ------------------------------------------------------------------ the router and its experts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,F,E,top", [(1, 64, 40, 5, 2), (9, 96, 24, 3, 3), (300, 80, 100, 7, 1), (700, 128, 64, 4, 2),
                                         (33, 72, 130, 12, 5), (3, 96, 32, 6, 2), (1000, 160, 96, 5, 3),
                                         (130, 256, 224, 3, 1), (70, 192, 128, 40, 6), (5, 256, 320, 9, 3),
                                         (2048, 256, 192, 8, 2), (1, 128, 64, 4, 4), (64, 352, 96, 14, 3)])
def test_router_and_experts(kernels, dtype, T, D, F, E, top):
    """The router's choice (largest logits first, softmax over the chosen ones) and
    down(relu(up x)^2) of the chosen experts: few tokens, many, sizes that end inside a tile,
    experts that nobody uses.  bfloat16 with sizes that are multiples of 32 runs on the tensor
    cores (multiples of 64: tcgen05, and once more with that switched off: mma.sync)."""
    g = torch.Generator().manual_seed(T + E)
    dt = DTYPES[dtype]
    x = torch.randn(T, D, generator=g).to(dt)
    x[:, 0] = 1.0
    w = {"m.router": (torch.randn(E, D, generator=g) * 4 / math.sqrt(D)).to(dt)}
    if E > 4:
        w["m.router"][E - 1] = 0
        w["m.router"][E - 1, 0] = -100.0                                    # an expert that nobody chooses
    for n in range(E):
        w[f"m.e{n}.up"] = (torch.randn(F, D, generator=g) / math.sqrt(D)).to(dt)
        w[f"m.e{n}.down"] = (torch.randn(D, F, generator=g) / math.sqrt(F)).to(dt)
    logits = (x.double() @ w["m.router"].double().T).float()
    best, order = torch.topk(logits.double(), top, dim=-1)
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    share = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.router_top(logits.to(DEV), chosen, share)
    assert torch.equal(chosen.cpu().long(), order), "the chosen experts, largest logit first"
    close(share, torch.softmax(best, dim=-1), 1e-6, "shares")
    ref = plain.routed_experts({n: t.double() for n, t in w.items()}, "m.", {"router": {"experts": E, "top": top}},
                               x.double())
    up = torch.stack([w[f"m.e{n}.up"] for n in range(E)]).to(DEV)
    down = torch.stack([w[f"m.e{n}.down"] for n in range(E)]).to(DEV)
    start = torch.randn(T, D, generator=g)
    route = torch.empty(kernels.route_words(T * top, E), dtype=torch.int32, device=DEV)
    act = torch.empty(T * top, F, dtype=dt, device=DEV)
    y = torch.empty(T * top, D, dtype=torch.float32, device=DEV)
    sorted_x = torch.empty(T * top, D, dtype=dt, device=DEV)
    fast = kernels.expert_tensor_cores(dt, D, F)
    for tcgen05 in ((True, False) if fast else (True,)):
        kernels.use_tcgen05_experts = tcgen05
        before = kernels.tensor_core_calls
        try:
            acc = start.clone().to(DEV)
            act.fill_(float("nan"))
            y.fill_(float("nan"))
            kernels.chosen_experts(x.to(DEV), chosen, share, up, down, acc, route, act, y, "relu2", sorted_x)
            kernels.check_error_word()
        finally:
            kernels.use_tcgen05_experts = True
        assert (kernels.tensor_core_calls > before) == fast
        close(acc.cpu() - start, ref, 2e-5 if dtype == "float32" else 2e-2, f"experts (tcgen05 {tcgen05})")


def test_router_ties_go_to_the_lower_number(kernels):
    logits = torch.tensor([[1.0, 3.0, 3.0, -1.0, 3.0], [0.0, 0.0, 0.0, 0.0, 0.0]], device=DEV)
    chosen = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    share = torch.empty(2, 2, dtype=torch.float32, device=DEV)
    kernels.router_top(logits, chosen, share)
    assert chosen.tolist() == [[1, 2], [0, 1]] and share.tolist() == [[0.5, 0.5], [0.5, 0.5]]


# ------------------------------------------------------------------ whole models
# |engine - plain| as a fraction of the request's largest |plain logit|.  32-bit: the limit of the
# package's other designs.  bfloat16: every sublayer's output is normalised before it joins the
# residual, so the rounding of a small output weighs as much as that of a large one, and more than in
# the other designs; the limit is about one and a half times the worst value that this file measures
# on a B200 (5.0e-2; the run prints them all).  Two of the design's steps decide by a comparison: the
# router's choice, and the sign that alone is left of the recurrence's output at a sequence's first
# token.  Where such a call is closer than rounding (``LEAST_MARGIN``) a run may rightly decide the
# other way, and its effect reaches every later position; requests are compared up to there.  With 8
# bits of mantissa that is a few positions in a hundred, so the bfloat16 runs use the same models with
# every expert chosen by every token (``all_experts``: the weights are the same); the router's choice
# in bfloat16 is covered above, kernel by kernel, from given logits.
TOL = {"float32": helpers.TOL["float32"], "bfloat16": 8e-2}


def model_for(config, dtype):
    return pitudra_models.all_experts(config) if dtype == "bfloat16" else config


def make_runner(folder, dtype, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests)
    runner.storage.poison()
    return runner


def compare(got, ref, margins, dtype, what, tol=None):
    a, b = pitudra_models.cut_to_safe(got, ref, margins, dtype)
    helpers.assert_logits_close(a, b, TOL[dtype] if tol is None else tol, what)


ALONE = {
    "latent": pitudra_models.latent(4, 32, 16, 32, 64, 48, window=70, base=50000.0),
    "latent, no window": pitudra_models.latent(2, 16, 8, 24, 24, 40),
    "recurrent": pitudra_models.recurrent(3, 40, 24),
    "attention": pitudra_models.attention(4, 2, 32, vdim=32, window=50),
    "attention, other value size": pitudra_models.attention(6, 3, 24, vdim=40, window=37),
    "experts": pitudra_models.recurrent(1, 16, 16, mlp=pitudra_models.moe(64, 6, 2)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(ALONE))
def test_one_layer_alone(tmp_path, kind, dtype):
    """A model of one layer (with and without the token input): prompt against token by token."""
    for side in (None, 10):
        cfg = {"architecture": "Pitudra", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "layers": [ALONE[kind]]}
        if side:
            cfg["token_side"] = {"dim": side}
        cfg = model_for(cfg, dtype)
        folder = pitudra_models.write_model(cfg, str(tmp_path / f"one_{side}"), seed=8)
        reqs = helpers.random_requests(cfg["vocab"], [3, 150], seed=3)
        margins = {}
        ref = pitudra_models.plain_logits(cfg, 8, reqs, margins=margins)
        runner = make_runner(folder, dtype, 8, 192)
        for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 90), "decoded"),
                            (helpers.trace_portions(reqs, seed=1), "portions")):
            got = helpers.run_trace(runner, trace)
            compare(got, ref, margins, dtype, f"pitudra one layer ({kind}) {dtype} {what}")
        runner.runtime.kernels.check_error_word()


CASES = {
    # name: (page size, request lengths, lengths of the mixed run)
    "P1": (4, [1, 33, 130, 260], [50, 100, 30, 128, 64, 90, 17]),
    "P2": (16, [2, 70, 131, 300], [1, 200, 33, 250, 64, 129, 7]),
    "P3": (16, [5, 129, 260, 400], [400, 31, 129, 64, 350, 3, 222]),
    "P4": (8, [3, 64, 129, 190], [150, 20, 65, 2, 180, 99, 40]),
    "P5": (16, [4, 66, 140, 300], [300, 20, 131, 64, 150, 2, 90]),
    "P6": (16, [3, 65, 150, 290], [290, 16, 130, 64, 170, 2, 49]),
}
SEED = 21


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("pitudra")
    return {(name, dtype): pitudra_models.write_model(model_for(pitudra_models.get(name), dtype),
                                                      str(root / f"{name}_{dtype}"), seed=SEED)
            for name in CASES for dtype in DTYPES}


@pytest.fixture(scope="module")
def expected():
    out = {}
    for name, (_, lengths, mixed_lengths) in CASES.items():
        for dtype in DTYPES:
            cfg = model_for(pitudra_models.get(name), dtype)
            reqs = helpers.random_requests(cfg["vocab"], lengths, seed=100)
            mixed = helpers.random_requests(cfg["vocab"], mixed_lengths, seed=200)
            m1, m2 = {}, {}
            out[name, dtype] = (reqs, pitudra_models.plain_logits(cfg, SEED, reqs, margins=m1), m1,
                                mixed, pitudra_models.plain_logits(cfg, SEED, mixed, margins=m2), m2)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(CASES))
def test_cutting_and_batching(folders, expected, case, dtype):
    page_size, lengths, _ = CASES[case]
    reqs, ref, margins, mixed_reqs, mixed_ref, mixed_margins = expected[case, dtype]
    runner = make_runner(folders[case, dtype], dtype, page_size, pool_tokens=helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"),
                        (helpers.trace_last_decoded(reqs, 32), "last 32 decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        compare(got, ref, margins, dtype, f"pitudra {case} {dtype} {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    runner.runtime.kernels.check_error_word()
    pool = 640 if sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > 640 else 384
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are used again
    runner2 = make_runner(folders[case, dtype], dtype, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    compare(got, mixed_ref, mixed_margins, dtype, f"pitudra {case} {dtype} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_against_each_request_alone(folders, dtype):
    """Four unequal requests in the same steps against each in steps of its own, both against the
    plain implementation."""
    cfg = model_for(pitudra_models.get("P3"), dtype)
    reqs = helpers.random_requests(cfg["vocab"], [90, 7, 140, 33], seed=17)
    margins = {}
    ref = pitudra_models.plain_logits(cfg, SEED, reqs, margins=margins)
    runner = make_runner(folders["P3", dtype], dtype, 16, 512)
    alone = helpers.run_trace(runner, helpers.trace_portions(reqs, seed=3))
    compare(alone, ref, margins, dtype, f"pitudra P3 {dtype} each alone")
    steps, pos = [], {r: 0 for r in reqs}
    sizes = {"r0": 13, "r1": 1, "r2": 40, "r3": 2}
    while any(pos[r] < len(ids) for r, ids in reqs.items()):
        entries, end = [], []
        for r, ids in reqs.items():
            if pos[r] < len(ids):
                n = min(sizes[r], len(ids) - pos[r])
                entries.append({"id": r, "tokens": ids[pos[r]:pos[r] + n], "want": list(range(n))})
                pos[r] += n
                if pos[r] == len(ids):
                    end.append(r)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    together = helpers.run_trace(runner, steps)
    compare(together, ref, margins, dtype, f"pitudra P3 {dtype} together")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """Three tokens of prompt, then 300 tokens one by one (captured steps replayed): windows of
    20, 13 and 33 positions pass over decoded tokens many times, the recurrent state is carried
    300 times."""
    cfg = model_for(pitudra_models.get("P1"), dtype)
    margins = {}
    for seed in range(9, 20):                       # a request whose first token's sign is no close call
        reqs = helpers.random_requests(cfg["vocab"], [303], seed=seed)
        ref = pitudra_models.plain_logits(cfg, SEED, reqs, margins=margins)
        if pitudra_models.safe_prefix(margins["r0"], pitudra_models.LEAST_MARGIN[dtype]) > 290:
            break
    runner = make_runner(folders["P1", dtype], dtype, 4, 320)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 300))
    compare(got, ref, margins, dtype, f"pitudra P1 {dtype} long decoding")
    assert runner.graph_replays > 200


def test_greedy_generation_through_the_entry_point(folders):
    """``LLM.generate`` (scheduler, sampler, portions of 16 tokens, three requests at a
    time): every generated token is the plain implementation's best one, wherever that
    leads by more than the rounding of a 32-bit run."""
    from chibillm_b200 import LLM
    cfg = pitudra_models.get("P3")
    prompts = list(helpers.random_requests(cfg["vocab"], [5, 40, 23, 61], seed=12).values())
    llm = LLM(folders["P3", "float32"], dtype="float32", context_length=128, max_sequences=3, max_batch_tokens=48,
              prefill_chunk_tokens=16, page_size=16)
    outs = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, new in zip(prompts, outs):
        assert len(new) == 12
        ref = pitudra_models.plain_logits(cfg, SEED, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok, f"token {i} of a prompt of {len(prompt)}"


def test_trace_program(folders, tmp_path):
    """bin/trace_run on a Pitudra folder: portions, single tokens, two live requests."""
    a_len, b_len = 40, 21
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("float32", "bfloat16"):
        cfg = model_for(pitudra_models.get("P4"), dtype)
        reqs = helpers.random_requests(cfg["vocab"], [a_len, b_len], seed=5)
        margins = {}
        ref = pitudra_models.plain_logits(cfg, SEED, reqs, margins=margins)
        safe = {r: pitudra_models.safe_prefix(margins[r], pitudra_models.LEAST_MARGIN[dtype]) for r in reqs}
        a, b = reqs["r0"], reqs["r1"]
        steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
                 {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]},
                                         {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
                 {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0, 1]},
                                         {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "b"]}]
        want = [[("r0", 0), ("r0", 29)], [("r0", 30), ("r1", 18)], [("r1", 19), ("r1", 20), ("r0", 39)]]
        out_dir = str(tmp_path / dtype)
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model",
                               folders["P4", dtype], "--dtype", dtype, "--out", out_dir, "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        compared = 0
        for i, rows in enumerate(want):
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(len(rows), -1))
            for j, (r, pos) in enumerate(rows):
                if pos < safe[r]:
                    compared += 1
                    scale = float(ref[r].abs().max())
                    assert float((got[j] - ref[r][pos]).abs().max()) <= TOL[dtype] * scale, (dtype, i, r, pos)
        assert compared >= 5


def test_random_weights_made_on_the_device(tmp_path):
    """``ModelRunner.from_random`` makes on the device the values that ``write_random_model``
    stores: both give the same logits."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    cfg = pitudra_models.get("P4")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=6)
    ids = helpers.random_requests(cfg["vocab"], [50], seed=2)["r0"]
    a = ModelRunner.from_folder(folder, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    b = ModelRunner.from_random(cfg, seed=6, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    la = a.step([StepEntry("x", ids, list(range(50)))]).clone()
    lb = b.step([StepEntry("x", ids, list(range(50)))]).clone()
    assert torch.equal(la, lb)
