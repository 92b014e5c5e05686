"""Dogetar on the GPU against the plain implementation of the design (tests/plain_dogetar.py): each
mechanism's kernels alone -- heads with biases, norms and rotation; attention with score maps that share
their values, a bias linear in the distance, a sink, windows and blocks (keys made to stand out just inside
and just outside, at page borders, far back, in prompts and for tokens decoded alone); the joining of two
maps; the convolution and the state-space scan over portions; the gated norm in parts; the clamped gate;
the router with groups and the experts with identity and shared ones; the bigram table's kept token; the
scaled sum with its norm -- then one layer of each kind alone and whole models through the step function:
whole prompts, the last tokens one by one, portions down to two tokens, mixed batches with reused pages and
slots, long decoding; then greedy generation through the package's entry point and the trace program."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dogetar_models
import helpers
import plain_dogetar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 2e-5, "bfloat16": 2e-2}


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


def rounded(t, dtype):
    return t.to(DTYPES[dtype]).double()


# ------------------------------------------------------------------ attention through pages
def run_attention(kernels, q, k, v, dtype, page_size, portions, scale, window=None, chunk=None, sink=None,
                  slopes=None, kv_share=1, float_out=False, bias=None, norms=None, eps=0.0, inv_freq=None, rot=0):
    """q [T, nq, d], k [T, nk, d], v [T, nv, e] of one sequence, fed in portions through the heads' kernel and
    the attention kernel with pages given out in a scrambled order; returns [T, nq, e]."""
    dt = DTYPES[dtype]
    T, nq, d = q.shape
    nk, nv, e = k.shape[1], v.shape[1], v.shape[2]
    pages = (T + page_size - 1) // page_size + 3
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(T))[:pages - 3]
    table = torch.full((2, pages), -1, dtype=torch.int32)
    table[1, :order.numel()] = order.to(torch.int32)
    table = table.to(DEV)
    kc = torch.full((pages, nk, page_size, d), float("nan"), dtype=dt, device=DEV)
    vc = torch.full((pages, nv, page_size, e), float("nan"), dtype=dt, device=DEV)
    row = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(dt).to(DEV)
    outs, pos = [], 0
    for n in portions:
        n = min(n, T - pos)
        if n <= 0:
            break
        positions, seq_of, rows = i32(list(range(pos, pos + n))), i32([0] * n), i32([1])
        q_out = torch.empty(n, nq * d, dtype=dt, device=DEV)
        kernels.heads_prepare_append(row[pos:pos + n], q_out, kc, vc, bias, norms[0] if norms else None,
                                     norms[1] if norms else None, eps, inv_freq, rot, positions, seq_of, table, nq, nk,
                                     nv, d, e, page_size, rows)
        out = torch.empty(n, nq * e, dtype=torch.float32 if float_out else dt, device=DEV)
        extra = {}
        if slopes is not None:
            extra["distance_bias"] = (slopes, None)
        kernels.attention(q_out, kc, vc, out, table, i32([0, n]), i32([pos + n]), seq_of, positions, nq, nk, d,
                          page_size, scale, window, n, pos + n, n, rows, chunk=chunk, value_dim=e, sink=sink,
                          kv_share=kv_share, **extra)
        outs.append(out.float().cpu().view(n, nq, e))
        pos += n
    kernels.check_error_word()
    return torch.cat(outs)


SHAPES = [(4, 2, 16, 8), (6, 3, 12, 12), (4, 1, 64, 64), (5, 5, 6, 9), (2, 1, 20, 4), (8, 2, 32, 64), (3, 3, 128, 128)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e", SHAPES)
def test_attention_with_a_sink_and_a_linear_bias_in_blocks(kernels, dtype, H, G, d, e):
    g = torch.Generator().manual_seed(H * 100 + d)
    T, block = 150, 37
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    sink = torch.randn(H, generator=g)
    scale = 1.5 / math.sqrt(d)
    qd, kd, vd = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
    i = torch.arange(T, dtype=torch.float64)
    bias = plain.distance_slopes(H, torch.float64)[:, None, None] * (i[:, None] - i[None, :])[None]
    ref = plain.softmax_attention(qd, kd, vd, scale, plain.visible(T, chunk=block), bias=bias, sink=sink.double())
    slopes = plain.distance_slopes(H, torch.float32).to(DEV)
    for portions in ([T], [40, 2, 1, 1, 70, 3, 33], [1] * T if d <= 16 else [100] + [1] * 50):
        got = run_attention(kernels, q, k, v, dtype, 16, portions, scale, chunk=block, sink=sink.to(DEV), slopes=slopes)
        close(got, ref, KTOL[dtype], f"attention {H} {G} {d} {e} {dtype} {portions[:3]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e,rot", [(4, 2, 8, 16, 4), (6, 2, 10, 14, 6), (4, 2, 32, 64, 32), (2, 1, 64, 128, 16),
                                         (2, 2, 12, 12, 0), (4, 2, 32, 32, 16), (3, 1, 16, 48, 8), (2, 2, 128, 128, 64)])
def test_two_maps_share_their_values(kernels, dtype, H, G, d, e, rot):
    """The differential layer's attention: the maps of a key head are key heads of their own, the values are
    stored once; then the maps are joined, normalised and gated."""
    g = torch.Generator().manual_seed(H + d + e)
    T, block, R = 90, 23, H // G
    q, k = torch.randn(T, H, 2, d, generator=g), torch.randn(T, G, 2, d, generator=g)
    v, gate = torch.randn(T, G, e, generator=g), torch.randn(T, H, generator=g)
    scale, lam, diff, eps = 1.2 / math.sqrt(d), 0.37, 0.3, 1e-5
    qd, kd, vd = rounded(q, dtype), rounded(k, dtype), rounded(v, dtype)
    rotation = {"base": 300.0, "dims": rot} if rot else None
    qr = plain.rotate(qd.view(T, 2 * H, d), rotation).view(T, H, 2, d)
    kr = plain.rotate(kd.view(T, 2 * G, d), rotation).view(T, G, 2, d)
    if dtype == "bfloat16":
        qr, kr = rounded(qr, dtype), rounded(kr, dtype)           # the rotated heads are stored in the activations' type
    mask = plain.visible(T, chunk=block)
    a1 = plain.softmax_attention(qr[:, :, 0], kr[:, :, 0], vd, scale, mask)
    a2 = plain.softmax_attention(qr[:, :, 1], kr[:, :, 1], vd, scale, mask)
    ref = plain.rms_unit(a1 - lam * a2, eps) * (1 - diff) * torch.sigmoid(rounded(gate, dtype))[:, :, None]
    # the order of the query rows that the part makes: (key/value head, map, head of the group)
    q_rows = q.view(T, G, R, 2, d).permute(0, 1, 3, 2, 4).reshape(T, 2 * H, d)
    inv_freq = torch.tensor(plain.rotary_frequencies(rotation), dtype=torch.float32, device=DEV) if rot else None
    for portions in ([T], [30, 2, 1, 1, 50, 6], [60] + [1] * 30):
        maps = run_attention(kernels, q_rows, k.view(T, 2 * G, d), v, dtype, 8, portions, scale, chunk=block, kv_share=2,
                             float_out=True, inv_freq=inv_freq, rot=rot)
        out = torch.empty(T, H * e, dtype=DTYPES[dtype], device=DEV)
        kernels.differential_combine(maps.reshape(T, -1).to(DEV), gate.to(DTYPES[dtype]).to(DEV), lam, eps, 1 - diff,
                                     out, H, e, R)
        close(out.view(T, H, e), ref, KTOL[dtype] * 2, f"two maps {H} {G} {d} {e} {dtype} {portions[:2]}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["window", "block", "block, two maps"])
def test_attention_sees_its_window_or_block_and_nothing_else(kernels, dtype, kind):
    """One key is made to stand out (its score beats all others by far, its value is known): queries that see
    it return its value, queries that do not return none of it.  The key sits far back, right before and
    right after a page border, just inside and just outside the window or block, for rows of a prompt and
    for tokens decoded alone."""
    H, G, d, e, T, page = 4, 2, 16, 16, 400, 16
    span = 100
    maps = 2 if kind.endswith("maps") else 1
    for key_pos in (0, 15, 16, 207, 299, 300, 301):
        g = torch.Generator().manual_seed(key_pos)
        q, k = torch.randn(T, H * maps, d, generator=g) * 0.1, torch.randn(T, G * maps, d, generator=g) * 0.1
        v = torch.randn(T, G, e, generator=g) * 0.01
        k[key_pos] = 3.0
        q[:, :, :] += 1.0                                       # q . k[key_pos] = 48 +- a little, all other scores about 0
        v[key_pos] = 7.0
        window = span if kind == "window" else None
        chunk = span if kind != "window" else None
        for portions in ([T], [300] + [1] * 100, [3, 2, 290, 2, 1, 1, 1, 2, 98]):
            got = run_attention(kernels, q, k, v, dtype, page, portions, 1.0, window=window, chunk=chunk,
                                kv_share=maps, float_out=maps > 1)
            for p in range(T):
                sees = key_pos <= p and (p - key_pos < span if kind == "window" else p // span == key_pos // span)
                row = got[p]
                if sees:
                    assert float((row - 7.0).abs().max()) < 0.1, (kind, dtype, key_pos, p, portions[:2])
                else:
                    assert float(row.abs().max()) < 0.1, (kind, dtype, key_pos, p, portions[:2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_large_sink_takes_the_weight(kernels, dtype):
    H, d, T = 2, 16, 20
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, H, d, generator=g) for _ in range(3))
    sink = torch.tensor([30.0, -30.0])
    got = run_attention(kernels, q, k, v, dtype, 4, [T], 0.1, sink=sink.to(DEV), slopes=torch.zeros(H, device=DEV))
    assert float(got[:, 0].abs().max()) < 1e-6
    ref = plain.softmax_attention(rounded(q, dtype), rounded(k, dtype), rounded(v, dtype), 0.1, plain.visible(T))
    close(got[:, 1], ref[:, 1], KTOL[dtype], "a sink far below the scores changes nothing")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,e,rot", [(6, 3, 12, 12, 12), (4, 1, 64, 64, 32), (2, 1, 20, 4, 20), (4, 2, 6, 10, 2),
                                         (3, 3, 16, 16, 0)])
def test_heads_with_biases_norms_and_rotation(kernels, dtype, H, G, d, e, rot):
    g = torch.Generator().manual_seed(d * 7 + e)
    T, eps = 70, 1e-5
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    bias = torch.randn(H * d + G * d + G * e, generator=g) * 0.3
    wq, wk = 0.5 + torch.rand(d, generator=g), 0.5 + torch.rand(d, generator=g)
    rotation = {"base": 77.0, "dims": rot, "scaling": {"factor": 2.0, "low": 0.5, "high": 8.0, "original": 16.0}} \
        if rot else None
    bq, bk, bv = bias[:H * d].view(H, d), bias[H * d:H * d + G * d].view(G, d), bias[H * d + G * d:].view(G, e)
    qd = plain.rotate(plain.rms_norm(rounded(q, dtype) + bq.double(), wq.double(), eps), rotation)
    kd = plain.rotate(plain.rms_norm(rounded(k, dtype) + bk.double(), wk.double(), eps), rotation)
    vd = rounded(v, dtype) + bv.double()
    if dtype == "bfloat16":
        qd, kd, vd = rounded(qd, dtype), rounded(kd, dtype), rounded(vd, dtype)
    scale = 1.0 / math.sqrt(d)
    ref = plain.softmax_attention(qd, kd, vd, scale, plain.visible(T, window=21))
    inv_freq = torch.tensor(plain.rotary_frequencies(rotation), dtype=torch.float32, device=DEV) if rot else None
    for portions in ([T], [20, 2, 1, 30, 17]):
        got = run_attention(kernels, q, k, v, dtype, 16, portions, scale, window=21, bias=bias.to(DEV),
                            norms=(wq.to(DEV), wk.to(DEV)), eps=eps, inv_freq=inv_freq, rot=rot)
        close(got, ref, KTOL[dtype], f"heads {H} {G} {d} {e} {rot} {dtype}")


# ------------------------------------------------------------------ the state-space branch
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,e,N,G,taps", [(4, 12, 8, 2, 3), (3, 10, 5, 1, 1), (4, 64, 64, 1, 4), (6, 7, 9, 3, 5),
                                          (2, 40, 130, 2, 2), (8, 16, 256, 4, 4), (2, 9, 300, 1, 2), (1, 20, 500, 1, 3)])
def test_convolution_and_scan_over_portions(kernels, dtype, H, e, N, G, taps):
    """Two sequences side by side, one in portions and one token by token from a slot that was used before,
    against the plain recurrence over the whole sequences; the kept state is compared too."""
    g = torch.Generator().manual_seed(H * e + N)
    dt_type = DTYPES[dtype]
    inner, C = H * e, H * e + 2 * G * N
    lens = [53, 30]
    raw = [torch.randn(n, C, generator=g) for n in lens]
    dts = [torch.randn(n, H, generator=g) for n in lens]
    conv_w, conv_b = torch.randn(C, taps, generator=g) * 0.5, torch.randn(C, generator=g) * 0.2
    dt_bias, a_log, skip = torch.rand(H, generator=g) * 2 - 2, torch.rand(H, generator=g) * 3 - 2, torch.rand(H, generator=g)
    refs, states = [], []
    for x, d in zip(raw, dts):
        xbc = plain.silu(plain.causal_conv(rounded(x, dtype), conv_w.double(), conv_b.double()))
        if dtype == "bfloat16":
            xbc = rounded(xbc, dtype)
        n = x.shape[0]
        y, S = plain.state_space_scan(xbc[:, :inner].reshape(n, H, e), xbc[:, inner:inner + G * N].reshape(n, G, N),
                                      xbc[:, inner + G * N:].reshape(n, G, N),
                                      plain.softplus(rounded(d, dtype) + dt_bias.double()), a_log.double(), skip.double())
        refs.append(y.reshape(n, inner))
        states.append(S)
    state = torch.full((3, H, e, N), 5.0, device=DEV)
    history = torch.full((3, max(taps - 1, 1), C), 5.0, dtype=dt_type, device=DEV)
    state[[2, 0]] = 0.0                                          # what admission does to a slot
    history[[2, 0]] = 0.0
    slots = [2, 0]
    steps = [(9, 1), (2, 1), (1, 1), (30, 1), (11, 1)] + [(0, 1)] * 25
    pos = [0, 0]
    got = [[], []]
    wt = conv_w.t().contiguous().to(DEV)
    for na, nb in steps:
        ns = [min(na, lens[0] - pos[0]), min(nb, lens[1] - pos[1])]
        live = [s for s in (0, 1) if ns[s] > 0]
        if not live:
            break
        x = torch.cat([raw[s][pos[s]:pos[s] + ns[s]] for s in live]).to(dt_type).to(DEV)
        d = torch.cat([dts[s][pos[s]:pos[s] + ns[s]] for s in live]).to(dt_type).to(DEV)
        q_start = i32([0] + list(np.cumsum([ns[s] for s in live])))
        sl = i32([slots[s] for s in live])
        xbc = torch.empty_like(x)
        kernels.causal_conv(x, conv_w.to(DEV), conv_b.to(DEV), history, xbc, q_start, sl, max(ns), activation="silu",
                            weight_t=wt)
        y = torch.empty(x.shape[0], inner, dtype=torch.float32, device=DEV)
        kernels.state_space_scan(xbc, d, dt_bias.to(DEV), a_log.to(DEV), skip.to(DEV), state, y, q_start, sl, H, G, e, N)
        at = 0
        for s in live:
            got[s].append(y[at:at + ns[s]].cpu())
            at += ns[s]
            pos[s] += ns[s]
    for s in (0, 1):
        close(torch.cat(got[s]), refs[s], KTOL[dtype], f"scan {H} {e} {N} {G} {taps} {dtype} sequence {s}")
        close(state[slots[s]].transpose(1, 2), states[s], KTOL[dtype], f"scan state {dtype} sequence {s}")
    assert float((state[1] - 5.0).abs().max()) == 0.0            # a slot of nobody is not touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_value_survives_long_in_the_state(kernels, dtype):
    """A head that hardly decays keeps what the first token wrote for 600 tokens; a head that decays fast has
    lost it after a few."""
    H, e, N, T = 2, 4, 4, 600
    dt_type = DTYPES[dtype]
    xbc = torch.zeros(T, H * e + 2 * N)
    xbc[0, :H * e] = 1.0
    xbc[0, H * e] = 1.0                                          # B of the first token: state row 0
    xbc[:, H * e + N] = 1.0                                      # C reads state row 0 at every token
    dt = torch.zeros(T, H)
    a_log = torch.tensor([-12.0, 2.0])
    state = torch.zeros(1, H, e, N, device=DEV)
    y = torch.empty(T, H * e, dtype=torch.float32, device=DEV)
    for a, b in ((0, 200), (200, 201), (201, 600)):
        kernels.state_space_scan(xbc[a:b].to(dt_type).to(DEV), dt[a:b].to(dt_type).to(DEV), torch.zeros(H, device=DEV),
                                 a_log.to(DEV), torch.zeros(H, device=DEV), state, y[a:b], i32([0, b - a]), i32([0]), H, 1,
                                 e, N)
    step = math.log(2.0)                                         # softplus(0)
    ref0 = step * math.exp(-math.exp(-12.0) * step * (T - 1))
    assert abs(float(y[T - 1, 0]) - ref0) < 1e-4 * ref0 and float(y[10, e]) < 1e-12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,W,parts", [(1, 48, 1), (37, 30, 3), (300, 256, 2), (5, 1000, 8), (3, 5000, 2), (2, 2048, 1)])
def test_gated_norm_in_parts(kernels, dtype, T, W, parts):
    g = torch.Generator().manual_seed(T + W)
    y, z, w = torch.randn(T, W, generator=g) * 3, torch.randn(T, W, generator=g), 0.5 + torch.rand(W, generator=g)
    v = y.double() * plain.silu(rounded(z, dtype))
    ref = plain.rms_unit(v.view(T, parts, W // parts), 1e-5).reshape(T, W) * w.double()
    wide = torch.randn(T, W + 24, generator=g).to(DTYPES[dtype]).to(DEV)      # z as a slice of a wider array
    wide[:, 8:8 + W] = z.to(DTYPES[dtype]).to(DEV)
    out = torch.empty(T, W, dtype=DTYPES[dtype], device=DEV)
    kernels.gated_group_rms(y.to(DEV), wide[:, 8:8 + W], w.to(DEV), 1e-5, parts, out)
    close(out, ref, KTOL[dtype], f"gated norm {T} {W} {parts} {dtype}")


# ------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [70, 72, 1024])                  # (multiples of 8: 16 bytes of bfloat16 a thread)
def test_clamped_gate(kernels, dtype, n):
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(33, 2 * n, generator=g) * 2
    gd = rounded(gu, dtype)
    a, u = gd[:, :n].clamp(max=1.25), gd[:, n:].clamp(-1.25, 1.25)
    ref = a * torch.sigmoid(1.702 * a) * (u + 1)
    out = torch.empty(33, n, dtype=DTYPES[dtype], device=DEV)
    kernels.clamped_swish_gate(gu.to(DTYPES[dtype]).to(DEV), out, 1.25, 1.702)
    close(out, ref, KTOL[dtype], f"clamped gate {dtype}")
    assert float(ref.max()) <= 1.25 * 2.25 and float((gd[:, :n] > 1.25).sum()) > 0 and float((gd[:, n:] < -1.25).sum()) > 0


@pytest.mark.parametrize("n,top,groups,keep", [(8, 2, 1, 1), (8, 3, 2, 1), (8, 2, 4, 2), (20, 3, 2, 1), (6, 1, 3, 2),
                                               (33, 5, 11, 7), (130, 8, 10, 3), (5, 5, 1, 1)])
def test_router_choice(kernels, n, top, groups, keep):
    g = torch.Generator().manual_seed(n * top)
    T = 257
    logits = torch.randn(T, n, generator=g) * 1.5
    corr = torch.randn(n, generator=g) * 0.05
    mlp = {"router": {"experts": n - 2, "identity": 2, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}}
    w = {"r.router": torch.eye(n, dtype=torch.float64), "r.correction": corr.double()}
    margins = torch.full((T,), float("inf"), dtype=torch.float64)
    ref_chosen, ref_weight = plain.route(logits.double(), mlp, w, "r.", margins)
    chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
    share = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.router_choose(logits.to(DEV), corr.to(DEV), chosen, share, groups, keep, 1.7, last_choice=n - 2)
    clear = margins > 1e-5
    assert int(clear.sum()) > T * 0.9
    assert torch.equal(chosen.cpu()[clear].long(), ref_chosen[clear].clamp(max=n - 2))
    close(share.cpu()[clear], ref_weight[clear], 1e-5, "router weights")


def test_router_ties_go_to_the_lower_number(kernels):
    logits = torch.zeros(3, 12, device=DEV)
    corr = torch.zeros(12, device=DEV)
    chosen = torch.empty(3, 4, dtype=torch.int32, device=DEV)
    share = torch.empty(3, 4, dtype=torch.float32, device=DEV)
    kernels.router_choose(logits, corr, chosen, share, 3, 2, 2.0)
    assert chosen.cpu().tolist() == [[0, 1, 2, 3]] * 3 and torch.allclose(share.cpu(), torch.full((3, 4), 2.0 / 12))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,F,E,identity,top", [(1, 64, 24, 6, 2, 2), (9, 48, 16, 4, 2, 1), (300, 96, 40, 5, 3, 4),
                                                  (700, 128, 64, 7, 1, 2), (64, 256, 128, 8, 0, 2), (5, 352, 160, 12, 2, 3),
                                                  (1500, 256, 64, 3, 1, 2), (40, 72, 24, 5, 3, 4)])
def test_gated_experts_with_identity_ones(kernels, dtype, T, D, F, E, identity, top):
    """Choices given (every output appears, identity ones too): the sum over a token's choices of weight *
    expert(x), an identity expert returning x; plain, mma.sync and tcgen05 kernels by size."""
    g = torch.Generator().manual_seed(T + D + F)
    dt = DTYPES[dtype]
    x = torch.randn(T, D, generator=g)
    outputs = E + identity
    chosen = torch.stack([torch.randperm(outputs, generator=g)[:top] for _ in range(T)])
    share = torch.rand(T, top, generator=g)
    gate, up = torch.randn(E, F, D, generator=g) / math.sqrt(D), torch.randn(E, F, D, generator=g) / math.sqrt(D)
    down = torch.randn(E, D, F, generator=g) / math.sqrt(F)
    xd = rounded(x, dtype)
    ref = torch.zeros(T, D, dtype=torch.float64)
    w = {}
    for e_ in range(E):
        w.update({f"e{e_}.gate": rounded(gate[e_], dtype), f"e{e_}.up": rounded(up[e_], dtype),
                  f"e{e_}.down": rounded(down[e_], dtype)})
    for e_ in range(outputs):
        rows = (chosen == e_).nonzero()
        if rows.numel() == 0:
            continue
        t_idx = rows[:, 0]
        wt = share[rows[:, 0], rows[:, 1]].double()[:, None]
        y = plain.expert_ff(xd[t_idx], w, f"e{e_}.") if e_ < E else xd[t_idx]
        ref.index_add_(0, t_idx, wt * y)
    buckets = E + (1 if identity else 0)
    inter = kernels.expert_tensor_cores(dt, D, F)
    stacked = torch.zeros(buckets, 2 * F, D, dtype=dt)
    stacked_down = torch.zeros(buckets, D, F, dtype=dt)
    for e_ in range(E):
        stacked[e_] = kernels.interleave_expert_gate_up(gate[e_].to(dt), up[e_].to(dt)) if inter else \
            torch.cat([gate[e_], up[e_]]).to(dt)
        stacked_down[e_] = down[e_].to(dt)
    pairs = T * top
    acc = torch.zeros(T, D, device=DEV)
    route = torch.empty(kernels.route_words(pairs, buckets), dtype=torch.int32, device=DEV)
    act = torch.empty(pairs, F, dtype=dt, device=DEV)
    y = torch.empty(pairs, D, dtype=torch.float32, device=DEV)
    sorted_x = torch.empty(pairs, D, dtype=dt, device=DEV)
    kernels.chosen_experts(x.to(dt).to(DEV), chosen.clamp(max=buckets - 1).to(torch.int32).to(DEV), share.to(DEV),
                           stacked.to(DEV), stacked_down.to(DEV), acc, route, act, y, "silu", sorted_x, gated=True,
                           interleaved=inter, identity=identity)
    kernels.check_error_word()
    close(acc, ref, KTOL[dtype] * 2, f"experts {T} {D} {F} {E} {identity} {top} {dtype}")


# ------------------------------------------------------------------ the stream
def test_bigram_rows_across_steps_and_slots(kernels):
    n, buckets, mp, mc = 24, 13, 1000003, 7
    g = torch.Generator().manual_seed(2)
    table = torch.randn(buckets + 1, n, generator=g)
    seqs = {0: torch.randint(0, 5000, (40,), generator=g).tolist(), 1: torch.randint(0, 5000, (9,), generator=g).tolist()}
    kept = torch.full((3, 1), 4321, dtype=torch.int32, device=DEV)
    slots = {0: 2, 1: 0}
    got = {0: [], 1: []}
    pos = {0: 0, 1: 0}
    for na, nb in ((5, 1), (1, 1), (20, 2), (2, 0), (12, 5)):
        live = [(s, m) for s, m in ((0, na), (1, nb)) if m > 0 and pos[s] < len(seqs[s])]
        toks = [t for s, m in live for t in seqs[s][pos[s]:pos[s] + m]]
        positions = [p for s, m in live for p in range(pos[s], pos[s] + m)]
        seq_of = [i for i, (s, m) in enumerate(live) for _ in range(m)]
        res = torch.zeros(len(toks), n, device=DEV)
        kernels.bigram_embed(res, table.to(DEV), kept, i32(toks), i32(positions), i32(seq_of),
                             i32([0] + list(np.cumsum([m for _, m in live]))), i32([slots[s] for s, _ in live]), mp, mc)
        at = 0
        for s, m in live:
            got[s].append(res[at:at + m].cpu())
            at += m
            pos[s] += m
    for s in (0, 1):
        rows = plain.bigram_rows(seqs[s], {"buckets": buckets, "mul_prev": mp, "mul_cur": mc})
        assert torch.equal(torch.cat(got[s]), table[rows])
    assert int(kept[1, 0]) == 4321 and int(kept[2, 0]) == seqs[0][-1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,n", [(1, 40), (37, 64), (5, 1000), (300, 257)])
def test_scaled_sum_and_norm(kernels, dtype, T, n):
    g = torch.Generator().manual_seed(T + n)
    x, delta, vec = torch.randn(T, n, generator=g), torch.randn(T, n, generator=g), torch.rand(n, generator=g)
    w = (0.5 + torch.rand(n, generator=g)).to(DTYPES[dtype])
    res = x.clone().to(DEV)
    out = torch.empty(T, n, dtype=DTYPES[dtype], device=DEV)
    kernels.scaled_add_norm(res, delta.to(DEV), vec.to(DEV), norm=(w.to(DEV), 1e-5, 0.0, out))
    new = x.double() + vec.double() * delta.double()
    close(res, new, 1e-6, "scaled sum")
    close(out, plain.rms_norm(new, w.double(), 1e-5), KTOL[dtype], "norm after the scaled sum")
    x0, step = torch.randn(T, n, generator=g), torch.randn(n, generator=g)
    kernels.stream_enter(res, x0.to(DEV), step.to(DEV))
    close(res, new + x0.double() + step.double(), 1e-6, "entering a pass")
    a, b = torch.randn(T, n, generator=g), torch.randn(T, n, generator=g)
    kernels.add_weighted(res, a.to(DEV), 0.7, b.to(DEV), -1.3)
    close(res, new + x0.double() + step.double() + 0.7 * a.double() - 1.3 * b.double(), 1e-6, "weighted branches")


# ------------------------------------------------------------------ whole models
SEED = 21
CASES = {"G1": (4, [1, 40, 100], [20, 70, 9, 130, 33, 2, 64]),
         "G2": (16, [2, 64, 90], [20, 70, 9, 100, 33, 2]),
         "G3": (16, [3, 70, 150], [150, 64, 9, 200, 33, 2, 100]),
         "G4": (8, [5, 33, 120], [20, 70, 9, 130, 33, 2, 64])}
TOL = {"float32": helpers.TOL["float32"], "bfloat16": 8e-2}


def weights_for(config, dtype, seed=SEED):
    w = dogetar_models.random_weights(config, seed)
    return dogetar_models.decisive(w) if dtype == "bfloat16" else w


def make_runner(folder, dtype, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests)
    runner.storage.poison()
    return runner


def compare(got, ref, margins, dtype, what):
    a, b = dogetar_models.cut_to_safe(got, ref, margins, dtype, most_lost=0.7 if dtype == "float32" else 0.1)
    helpers.assert_logits_close(a, b, TOL[dtype], what)


ALONE = {
    "window": dogetar_models.windowed(4, 2, 32, 32, window=50, rot=16, bands=(4.0, 1.0, 4.0, 64.0)),
    "window, other value size": dogetar_models.windowed(6, 3, 24, 40, window=37, rot=24),
    "two maps": dogetar_models.differential(4, 2, 16, 32, chunk=40, rot=16),
    "two maps, three heads to a key head": dogetar_models.differential(6, 2, 12, 20, chunk=64, rot=6),
    "parallel": dogetar_models.parallel((4, 2, 16, 24, 48), {"heads": 4, "vdim": 16, "state": 16, "groups": 2, "conv": 4,
                                                             "norm_groups": 2}, 0.8, 1.3),
    "dense": dogetar_models.windowed(1, 1, 16, mlp=dogetar_models.dense(72, 0.5)),
    "experts": dogetar_models.windowed(1, 1, 16, mlp=dogetar_models.moe(64, 6, 2, identity=2, groups=(4, 2), scale=2.5,
                                                                        shared=32)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", list(ALONE))
def test_one_layer_alone(tmp_path, kind, dtype):
    cfg = {"architecture": "Dogetar", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "layers": [ALONE[kind]]}
    w = weights_for(cfg, dtype, 7)
    folder = dogetar_models.write_model(cfg, str(tmp_path / "one"), seed=7, weights=w)
    reqs = helpers.random_requests(cfg["vocab"], [1, 30, 130], seed=3)
    margins = {}
    ref = dogetar_models.plain_logits(cfg, 7, reqs, weights=w, margins=margins)
    runner = make_runner(folder, dtype, 16, 192)
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 40), "decoded"),
                        (helpers.trace_portions(reqs, seed=5), "portions")):
        compare(helpers.run_trace(runner, trace), ref, margins, dtype, f"dogetar one layer ({kind}) {dtype} {what}")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("dogetar")
    return {(name, dtype): dogetar_models.write_model(dogetar_models.get(name), str(root / f"{name}_{dtype}"), seed=SEED,
                                                      weights=weights_for(dogetar_models.get(name), dtype))
            for name in CASES for dtype in DTYPES}


@pytest.fixture(scope="module")
def expected():
    out = {}
    for name, (_, lengths, mixed_lengths) in CASES.items():
        for dtype in DTYPES:
            cfg = dogetar_models.get(name)
            w = weights_for(cfg, dtype)
            reqs = helpers.random_requests(cfg["vocab"], lengths, seed=100)
            mixed = helpers.random_requests(cfg["vocab"], mixed_lengths, seed=200)
            m1, m2 = {}, {}
            out[name, dtype] = (reqs, dogetar_models.plain_logits(cfg, SEED, reqs, weights=w, margins=m1), m1,
                                mixed, dogetar_models.plain_logits(cfg, SEED, mixed, weights=w, margins=m2), m2)
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
        compare(got, ref, margins, dtype, f"dogetar {case} {dtype} {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    runner.runtime.kernels.check_error_word()
    pool = 384
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are used again
    runner2 = make_runner(folders[case, dtype], dtype, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    compare(got, mixed_ref, mixed_margins, dtype, f"dogetar {case} {dtype} mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_against_each_request_alone(folders, dtype):
    """Four unequal requests in the same steps against each in steps of its own, both against the plain
    implementation."""
    cfg = dogetar_models.get("G3")
    w = weights_for(cfg, dtype)
    reqs = helpers.random_requests(cfg["vocab"], [90, 7, 140, 33], seed=17)
    margins = {}
    ref = dogetar_models.plain_logits(cfg, SEED, reqs, weights=w, margins=margins)
    runner = make_runner(folders["G3", dtype], dtype, 16, 512)
    alone = helpers.run_trace(runner, helpers.trace_portions(reqs, seed=3))
    compare(alone, ref, margins, dtype, f"dogetar G3 {dtype} each alone")
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
    compare(together, ref, margins, dtype, f"dogetar G3 {dtype} together")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(folders, dtype):
    """1,300 tokens through the model of tensor-core sizes: whole, in portions of 100 to 130 tokens (few query
    rows over a long context, where the prompt kernels cut the keys into ranges) and with its last 40 tokens
    decoded; windows, blocks and the looped layers' caches far from the sequence's start."""
    cfg = dogetar_models.get("G3")
    w = weights_for(cfg, "bfloat16")                 # (the corrections spaced out: 1,300 positions without a close call)
    reqs = helpers.random_requests(cfg["vocab"], [1300], seed=31)
    margins = {}
    ref = dogetar_models.plain_logits(cfg, SEED, reqs, weights=w, margins=margins)
    runner = make_runner(folders["G3", "bfloat16"], dtype, 16, 1344)
    ids = reqs["r0"]
    steps, pos, sizes, k = [], 0, [100, 130, 128, 3, 117], 0
    while pos < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - pos)
        k += 1
        steps.append({"step": len(steps), "entries": [{"id": "r0", "tokens": ids[pos:pos + n], "want": list(range(n))}],
                      "end": ["r0"] if pos + n == len(ids) else []})
        pos += n
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (steps, "portions of about 100"),
                        (helpers.trace_last_decoded(reqs, 40), "last 40 decoded")):
        compare(helpers.run_trace(runner, trace), ref, margins, dtype, f"dogetar G3 {dtype} long prompt {what}")
    runner.runtime.kernels.check_error_word()


def test_long_decoding(folders):
    """Three tokens of prompt, then 300 tokens one by one (captured steps replayed): blocks of 24 and 20
    positions and a window of 13 pass over decoded tokens many times, the state-space branch's state is
    carried 300 times in each of its two passes."""
    cfg = dogetar_models.get("G1")
    w = weights_for(cfg, "bfloat16")
    reqs = helpers.random_requests(cfg["vocab"], [303], seed=9)
    margins = {}
    ref = dogetar_models.plain_logits(cfg, SEED, reqs, weights=w, margins=margins)
    runner = make_runner(folders["G1", "bfloat16"], "bfloat16", 4, 320)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 300))
    compare(got, ref, margins, "bfloat16", "dogetar G1 bfloat16 long decoding")
    assert runner.graph_replays > 200


def test_greedy_generation_through_the_entry_point(folders):
    """``LLM.generate`` (scheduler, sampler, portions of 16 tokens, three requests at a time): every generated
    token is the plain implementation's best one, wherever that leads by more than the rounding of a 32-bit
    run and no router's choice was a close call."""
    from chibillm_b200 import LLM
    cfg = dogetar_models.get("G3")
    w = dogetar_models.decisive(dogetar_models.random_weights(cfg, SEED))
    prompts = list(helpers.random_requests(cfg["vocab"], [5, 40, 23, 61], seed=12).values())
    llm = LLM(folders["G3", "bfloat16"], dtype="float32", context_length=128, max_sequences=3, max_batch_tokens=48,
              prefill_chunk_tokens=16, page_size=16)
    outs = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for prompt, new in zip(prompts, outs):
        assert len(new) == 12
        ref = dogetar_models.plain_logits(cfg, SEED, {"a": prompt + new}, weights=w)["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok, f"token {i} of a prompt of {len(prompt)}"


def test_trace_program(folders, tmp_path):
    """bin/trace_run on a Dogetar folder: portions, single tokens, two live requests."""
    a_len, b_len = 40, 21
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dogetar_models.get("G4")
    w = weights_for(cfg, "bfloat16")
    reqs = helpers.random_requests(cfg["vocab"], [a_len, b_len], seed=5)
    ref = dogetar_models.plain_logits(cfg, SEED, reqs, weights=w)
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]},
                                     {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0, 1]},
                                     {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "b"]}]
    want = [[("r0", 0), ("r0", 29)], [("r0", 30), ("r1", 18)], [("r1", 19), ("r1", 20), ("r0", 39)]]
    for dtype in ("float32", "bfloat16"):
        out_dir = str(tmp_path / dtype)
        proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model",
                               folders["G4", "bfloat16"], "--dtype", dtype, "--out", out_dir, "--max-tokens", "128"],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                              timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for i, rows in enumerate(want):
            got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(len(rows), -1))
            for j, (r, pos) in enumerate(rows):
                scale = float(ref[r].abs().max())
                assert float((got[j] - ref[r][pos]).abs().max()) <= TOL[dtype] * scale, (dtype, i, r, pos)


def test_random_weights_made_on_the_device(tmp_path):
    """``ModelRunner.from_random`` makes on the device the values that ``write_random_model`` stores: both
    give the same logits."""
    from chibillm_b200.engine.batch import StepEntry
    from chibillm_b200.engine.runner import ModelRunner
    from chibillm_b200.weights import write_random_model
    cfg = dogetar_models.get("G4")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=6)
    ids = helpers.random_requests(cfg["vocab"], [50], seed=2)["r0"]
    a = ModelRunner.from_folder(folder, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    b = ModelRunner.from_random(cfg, seed=6, dtype="float32", device=DEV, page_size=8, pool_tokens=64)
    la = a.step([StepEntry("x", ids, list(range(50)))]).clone()
    lb = b.step([StepEntry("x", ids, list(range(50)))]).clone()
    assert torch.equal(la, lb)
