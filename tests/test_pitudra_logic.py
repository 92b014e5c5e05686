"""Pitudra without a GPU: the configuration reader, the plain implementation's own
consistency on cases worked out by hand, and the engine's logic (batching, paging,
state slots, a layer that reads another layer's latents, routed experts, the token
input) on the plain PyTorch stand-ins of the kernels, against the plain
implementation of the design."""
import io
import json
import math
import os

import pytest
import torch

import helpers
import pitudra_models
import plain_pitudra as plain
from reference_ops import ReferenceKernels


def cpu_runner(folder, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests,
                                     kernels=ReferenceKernels())
    runner.storage.poison()
    return runner


# ------------------------------------------------------------------ configuration
def test_parts_follow_the_file(tmp_path):
    from chibillm_b200.config import load_config
    folder = pitudra_models.write_model(pitudra_models.get("P1"), str(tmp_path / "p1"), seed=1)
    arch, config, spec = load_config(folder)
    assert arch.name == "Pitudra" and spec.max_positions == 0
    assert [(s.layer, s.cache_of) for s in spec.run_order] == [(0, None), (1, None), (2, None), (3, 0)]
    assert [l.arrangement for l in spec.layers] == ["postnorm"] * 4 and all(l.token_shift for l in spec.layers)
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "gated_recurrence", "attention",
                                                   "latent_attention"]
    lat, rec, att, reader = (l.mixer for l in spec.layers)
    assert (lat.num_heads, lat.head_dim, lat.rope_dim, lat.value_dim, lat.q_rank, lat.kv_rank, lat.window, lat.own_kv,
            lat.sink, lat.norm_eps) == (3, 16, 8, 24, 40, 24, 20, True, True, 1e-5)
    assert (lat.position.rotary_dim, lat.position.theta) == (8, 1000.0)
    # the source keeps its latents as long as its reader's longer window needs them
    assert lat.cache_window == 33 and reader.cache_window == 33 and reader.window == 33 and not reader.own_kv
    assert (rec.num_heads, rec.head_dim, rec.value_dim) == (2, 24, 16)
    assert (att.num_heads, att.num_kv_heads, att.head_dim, att.value_dim, att.window, att.sink, att.biases,
            att.output_gate, att.whole_norm_eps, att.position.kind) == (4, 2, 16, 8, 13, True, True, True, 1e-5, "none")
    ff = [l.feed_forward for l in spec.layers]
    assert [(f.kind, f.num_experts, f.top, f.intermediate_size, f.activation) for f in ff] == \
        [("routed_experts", 5, 2, 40, "relu2"), ("routed_experts", 3, 3, 24, "relu2"),
         ("routed_experts", 4, 1, 32, "relu2"), ("routed_experts", 5, 2, 40, "relu2")]
    assert [l.token_input.offset for l in spec.layers] == [0, 12, 24, 36] and spec.shared_tensors[0][1] == (211, 48)
    assert spec.final_norm.kind == "layernorm" and spec.layers[0].mixer_norm.kind == "layernorm"

    _, _, bare = load_config(pitudra_models.write_model(pitudra_models.get("P2"), str(tmp_path / "p2"), seed=1))
    assert bare.shared_tensors == () and all(l.token_input is None for l in bare.layers)
    assert bare.layers[1].feed_forward is None and bare.layers[1].feed_forward_norm is None
    assert all(l.mixer.window is None for l in bare.layers if l.mixer.kind != "gated_recurrence")
    assert bare.layers[2].mixer.cache_window is None and bare.layers[1].mixer.value_dim == 24


def test_config_errors_name_the_key():
    from chibillm_b200.config import ConfigError, PitudraConfig
    good = pitudra_models.get("P1")

    def read(change):
        obj = json.loads(json.dumps(good))
        change(obj)
        return PitudraConfig.from_dict(obj)

    read(lambda o: None)
    for change, word in [
            (lambda o: o.pop("vocab"), "vocab"),
            (lambda o: o["norm"].pop("eps"), "eps"),
            (lambda o: o.update(layers=[]), "layers"),
            (lambda o: o["layers"][0].update(type="recurrent"), "type"),
            (lambda o: o["layers"][2]["mixer"].update(kv_heads=3), "kv_heads"),
            (lambda o: o["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
            (lambda o: o["layers"][0]["mixer"].update(rot_dim=7) or o["layers"][0]["mixer"]["rot"].update(dims=7),
             "rot.dims"),
            (lambda o: o["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
            (lambda o: o["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
            (lambda o: o["layers"][3]["mixer"].update(kv_rank=16), "kv_rank"),
            (lambda o: o["layers"][3]["mixer"]["rot"].update(base=10.0), "rotation"),
            (lambda o: o["layers"][1]["mlp"]["router"].update(top=4), "top"),
            (lambda o: o["layers"][1]["mlp"].update(kind="dense"), "kind"),
            (lambda o: o["layers"][0]["mixer"]["mask"].update(size=0), "size"),
            (lambda o: o["layers"][2]["mixer"].pop("scale"), "scale")]:
        with pytest.raises(ConfigError) as e:
            read(change)
        assert word in str(e.value), str(e.value)


# ------------------------------------------------------------------ the plain implementation itself
def test_plain_token_shift_and_norm_by_hand():
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [-1.0, 0.0]], dtype=torch.float64)
    mix = torch.tensor([0.25, 1.0], dtype=torch.float64)
    got = plain.token_shift(h, mix)
    # the first token moves towards zeros; with mix 1 a feature IS the previous token's
    assert got.tolist() == [[0.75, 0.0], [2.5, 2.0], [0.0, 6.0]]
    x = torch.tensor([[1.0, 3.0]], dtype=torch.float64)
    w, b = torch.tensor([2.0, 0.5], dtype=torch.float64), torch.tensor([0.1, -0.1], dtype=torch.float64)
    y = plain.layer_norm(x, w, b, 0.5)                      # mean 2, variance 1
    assert abs(float(y[0, 0]) - (-1 / math.sqrt(1.5) * 2.0 + 0.1)) < 1e-15
    assert abs(float(y[0, 1]) - (1 / math.sqrt(1.5) * 0.5 - 0.1)) < 1e-15
    assert abs(float(plain.unit_rms(x, 1.0)[0, 1]) - 3.0 / math.sqrt(6.0)) < 1e-15    # mean square 5, + eps


def test_plain_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).repeat(3, 1, 1)
    y = plain.rotate(x, torch.tensor([0, 1, 2]), 100.0, 4)
    assert torch.equal(y[0], x[0])
    f = [1.0, 100.0 ** -0.5]
    for p in (1, 2):
        for i in range(2):
            a = p * f[i]
            assert abs(float(y[p, 0, i]) - (x[p, 0, i] * math.cos(a) - x[p, 0, i + 2] * math.sin(a))) < 1e-12
            assert abs(float(y[p, 0, i + 2]) - (x[p, 0, i + 2] * math.cos(a) + x[p, 0, i] * math.sin(a))) < 1e-12
        assert float(y[p, 0, 4]) == 5.0


def test_plain_window_and_sink_by_hand():
    assert plain.window_mask(5, 2).int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0],
                                                      [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert plain.window_mask(3, None).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    assert plain.window_mask(3, 1).int().tolist() == [[1, 0, 0], [0, 1, 0], [0, 0, 1]]
    scores = torch.tensor([[[0.0, 9.0], [math.log(2.0), 0.0]]], dtype=torch.float64)
    sink = torch.tensor([math.log(3.0)], dtype=torch.float64)
    p = plain.softmax_with_sink(scores, sink, plain.window_mask(2, None))
    # row 0 sees one key of weight 1 and the sink of weight 3; row 1: 2, 1 and 3
    assert torch.allclose(p[0], torch.tensor([[0.25, 0.0], [2.0 / 6.0, 1.0 / 6.0]], dtype=torch.float64), atol=1e-15)
    assert torch.allclose(plain.softmax_with_sink(scores, None, plain.window_mask(2, None))[0, 1].sum(),
                          torch.tensor(1.0, dtype=torch.float64))


def test_plain_recurrence_by_hand():
    """One head, two key channels, one value channel, weights that pass h through."""
    big = 40.0
    w = {"m.q": torch.eye(2, 3, dtype=torch.float64), "m.v": torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64),
         "m.f": torch.zeros(2, 3, dtype=torch.float64), "m.f.b": torch.tensor([0.0, -big], dtype=torch.float64),
         "m.lower": torch.tensor([0.0, 0.5], dtype=torch.float64), "m.norm": torch.ones(1, dtype=torch.float64),
         "m.o": torch.ones(1, 1, dtype=torch.float64)}
    # f = (sigmoid(0), 0.5 + 0.5 * sigmoid(-40)) = (0.5, 0.5): the floor alone holds the second channel up
    h = torch.tensor([[1.0, 2.0, 4.0], [3.0, -1.0, 8.0]], dtype=torch.float64)
    m = {"heads": 1, "dim": 2, "vdim": 1}
    # wide eps 0 is not allowed by the norm's root, so compare before the norm: o / rms(o) = sign(o) for one value
    out = plain.gated_recurrence(w, "m.", m, h, 1e-30)
    silu = lambda z: z / (1.0 + math.exp(-z))
    s1 = [0.5 * 4.0, 0.5 * 4.0]
    o1 = s1[0] * silu(1.0) + s1[1] * silu(2.0)
    s2 = [0.5 * s1[0] + 0.5 * 8.0, 0.5 * s1[1] + 0.5 * 8.0]
    o2 = s2[0] * silu(3.0) + s2[1] * silu(-1.0)
    assert out.tolist() == [[math.copysign(1.0, o1)], [math.copysign(1.0, o2)]]
    w["m.norm"] = torch.tensor([2.0], dtype=torch.float64)
    wide = plain.gated_recurrence(w, "m.", m, h, 9.0)            # o / sqrt(o^2 + 9) * 2
    assert abs(float(wide[1, 0]) - 2.0 * o2 / math.sqrt(o2 * o2 + 9.0)) < 1e-12
    assert abs(float(wide[0, 0]) - 2.0 * o1 / math.sqrt(o1 * o1 + 9.0)) < 1e-12


def test_plain_experts_by_hand():
    x = torch.tensor([[1.0, -2.0], [0.5, 3.0]], dtype=torch.float64)
    w = {"m.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, -1.0]], dtype=torch.float64)}
    for e in range(3):
        w[f"m.e{e}.up"] = torch.tensor([[1.0 + e, 0.0], [0.0, -1.0]], dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.tensor([[1.0, 1.0], [float(e), 0.0]], dtype=torch.float64)
    out = plain.routed_experts(w, "m.", {"router": {"experts": 3, "top": 2}}, x)

    def expert(e, v):
        a = [max((1.0 + e) * v[0], 0.0) ** 2, max(-v[1], 0.0) ** 2]
        return [a[0] + a[1], e * a[0]]
    # token 0: logits (1, -2, 1) -> experts 0 and 2 with equal shares; token 1: (0.5, 3, -3.5) -> 1 and 0
    want0 = [(expert(0, x[0].tolist())[c] + expert(2, x[0].tolist())[c]) / 2 for c in range(2)]
    a, b = math.exp(3.0), math.exp(0.5)
    want1 = [(a * expert(1, x[1].tolist())[c] + b * expert(0, x[1].tolist())[c]) / (a + b) for c in range(2)]
    assert all(abs(float(out[0, c]) - want0[c]) < 1e-12 and abs(float(out[1, c]) - want1[c]) < 1e-12 for c in range(2))


def single_layer(layer, width=32, vocab=61, side=None):
    cfg = {"architecture": "Pitudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


@pytest.mark.parametrize("kind", ["latent", "attention"])
def test_plain_logits_depend_on_the_window_only(kind):
    """One layer with a window of 6 (the token shift makes a position read one token more):
    changing token j changes the logits of j .. j + 6 and of nothing after."""
    layer = pitudra_models.latent(2, 8, 4, 8, 12, 10, window=6) if kind == "latent" else \
        pitudra_models.attention(2, 1, 8, vdim=4, window=6)
    cfg = single_layer(layer)
    w = pitudra_models.random_weights(cfg, 5)
    ids = helpers.random_requests(cfg["vocab"], [30], seed=2)["r0"]
    base = plain.forward(cfg, w, ids)
    other = list(ids)
    other[10] = (other[10] + 1) % cfg["vocab"]
    changed = plain.forward(cfg, w, other)
    assert float((changed[:10] - base[:10]).abs().max()) == 0.0
    assert float((changed[17:] - base[17:]).abs().max()) < 1e-12
    assert float((changed[16] - base[16]).abs().max()) > 1e-6        # through the shifted key at position 11
    assert float((changed[15] - base[15]).abs().max()) > 1e-6


# ------------------------------------------------------------------ the engine on the stand-in kernels
@pytest.mark.parametrize("name,page_size,lengths", [("P1", 4, [1, 30, 75]), ("P2", 16, [2, 40, 70]),
                                                    ("P4", 8, [3, 23, 66]), ("P5", 16, [5, 70]),
                                                    ("P6", 16, [2, 35, 66])])
def test_cutting_and_batching_on_cpu(tmp_path, name, page_size, lengths):
    cfg = pitudra_models.get(name)
    folder = pitudra_models.write_model(cfg, str(tmp_path / name), seed=11)
    reqs = helpers.random_requests(cfg["vocab"], lengths, seed=4)
    ref = pitudra_models.plain_logits(cfg, 11, reqs)
    runner = cpu_runner(folder, page_size, helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 12), "decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"pitudra {name} cpu {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    mixed_reqs = helpers.random_requests(cfg["vocab"], [20, 64, 9, 50, 33, 2], seed=8)
    mixed_ref = pitudra_models.plain_logits(cfg, 11, mixed_reqs)
    pool = 192
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6, decode_tail=5)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are reused
    runner2 = cpu_runner(folder, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL["float32"], f"pitudra {name} cpu mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


def test_token_by_token_from_the_first(tmp_path):
    """Every token alone, from position 0: the shift's and the recurrence's state start at
    zero in a slot that another request has just left, and the first windows fill up."""
    cfg = pitudra_models.get("P1")
    folder = pitudra_models.write_model(cfg, str(tmp_path / "p1"), seed=3)
    reqs = helpers.random_requests(cfg["vocab"], [45, 38], seed=6)
    ref = pitudra_models.plain_logits(cfg, 3, reqs)
    runner = cpu_runner(folder, 4, 64, max_requests=1)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 1000))
    helpers.assert_logits_close(got, ref, helpers.TOL["float32"], "pitudra P1 cpu token by token")


def test_a_reader_layer_holds_no_pages_of_its_own(tmp_path):
    cfg = pitudra_models.get("P1")
    folder = pitudra_models.write_model(cfg, str(tmp_path / "p1"), seed=2)
    runner = cpu_runner(folder, 4, 128)
    from chibillm_b200.cache.storage import PagedKVView
    paged = []
    for v in runner.storage.views:
        paged.append([m for m in (v if isinstance(v, tuple) else (v,)) if isinstance(m, PagedKVView)])
    assert [len(p) for p in paged] == [1, 0, 1, 1]                                 # the recurrence has no pages
    source, reader = paged[0][0], paged[3][0]
    assert (source.writes, paged[2][0].writes, reader.writes) == (True, True, False)
    assert reader.keys.data_ptr() == source.keys.data_ptr()
    assert source.values.data_ptr() == source.keys.data_ptr()                       # one row serves as key and value
    assert tuple(source.keys.shape[1:]) == (1, 4, 8 + 24)                           # rotated part | latent
    # the state slots: the shifted input of every layer, and one matrix per head of the recurrent layer
    shapes = sorted(tuple(t.shape[1:]) for v in runner.storage.state_views() for t in v.arrays.values())
    assert shapes.count((64,)) == 4 and (2, 24, 16) in shapes and len(shapes) == 5
    assert all(t.dtype == torch.float32 for v in runner.storage.state_views() for t in v.arrays.values())


def test_random_model_folder_of_the_package(tmp_path):
    """``write_random_model`` takes a Pitudra configuration; the folder runs and agrees
    with the plain implementation on the stored weights."""
    from chibillm_b200.weights import write_random_model
    from safetensors import safe_open
    cfg = pitudra_models.get("P4")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=2)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name)
    assert set(weights) == set(pitudra_models.random_weights(cfg, 0))
    reqs = helpers.random_requests(cfg["vocab"], [30], seed=1)
    ref = pitudra_models.plain_logits(cfg, 0, reqs, weights=weights)
    got = helpers.run_trace(cpu_runner(folder, 4, 64), helpers.trace_portions(reqs, seed=1))
    helpers.assert_logits_close(got, ref, helpers.TOL["float32"], "pitudra random folder")


def test_command_line_and_scheduler_on_cpu(tmp_path):
    """Four prompts through the package's command line with room for three at a time and
    portions of 8 tokens: every greedy token is the plain implementation's best one
    (wherever that leads by more than rounding)."""
    from chibillm_b200 import cli
    cfg = pitudra_models.get("P1")
    folder = pitudra_models.write_model(cfg, str(tmp_path / "p1"), seed=4)
    prompts = list(helpers.random_requests(cfg["vocab"], [1, 7, 23, 30], seed=1).values())
    argv = ["--context-length", "64", "--max-tokens", "5", "--max-seqs", "3", "--max-batch-tokens", "16",
            "--prefill-chunk", "8", "--dtype", "float32", "--ignore-eos", "--no-stream"]
    for p in prompts:
        argv += ["--prompt-ids", ",".join(map(str, p))]
    out, err = io.StringIO(), io.StringIO()
    assert cli.run(cli.parse_cli_options(argv + [folder]), io.StringIO(""), out, err,
                   kernels=ReferenceKernels(), device="cpu") == 0, err.getvalue()
    replies = [[int(t) for t in line.split()] for line in out.getvalue().splitlines()]
    assert len(replies) == 4 and all(len(r) == 5 for r in replies)
    for prompt, new in zip(prompts, replies):
        ref = pitudra_models.plain_logits(cfg, 4, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok
