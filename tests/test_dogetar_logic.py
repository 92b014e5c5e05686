"""Dogetar without a GPU: the configuration reader, the plain implementation's own consistency on
cases worked out by hand, and the engine's logic (batching, paging, state slots, the loop, the
bigram table's kept token, routed experts) on the plain PyTorch stand-ins of the kernels, against
the plain implementation of the design."""
import io
import math
import os

import pytest
import torch

import dogetar_models
import helpers
import plain_dogetar as plain
from reference_ops import ReferenceKernels


def cpu_runner(folder, page_size, pool_tokens, max_requests=4):
    from chibillm_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_folder(folder, dtype="float32", device="cpu", page_size=page_size,
                                     pool_tokens=pool_tokens, max_requests=max_requests,
                                     kernels=ReferenceKernels())
    runner.storage.poison()
    return runner


# ------------------------------------------------------------------ configuration
def test_parts_follow_the_file():
    from chibillm_b200.config import DogetarConfig
    spec = DogetarConfig.from_dict(dogetar_models.get("G1")).model_spec()
    assert [(s.layer, s.enter, s.turn) for s in spec.run_order] == [(0, 0, 0), (1, None, 0), (0, 0, 1), (1, None, 1),
                                                                     (2, None, 0)]
    par, diff, win = (l.mixer for l in spec.layers)
    assert par.kind == "parallel_mixers" and (par.left_scale, par.right_scale) == (0.7, 1.1)
    assert (par.left.chunk, par.left.window, par.left.sink, par.left.distance_bias) == (24, None, True, "linear")
    assert (par.right.state_size, par.right.groups, par.right.conv_taps, par.right.norm_groups) == (8, 2, 3, 1)
    assert (diff.query_maps, diff.differential, diff.head_gate, diff.chunk, diff.value_dim) == (2, 0.3, True, 20, 16)
    assert diff.position.rotary_dim == 4 and diff.position.wavelength_bands is None
    assert (win.window, win.chunk, win.biases, win.qk_norm.size) == (13, None, True, 12)
    assert win.position.wavelength_bands == (8.0, 1.0, 4.0, 64.0)
    ff = spec.layers[0].feed_forward
    assert (ff.num_experts, ff.identity_experts, ff.group_count, ff.group_keep, ff.weight_scale, ff.shared_size,
            ff.gated, ff.scores) == (6, 2, 2, 1, 1.5, 16, True, "softmax_all")
    assert spec.layers[1].feed_forward.activation == "swish_clamped" and spec.layers[1].feed_forward.limit == 2.0
    assert [a.kind for a in spec.input_adapters + spec.stream_adapters + spec.logit_adapters] == [
        "bigram", "reentry_add", "softcap"]
    bare = DogetarConfig.from_dict(dogetar_models.get("G2")).model_spec()
    assert not bare.input_adapters and not bare.stream_adapters and not bare.logit_adapters
    assert bare.layers[0].feed_forward is None and bare.layers[0].mixer.window is None
    assert bare.layers[0].mixer.num_kv_heads == 3 and bare.layers[0].mixer.position.kind == "none"
    assert bare.layers[2].mixer.right.groups == 1 and bare.layers[2].mixer.left_scale == 1.0


def test_config_errors_name_the_key():
    from chibillm_b200.config import ConfigError, DogetarConfig

    def read(change):
        cfg = dogetar_models.get("G1")
        change(cfg)
        return DogetarConfig.from_dict(cfg)

    for change, word in ((lambda c: c.pop("width"), "width"),
                         (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
                         (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=13), "rot.dims"),
                         (lambda c: c["layers"][0].update(type="conv"), "type"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
                         (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
                         (lambda c: c["loop"].update(stop=9), "loop"),
                         (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
                         (lambda c: c["layers"][0]["mixer"]["right"].update(groups=3), "groups")):
        with pytest.raises(ConfigError) as e:
            read(change)
        assert word in str(e.value)


# ------------------------------------------------------------------ the plain implementation, by hand
def test_plain_bigram_rows_and_bands_by_hand():
    cfg = {"buckets": 10, "mul_prev": 3, "mul_cur": 7}
    assert plain.bigram_rows([4, 9, 0, 5], cfg) == [10, (4 * 3 + 9 * 7) % 10, (9 * 3) % 10, 35 % 10]
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40.0}}
    plain_f = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    got = plain.rotary_frequencies(rot)
    # wavelengths 6.3, 19.9, 62.8, 198.7 against the borders 10 and 40: kept, blended, divided, divided
    assert got[0] == plain_f[0] and got[2] == plain_f[2] / 4 and got[3] == plain_f[3] / 4
    s = (40.0 / (2 * math.pi / plain_f[1]) - 1.0) / 3.0
    assert abs(got[1] - ((1 - s) * plain_f[1] / 4 + s * plain_f[1])) < 1e-15 and plain_f[1] / 4 < got[1] < plain_f[1]


def test_plain_masks_sink_and_bias_by_hand():
    m = plain.visible(9, window=3)
    assert m[5].tolist() == [False] * 3 + [True] * 3 + [False] * 3
    m = plain.visible(9, chunk=4)
    assert m[5].tolist() == [False] * 4 + [True, True] + [False] * 3 and m[4].tolist() == [False] * 4 + [True] + [False] * 4
    # one key, score 0, sink 0: the weight of the key is one half
    q = torch.zeros(1, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[3.0, 5.0]]], dtype=torch.float64)
    out = plain.softmax_attention(q, q, v, 1.0, plain.visible(1), sink=torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(out, v / 2)
    # the distance bias: with equal scores the weights fall by exp(-slope) per position
    T = 4
    q = torch.zeros(T, 2, 2, dtype=torch.float64)
    slopes = plain.distance_slopes(2, torch.float64)
    assert torch.allclose(slopes, torch.tensor([2.0 ** -4, 2.0 ** -8], dtype=torch.float64))
    i = torch.arange(T, dtype=torch.float64)
    bias = slopes[:, None, None] * (i[:, None] - i[None, :])[None]
    vals = torch.eye(T, dtype=torch.float64)[:, None, :]
    out = plain.softmax_attention(q, q[:, :1], vals, 1.0, plain.visible(T), bias=bias)
    wts = out[3, 0]
    assert torch.allclose(wts[:-1] / wts[1:], torch.full((3,), math.exp(-2.0 ** -4), dtype=torch.float64))


def test_plain_router_by_hand():
    # six outputs in three groups of two, two groups kept, top 3; the last two outputs are identity experts
    mlp = {"router": {"experts": 4, "identity": 2, "top": 3, "scale": 2.0, "groups": {"count": 3, "keep": 2}}}
    z = torch.log(torch.tensor([[0.05, 0.30, 0.20, 0.10, 0.25, 0.10]], dtype=torch.float64))
    w = {"r.router": torch.eye(6, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, -0.2, 0.17],
                                                                                    dtype=torch.float64)}
    chosen, weight = plain.route(z, mlp, w, "r.")
    # choice scores .05 .30 | .20 .10 | .05 .27: groups 0 and 2 stay; of .05 .30 .05 .27 the best three
    assert chosen.tolist() == [[1, 5, 0]] or chosen.tolist() == [[1, 5, 4]]
    assert torch.allclose(weight[0, :2], torch.tensor([0.60, 0.20], dtype=torch.float64))
    h = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], dtype=torch.float64)
    w.update({f"r.e{e}.{n}": torch.zeros(6, 6, dtype=torch.float64) for e in range(4) for n in ("gate", "up", "down")})
    w["r.router"] = torch.zeros(6, 6, dtype=torch.float64)        # equal scores: the corrections decide
    out = plain.moe_ff(h, {"router": {"experts": 4, "identity": 2, "top": 1, "scale": 3.0}}, w, "r.")
    assert torch.allclose(out, 3.0 / 6 * h)                       # the identity expert 5: its input times its weight


def test_plain_state_space_and_convolution_by_hand():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    y = plain.causal_conv(x, torch.tensor([[0.5, 1.0, 2.0]], dtype=torch.float64), torch.tensor([0.25], dtype=torch.float64))
    assert y.flatten().tolist() == [2.25, 5.25, 10.75]
    dt = torch.tensor([[0.5], [1.0]], dtype=torch.float64)
    xs = torch.tensor([[[2.0]], [[3.0]]], dtype=torch.float64)
    B = torch.tensor([[[1.0, 0.0]], [[1.0, 1.0]]], dtype=torch.float64)
    C = torch.tensor([[[1.0, 1.0]], [[1.0, 2.0]]], dtype=torch.float64)
    yy, S = plain.state_space_scan(xs, B, C, dt, torch.zeros(1, dtype=torch.float64), torch.tensor([10.0], dtype=torch.float64))
    # S1 = .5 * 2 * [1, 0]; y1 = 1 + 20;  S2 = e^-1 [1, 0] + 3 [1, 1]; y2 = (e^-1 + 3) + 2 * 3 + 30
    assert abs(float(yy[0, 0, 0]) - 21.0) < 1e-12 and abs(float(yy[1, 0, 0]) - (math.exp(-1) + 39.0)) < 1e-12
    assert torch.allclose(S[0, :, 0], torch.tensor([math.exp(-1) + 3.0, 3.0], dtype=torch.float64))


def test_plain_logits_depend_on_window_and_block_only():
    """A token outside every window and block of a later position cannot change it, one inside can (one layer
    of each kind, no state-space branch in the way: the left branch's scale alone)."""
    for layer, reach in ((dogetar_models.windowed(2, 1, 8, 6, window=5, rot=4), lambda p: p - 4),
                         (dogetar_models.differential(2, 1, 8, 6, chunk=6, rot=8), lambda p: p - p % 6)):
        cfg = {"architecture": "Dogetar", "vocab": 50, "width": 16, "norm": {"eps": 1e-5}, "layers": [layer]}
        w = {k: v.double() for k, v in dogetar_models.random_weights(cfg, 5).items()}
        ids = torch.arange(3, 23)
        base = plain.forward(ids, cfg, w)
        for p in (9, 17):
            first = reach(p)
            changed = ids.clone()
            changed[first - 1] = 49
            assert float((plain.forward(changed, cfg, w)[p] - base[p]).abs().max()) < 1e-12
            changed = ids.clone()
            changed[first] = 49
            assert float((plain.forward(changed, cfg, w)[p] - base[p]).abs().max()) > 1e-6


# ------------------------------------------------------------------ the engine on the stand-in kernels
@pytest.mark.parametrize("name,page_size,lengths", [("G1", 4, [1, 30, 75]), ("G2", 16, [2, 40, 70]),
                                                    ("G3", 16, [5, 70]), ("G4", 8, [3, 23, 66])])
def test_cutting_and_batching_on_cpu(tmp_path, name, page_size, lengths):
    cfg = dogetar_models.get(name)
    folder = dogetar_models.write_model(cfg, str(tmp_path / name), seed=11)
    reqs = helpers.random_requests(cfg["vocab"], lengths, seed=4)
    ref = dogetar_models.plain_logits(cfg, 11, reqs)
    runner = cpu_runner(folder, page_size, helpers.round64(max(lengths)))
    for trace, what in ((helpers.trace_whole(reqs), "whole"), (helpers.trace_last_decoded(reqs, 12), "decoded"),
                        (helpers.trace_portions(reqs, seed=2), "portions")):
        got = helpers.run_trace(runner, trace)
        helpers.assert_logits_close(got, ref, helpers.TOL["float32"], f"dogetar {name} cpu {what}")
        runner.cache.check_invariants()
        assert not runner.cache.requests
    mixed_reqs = helpers.random_requests(cfg["vocab"], [20, 64, 9, 50, 33, 2], seed=8)
    mixed_ref = dogetar_models.plain_logits(cfg, 11, mixed_reqs)
    pool = 192
    trace = helpers.trace_mixed(mixed_reqs, pool, seed=6, decode_tail=5)
    assert sum(helpers.round64(len(v)) for v in mixed_reqs.values()) > pool       # pages and slots are reused
    runner2 = cpu_runner(folder, page_size, pool)
    got = helpers.run_trace(runner2, trace)
    helpers.assert_logits_close(got, mixed_ref, helpers.TOL["float32"], f"dogetar {name} cpu mixed")
    runner2.cache.check_invariants()
    assert not runner2.cache.requests


def test_token_by_token_from_the_first(tmp_path):
    """Every token alone, from position 0: the kept token, the convolution's history and the scan's state start
    at zero in a slot that another request has just left, and the first windows and blocks fill up."""
    cfg = dogetar_models.get("G4")
    folder = dogetar_models.write_model(cfg, str(tmp_path / "g4"), seed=3)
    reqs = helpers.random_requests(cfg["vocab"], [45, 38], seed=6)
    ref = dogetar_models.plain_logits(cfg, 3, reqs)
    runner = cpu_runner(folder, 4, 64, max_requests=1)
    got = helpers.run_trace(runner, helpers.trace_last_decoded(reqs, 1000))
    helpers.assert_logits_close(got, ref, helpers.TOL["float32"], "dogetar G4 cpu token by token")


def test_cache_plan_and_state(tmp_path):
    cfg = dogetar_models.get("G1")
    folder = dogetar_models.write_model(cfg, str(tmp_path / "g1"), seed=2)
    runner = cpu_runner(folder, 4, 128)
    from chibillm_b200.cache.storage import FixedStateView, PagedKVView
    views = runner.storage.views
    assert len(views) == 5 + 1                                   # five layer runs and the bigram table's kept token
    # the looped layers have a cache of their own in every pass
    assert views[0][0].keys.data_ptr() != views[2][0].keys.data_ptr()
    assert views[0][1].arrays["state"].data_ptr() != views[2][1].arrays["state"].data_ptr()
    par = views[0]
    assert isinstance(par[0], PagedKVView) and isinstance(par[1], FixedStateView)
    assert tuple(par[1].arrays["state"].shape[1:]) == (4, 12, 8) and par[1].arrays["state"].dtype == torch.float32
    assert tuple(par[1].arrays["history"].shape[1:]) == (2, 4 * 12 + 2 * 2 * 8)
    diff = views[1]
    assert tuple(diff.keys.shape[1:]) == (2 * 2, 4, 8) and tuple(diff.values.shape[1:]) == (2, 4, 16)
    assert tuple(views[5].arrays["last_token"].shape[1:]) == (1,) and views[5].arrays["last_token"].dtype == torch.int32


def test_a_step_taken_back_leaves_no_trace(tmp_path):
    """A provisional step that is rolled back: the kept token, the history and the state go back too."""
    from chibillm_b200.engine.batch import StepEntry
    cfg = dogetar_models.get("G1")
    folder = dogetar_models.write_model(cfg, str(tmp_path / "g1"), seed=5)
    ids = helpers.random_requests(cfg["vocab"], [21], seed=2)["r0"]
    ref = dogetar_models.plain_logits(cfg, 5, {"a": ids})["a"]
    runner = cpu_runner(folder, 4, 64)
    runner.step([StepEntry("a", ids[:9], [])])
    runner.step([StepEntry("a", [7, 7, 7, 7, 7], [4])], provisional=True)
    runner.rollback_step()
    got = runner.step([StepEntry("a", ids[9:], list(range(len(ids) - 9)))])
    helpers.assert_logits_close({"a": got}, {"a": ref[9:]}, helpers.TOL["float32"], "dogetar rollback")


def test_random_model_folder_of_the_package(tmp_path):
    """``write_random_model`` takes a Dogetar configuration; the folder runs and agrees with the plain
    implementation on the stored weights."""
    from chibillm_b200.weights import write_random_model
    from safetensors import safe_open
    cfg = dogetar_models.get("G4")
    folder = write_random_model(cfg, str(tmp_path / "random"), seed=2)
    weights = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name)
    assert set(weights) == set(dogetar_models.random_weights(cfg, 0))
    reqs = helpers.random_requests(cfg["vocab"], [30], seed=1)
    ref = dogetar_models.plain_logits(cfg, 0, reqs, weights=weights)
    got = helpers.run_trace(cpu_runner(folder, 4, 64), helpers.trace_portions(reqs, seed=1))
    helpers.assert_logits_close(got, ref, helpers.TOL["float32"], "dogetar random folder")


def test_command_line_and_scheduler_on_cpu(tmp_path):
    """Four prompts through the package's command line with room for three at a time and portions of 8
    tokens: every greedy token is the plain implementation's best one (wherever that leads by more than
    rounding)."""
    from chibillm_b200 import cli
    cfg = dogetar_models.get("G1")
    folder = dogetar_models.write_model(cfg, str(tmp_path / "g1"), seed=4)
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
        ref = dogetar_models.plain_logits(cfg, 4, {"a": prompt + new})["a"]
        for i, tok in enumerate(new):
            row = ref[len(prompt) + i - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(torch.argmax(row)) == tok
