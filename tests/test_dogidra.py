"""Dogidra without a GPU: its configuration, what the model asks of the weights and of the cache, and the plain
implementation against itself (a prompt whole, in portions and token by token through the explicit caches and
states) and on values worked by hand."""

import copy
import math

import pytest
import torch

import plain_dogidra as plain
from dogidra_models import CONFIGS, DOGIDRA_X, DOGIDRA_Y, DOGIDRA_Z, make_folder, tensor_shapes

F64 = plain.F64


def model_of(config):
    from qwen3_from_scratch_b200.engine.model import Model
    from qwen3_from_scratch_b200.registry import build_model_spec, config_from_dict
    return Model(build_model_spec(config_from_dict(config)))


@pytest.mark.parametrize("key", list(CONFIGS))
def test_the_model_asks_for_the_tensors_the_design_names(key):
    config = CONFIGS[key][0]
    asked = {s.name: tuple(s.shape) for s in model_of(config).weight_specs()}
    assert asked == tensor_shapes(config)


def test_configuration_round_trip():
    from qwen3_from_scratch_b200.registry import config_from_dict
    cfg = config_from_dict(DOGIDRA_X)
    assert cfg.architecture == "Dogidra" and cfg.loop == (1, 3, 3) and cfg.taps == 4 and cfg.embedding_scale == 3.0
    first, second = cfg.layers[0], cfg.layers[1]
    assert (first.left.heads, first.left.kv_heads, first.left.dim, first.left.vdim) == (4, 2, 24, 40)
    assert (first.left.window, first.left.pool, first.left.softcap) == (9, 4, 5.0)
    assert first.left.rot_scaling.factor == 4.0 and second.left.rot_scaling is None and second.left.softcap is None
    assert second.mlp is None and first.mlp.shared_ff == 40 and cfg.layers[2].mlp.shared_ff is None
    assert (first.left_scale, first.right_scale, first.right_width) == (0.7, 1.2, 72)
    assert config_from_dict(cfg.to_dict()) == cfg
    y = config_from_dict(DOGIDRA_Y)
    assert y.loop is None and config_from_dict(y.to_dict()) == y


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="hyena"), "not built"),
    (lambda c: c["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "moe"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("pool"), "pool"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=17), "dims"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["canon"].pop("taps"), "taps"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, message):
    from qwen3_from_scratch_b200.config.model_config import ConfigError
    from qwen3_from_scratch_b200.registry import config_from_dict
    config = copy.deepcopy(DOGIDRA_X)
    change(config)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_run_order_and_cache_needs():
    """The looped span becomes further runs of the same layers, each with a cache id of its own.  An attention run
    keeps token pages, of which only those the window (or a block that is still open) touches stay, and block pages
    with one entry per ``pool`` tokens; the recurrence keeps a float32 state, the two convolutions their tails."""
    from qwen3_from_scratch_b200.parts.base import StateSpec
    model = model_of(DOGIDRA_X)
    assert [c.layer for c in model.spec.order] == [0, 1, 2, 1, 2, 1, 2, 3] == plain.run_order(DOGIDRA_X)
    assert [c.cache for c in model.spec.order] == list(range(8))
    layout = model.cache_layout()
    groups = {tuple((p.name, p.heads, p.width) for p in g.spec.planes): (g.cache_ids, g.spec.window, g.spec.entry_tokens)
              for g in layout.groups}
    assert groups[(("k", 2, 16), ("v", 2, 8))] == ([(1, "left"), (3, "left"), (5, "left")], 7, 1)  # a block of 7 > window 5
    assert groups[(("pk", 2, 16), ("pv", 2, 8))] == ([(1, "left.pooled"), (3, "left.pooled"), (5, "left.pooled")], None, 7)
    assert groups[(("k", 2, 24), ("v", 2, 40))] == ([(0, "left")], 9, 1)
    assert layout.states[(0, "right")] == StateSpec((72,), "float32") and layout.states[(5, "right")] == StateSpec((40,), "float32")
    assert layout.states[(0, "conv1")] == StateSpec((3, 64), "float32") == layout.states[(0, "conv2")]
    assert (1, "conv2") not in layout.states and (1, "conv1") in layout.states  # a layer without feed-forward
    assert not any(k[1].startswith("conv") for k in model_of(DOGIDRA_Y).cache_layout().states)  # a single tap keeps nothing
    assert len(model.layers) == 4


def test_random_model_folder_through_the_framework_writer(tmp_path):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(DOGIDRA_Y), seed=1)
    cfg, w = plain.read_model_folder(folder)
    assert {k: tuple(v.shape) for k, v in w.items()} == tensor_shapes(DOGIDRA_Y)
    assert torch.isfinite(plain.forward_logits(cfg, w, [3, 1, 4, 1, 5])).all()


@pytest.mark.parametrize("key", ["x", "y"])
def test_plain_whole_prompt_equals_plain_in_portions_and_token_by_token(tmp_path, key):
    config, seed = CONFIGS[key]
    cfg, w = plain.read_model_folder(make_folder(str(tmp_path / key), config, seed))
    ids = torch.randint(0, cfg["vocab"], (37,), generator=torch.Generator().manual_seed(5)).tolist()
    whole = plain.forward_logits(cfg, w, ids)
    state, rows = plain.new_state(cfg), []
    for cut in ([ids[:9], ids[9:11], ids[11:24]] + [[t] for t in ids[24:]]):
        rows.append(plain.forward(cfg, w, cut, state))
    assert float((torch.cat(rows) - whole).abs().max()) < 1e-9 * float(whole.abs().max())


def test_what_a_position_reads():
    # window 5, blocks of 3: position 9 reads 5..9; block b is read once its last token is at or before 9 - 5 = 4
    assert plain.visible(9, 5, 3) == ([5, 6, 7, 8, 9], [0])            # block 1 (3..5) ends at 5 > 4: token 3, 4 unseen
    assert plain.visible(10, 5, 3) == ([6, 7, 8, 9, 10], [0, 1])       # ... and is read one token later
    assert plain.visible(4, 5, 3) == ([0, 1, 2, 3, 4], [])
    assert plain.visible(7, 5, 3) == ([3, 4, 5, 6, 7], [0])            # block 0 ends at 2 = 7 - 5
    assert plain.visible(6, 5, 3) == ([2, 3, 4, 5, 6], [])             # token 0 and 1 are unseen here
    assert plain.visible(3, 1, 1) == ([3], [0, 1, 2])                  # blocks of one token: everything is read
    assert plain.visible(6, 2, 7) == ([5, 6], [])                      # a block longer than the window, still open
    assert plain.visible(8, 2, 7) == ([7, 8], [0])


def test_plain_mechanisms_on_values_worked_by_hand():
    t = lambda *v: torch.tensor(v, dtype=F64)  # noqa: E731
    # layer norm: mean 2, variance 2/3
    out = plain.layer_norm(t([1.0, 2.0, 3.0]), t(2.0, 2.0, 2.0), t(0.5, 0.5, 0.5), 0.0)
    assert torch.allclose(out, t(0.5 - 2 * math.sqrt(1.5), 0.5, 0.5 + 2 * math.sqrt(1.5)))
    # the convolution adds to its input; the last column multiplies the current token; the tail is carried
    y, tail = plain.input_conv(t([1.0], [2.0], [3.0]), t([100.0, 10.0, 1.0]), torch.zeros(2, 1, dtype=F64))
    assert y[:, 0].tolist() == [2.0, 14.0, 126.0] and tail[:, 0].tolist() == [2.0, 3.0]
    y2, _ = plain.input_conv(t([4.0]), t([100.0, 10.0, 1.0]), tail)
    assert y2[0, 0].item() == 4.0 + 234.0
    # stretched frequencies: pair(10) = 0, pair(1) = 8 ln 10 / (2 ln 100) = 2: ramp 0, 0.5, 1, 1
    f, mag = plain.stretched_frequencies({"dims": 8, "base": 100.0})
    assert mag == 1.0 and torch.allclose(f, t(1.0, 100 ** -0.25, 0.1, 100 ** -0.75))
    f2, mag2 = plain.stretched_frequencies({"dims": 8, "base": 100.0, "scaling": {
        "factor": 4.0, "original": 2 * math.pi * 10, "fast": 10.0, "slow": 1.0}})
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-12 and torch.allclose(f2, f * t(1.0, 0.625, 0.25, 0.25))
    # rotation of the pair (i, i + dims / 2), the rest passing
    x = t([[1.0, 0.0, 0.0, 1.0, 7.0]])[None]
    rot = {"dims": 4, "base": 1.0}  # base 1: every frequency is 1
    out = plain.rotate(x, [math.pi / 2], rot)
    assert torch.allclose(out, t([[[0.0, -1.0, 1.0, 0.0, 7.0]]]), atol=1e-12)
    # the recurrence: z = 1/2 everywhere; candidates 1.5 (u = 1) and sigmoid(-1); gate silu(0) = 0 kills the output
    w = {"z": torch.zeros(1, 1, dtype=F64), "z.b": t(0.0), "x": t([1.0]), "x.b": t(0.0), "g": t([1.0]), "o": t([1.0])}
    out, s = plain.min_gru(t([1.0], [-1.0]), w, "", t(0.0))
    s1 = 0.75
    s2 = 0.5 * s1 + 0.5 / (1 + math.e)
    assert abs(float(s) - s2) < 1e-12
    assert torch.allclose(out[:, 0], t(s1 / (1 + math.exp(-1.0)), -s2 / (1 + math.e)))
    # the router: the correction changes who is chosen, not the weights; weights are not renormalised
    mlp = {"router": {"experts": 3, "top": 1, "scale": 2.0}, "expert": {"ff": 1}}
    w = {"router": t([0.0], [1.0], [2.0]), "correction": t(1.0, 0.0, 0.0)}
    for e, up in enumerate((1.0, 10.0, 100.0)):
        w[f"e{e}.up"], w[f"e{e}.down"] = t([up]), t([1.0])
    # h = 1: scores 0.5, 0.73, 0.88; with the correction expert 0 wins (1.5); its weight is 0.5 * 2, its output relu(1)^2
    assert torch.allclose(plain.routed_experts(t([1.0]), w, "", mlp), t([1.0]))
    w["correction"] = t(0.0, 0.0, 0.0)
    assert torch.allclose(plain.routed_experts(t([1.0]), w, "", mlp), t([2.0 / (1 + math.exp(-2.0)) * 100.0 ** 2]))
    assert torch.allclose(plain.routed_experts(t([-1.0]), w, "", mlp), t([0.0]))  # relu


def test_pooled_blocks_and_tokens_share_one_softmax():
    """One head, keys and values chosen by hand: with a zero query every visible key weighs the same, so the output is
    the mean of the visible values, a block counting once with the mean of its values."""
    m = {"heads": 1, "kv_heads": 1, "mask": {"size": 2, "pool": 2}, "scale": 1.0}
    values = torch.tensor([1.0, 3.0, 10.0, 20.0, 100.0, 200.0], dtype=F64).view(6, 1, 1)
    keys = torch.zeros(6, 1, 4, dtype=F64)
    q = torch.zeros(1, 1, 4, dtype=F64)
    out = plain.windowed_pooled_attention(q, keys, values, [5], m)     # tokens 4, 5; blocks 0 (ends 1) and 1 (ends 3 = 5 - 2)
    assert abs(float(out) - (100.0 + 200.0 + 2.0 + 15.0) / 4) < 1e-12
    out = plain.windowed_pooled_attention(q, keys[:5], values[:5], [4], m)   # tokens 3, 4; block 0; token 2 unseen
    assert abs(float(out) - (20.0 + 100.0 + 2.0) / 3) < 1e-12
    # a cap bounds the scores: a huge score and one half its size weigh nearly the same under a cap of 1
    m2 = dict(m, softcap=1.0, mask={"size": 2, "pool": 9})
    keys2 = torch.tensor([[50.0], [100.0]], dtype=F64).view(2, 1, 1)
    out = plain.windowed_pooled_attention(torch.ones(1, 1, 1, dtype=F64), keys2, values[:2], [1], m2)
    assert abs(float(out) - 2.0) < 1e-6
