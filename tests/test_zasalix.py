"""Zasalix without a GPU: its configuration, what the model asks of the weights and of the cache, the cache manager
with a window that keeps a request's first tokens, and the plain implementation against itself (a prompt whole, in
portions and token by token through the explicit caches and states) and on values worked by hand."""

import copy
import math

import pytest
import torch

import plain_zasalix as plain
from zasalix_models import CONFIGS, ZASALIX_X, ZASALIX_Y, ZASALIX_Z, make_folder, tensor_shapes

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
    cfg = config_from_dict(ZASALIX_X)
    assert cfg.architecture == "Zasalix" and cfg.loop == (1, 3, 3) and cfg.side_dim == 8 and cfg.norm_eps == 1e-5
    first, second, third = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert (first.type, first.mixer.heads, first.mixer.rot_dim, first.mixer.rot_dims, first.mixer.kv_rank) == (
        "latent_attention", 4, 8, 4, 48)
    left = second.mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.window, left.keep_first) == (4, 2, 24, 40, 9, 4)
    assert (second.mixer.left_scale, second.mixer.right_scale, second.mixer.right.gate_cap) == (0.7, 1.2, 8.0)
    assert third.type == "mlstm" and third.mlp is None and second.mlp.ff == 96
    assert (first.mlp.experts, first.mlp.top, first.mlp.shared_ff) == (5, 2, 40) and cfg.layers[3].mlp.shared_ff is None
    assert config_from_dict(cfg.to_dict()) == cfg and cfg.to_dict() == ZASALIX_X
    y = config_from_dict(ZASALIX_Y)
    assert y.loop is None and y.side_dim is None and config_from_dict(y.to_dict()) == y


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0].update(type="hyena"), "not built"),
    (lambda c: c["layers"][0].update(mlp={"kind": "glu", "ff": 8}), "dense"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["left"]["mask"].pop("keep_first"), "keep_first"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=26), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_configuration_errors_name_the_key(change, message):
    from qwen3_from_scratch_b200.config.model_config import ConfigError
    from qwen3_from_scratch_b200.registry import config_from_dict
    config = copy.deepcopy(ZASALIX_X)
    change(config)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(config)


def test_run_order_and_cache_needs():
    """The looped span becomes further runs of the same layers, each with a cache id of its own and the number of its
    pass.  A latent attention keeps pages of latents, a windowed one pages of keys and values of which the window's and
    the first tokens' stay, a matrix memory three float32 states."""
    from qwen3_from_scratch_b200.parts.base import StateSpec
    model = model_of(ZASALIX_X)
    assert [c.layer for c in model.spec.order] == [0, 1, 2, 1, 2, 1, 2, 3, 4] == plain.run_order(ZASALIX_X)
    assert [c.cache for c in model.spec.order] == list(range(9))
    assert [c.repeat for c in model.spec.order] == [0, 0, 0, 1, 1, 2, 2, 0, 0]
    layout = model.cache_layout()
    groups = {tuple((p.name, p.heads, p.width) for p in g.spec.planes): (g.cache_ids, g.spec.window, g.spec.keep_first)
              for g in layout.groups}
    assert groups[(("c", 1, 48), ("r", 1, 8))] == ([0], None, 0)
    assert groups[(("c", 1, 24), ("r", 1, 16))] == ([8], None, 0)
    assert groups[(("k", 2, 24), ("v", 2, 40))] == ([(1, "left"), (3, "left"), (5, "left")], 9, 4)
    assert groups[(("k", 2, 16), ("v", 2, 8))] == ([(7, "left")], 5, 7)
    assert layout.states[(2, "memory")] == StateSpec((2, 24, 40), "float32")  # kept column by column: [heads, vdim, dim]
    assert layout.states[(1, "right.normaliser")] == StateSpec((3, 16), "float32")
    assert layout.states[(5, "right.maximum")] == StateSpec((3,), "float32")


def test_a_window_that_keeps_the_first_tokens_keeps_their_pages():
    """Pages that the window has passed go back to the pool, except those with one of the first ``keep_first`` tokens;
    a page given back is handed out again; everything returns when the request ends."""
    from qwen3_from_scratch_b200.cache.manager import CacheManager, layout_of
    from qwen3_from_scratch_b200.parts.base import CachePlane, PagedCacheSpec
    spec = PagedCacheSpec((CachePlane("k", 1, 8), CachePlane("v", 1, 8)), window=6, keep_first=5)
    m = CacheManager(layout_of({0: spec}), page_size=4, num_pages=9, max_seqs=2)
    m.open("a")
    for length in range(1, 30):
        m.reserve("a", length)
        m.advance("a", length)
        table = m.table(0, "a")
        first_read = max(0, length - 6 + 1)  # a query at position >= length reads from here on, and 0 .. 4
        for page, entry in enumerate(table):
            needed = page * 4 < 5 or (page + 1) * 4 > first_read
            assert (entry >= 0) == needed, (length, page, table)
        m.check()
    assert m.free_pages(0) == 9 - sum(1 for e in m.table(0, "a") if e >= 0) == 9 - 4
    m.open("b")
    m.reserve("b", 20)  # takes pages that "a" gave back
    m.check()
    m.close("a"), m.close("b")
    assert m.free_pages(0) == 9 and m.free_slots() == 2
    # without kept tokens the first pages go like the others
    plain_window = PagedCacheSpec((CachePlane("k", 1, 8),), window=6)
    m = CacheManager(layout_of({0: plain_window}), page_size=4, num_pages=9, max_seqs=1)
    m.open("a"), m.reserve("a", 29), m.advance("a", 29)
    assert m.table(0, "a")[:5] == [-1] * 5


def test_random_model_folder_through_the_framework_writer(tmp_path):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config_from_dict(ZASALIX_Z), seed=1)
    config, w = plain.read_model_folder(folder)
    assert {k: tuple(v.shape) for k, v in w.items()} == tensor_shapes(ZASALIX_Z)
    logits = plain.forward_logits(config, w, [5, 17, 3, 250, 9])
    assert logits.shape == (5, 300) and torch.isfinite(logits).all()


@pytest.mark.parametrize("key", list(CONFIGS))
def test_plain_whole_prompt_equals_plain_in_portions_and_token_by_token(tmp_path, key):
    config, seed = CONFIGS[key]
    cfg, w = plain.read_model_folder(make_folder(str(tmp_path / key), config, seed))
    ids = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(7)).tolist()
    whole = plain.forward_logits(cfg, w, ids)
    for cuts in ([30, 2, 1, 37], [1] * 70, [2] * 35):
        state, rows, at = plain.new_state(cfg), [], 0
        for c in cuts:
            rows.append(plain.forward(cfg, w, ids[at:at + c], state))
            at += c
        assert float((torch.cat(rows) - whole).abs().max()) < 1e-9 * float(whole.abs().max())


def test_plain_mechanisms_on_values_worked_by_hand():
    # the norm without statistics
    w = {"n": torch.tensor([2.0, 0.5], dtype=F64), "n.b": torch.tensor([0.1, -0.1], dtype=F64), "n.alpha": torch.tensor(0.5, dtype=F64)}
    got = plain.dynamic_tanh(torch.tensor([[1.0, -2.0]], dtype=F64), w, "n")
    assert torch.allclose(got, torch.tensor([[2 * math.tanh(0.5) + 0.1, 0.5 * math.tanh(-1.0) - 0.1]], dtype=F64))
    # neighbours turn together, halves turn together: a quarter turn at position 1 with base chosen so that f_0 = pi / 2
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=F64)
    half_pi = math.pi / 2
    n = plain.rotate_neighbours(v * 1.0, [1], 1.0, 2)  # dims 2: one pair, f_0 = 1; angle 1
    assert torch.allclose(n[0, 0, :2], torch.tensor([math.cos(1) - 2 * math.sin(1), 2 * math.cos(1) + math.sin(1)], dtype=F64))
    assert torch.equal(n[0, 0, 2:], v[0, 0, 2:])
    h = plain.rotate_halves(v * 1.0, [1], (1 / half_pi) ** 2, 4)  # f_0 = 1, f_1 = base^(-1/2) = pi / 2: a quarter turn
    assert torch.allclose(h[0, 0, 1], torch.tensor(-4.0, dtype=F64)) and torch.allclose(h[0, 0, 3], torch.tensor(2.0, dtype=F64))
    assert torch.allclose(h[0, 0, 0], torch.tensor(math.cos(1) - 3 * math.sin(1), dtype=F64)) and h[0, 0, 4] == 5.0
    # position 0 is never turned
    assert torch.equal(plain.rotate_neighbours(v * 1.0, [0], 100.0, 4), v)


def test_the_matrix_memory_by_hand():
    """One head, keys and values of one number: the recurrence written out for three tokens."""
    W = 2
    w = {k: torch.zeros(1, W, dtype=F64) for k in ("q", "k", "v", "g", "i", "f")}
    w["q"][0, 0] = w["k"][0, 0] = w["v"][0, 1] = 1.0
    w["i"][0, 0], w["f"][0, 1] = 1.0, 1.0
    w.update({"i.b": torch.tensor([0.5], dtype=F64), "f.b": torch.tensor([-0.2], dtype=F64), "norm": torch.tensor([3.0], dtype=F64),
              "o": torch.tensor([[1.0], [0.0]], dtype=F64)})
    m = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 2.0}
    h = torch.tensor([[1.0, 2.0], [-1.0, 0.5], [2.0, -3.0]], dtype=F64)
    st = {"S": torch.zeros(1, 1, 1, dtype=F64), "n": torch.zeros(1, 1, dtype=F64), "m": torch.zeros(1, dtype=F64)}
    got = plain.matrix_memory(h, w, "", m, 1e-6, st)
    S = n = mx = 0.0
    want = []
    for a, b in h.tolist():
        q, k, v = a, a, b
        i = 2 * math.tanh((a + 0.5) / 2)
        f = 2 * math.tanh((b - 0.2) / 2)
        f = -math.log1p(math.exp(-f))
        new = max(f + mx, i)
        S = math.exp(f + mx - new) * S + math.exp(i - new) * k * v
        n = math.exp(f + mx - new) * n + math.exp(i - new) * k
        mx = new
        o = S * q / (max(abs(n * q), math.exp(-mx)) + 1e-6)
        want.append(o / math.sqrt(o * o + 1e-6) * 3.0 * 0.5)  # unit rms of one value, the weight, sigmoid(0)
    assert torch.allclose(got[:, 0], torch.tensor(want, dtype=F64), atol=1e-12) and float(got[:, 1].abs().max()) == 0
    assert abs(float(st["m"]) - mx) < 1e-12 and abs(float(st["S"]) - S) < 1e-12


def test_what_a_windowed_query_reads_and_what_the_sink_takes():
    """All keys equal, values that name their position: the output is the mean of the positions read, so one key too
    many or too few shows; in the latent attention the sink takes its share of the weight and gives nothing."""
    W, n = 4, 12
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "mask": {"size": 3, "keep_first": 2},
         "rot": {"base": 10.0, "dims": 0}}
    w = {"q": torch.zeros(2, W, dtype=F64), "k": torch.zeros(2, W, dtype=F64), "v": torch.zeros(1, W, dtype=F64),
         "g": torch.zeros(1, W, dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    w["v"][0, 0] = 1.0
    h = torch.zeros(n, W, dtype=F64)
    h[:, 0] = torch.arange(n, dtype=F64)
    st = {"k": torch.zeros(0, 1, 2, dtype=F64), "v": torch.zeros(0, 1, 1, dtype=F64)}
    got = plain.window_attention(h, w, "", m, list(range(n)), st)[:, 0] * 2  # the gate is sigmoid(0)
    for i in range(n):
        read = [j for j in range(i + 1) if i - j < 3 or j < 2]
        assert abs(float(got[i]) - sum(read) / len(read)) < 1e-12, i
    assert abs(float(got[8]) - (0 + 1 + 6 + 7 + 8) / 5) < 1e-12
    # the sink: one head, scores all zero, a sink of ln 3 weighs as three keys
    lat = {"heads": 1, "dim": 1, "rot_dim": 0, "vdim": 1, "kv_rank": 1, "q_rank": 1, "scale": 1.0, "rot": {"base": 10.0, "dims": 0}}
    w = {"dq": torch.zeros(1, W, dtype=F64), "dq.norm": torch.ones(1, dtype=F64), "uq": torch.zeros(1, 1, dtype=F64),
         "dkv": torch.zeros(1, W, dtype=F64), "dkv.norm": torch.ones(1, dtype=F64), "uk": torch.zeros(1, 1, dtype=F64),
         "uv": torch.ones(1, 1, dtype=F64), "sink": torch.tensor([math.log(3.0)], dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    w["dkv"][0, 0] = 1.0
    h = torch.ones(5, W, dtype=F64)  # every latent norms to (almost) one: values of one
    st = {"c": torch.zeros(0, 1, dtype=F64), "r": torch.zeros(0, 0, dtype=F64)}
    got = plain.latent_attention(h, w, "", lat, 1e-12, list(range(5)), st)[:, 0]
    for i in range(5):
        assert abs(float(got[i]) - (i + 1) / (i + 1 + 3)) < 1e-9


def test_the_router_weight_scales_what_the_expert_reads():
    W = 3
    mlp = {"kind": "moe", "expert": {"ff": 2}, "router": {"experts": 2, "top": 1}}
    g = torch.Generator().manual_seed(3)
    w = {"router": torch.tensor([[2.0, 0, 0], [-2.0, 0, 0]], dtype=F64)}
    for e in range(2):
        w.update({f"e{e}.gate": torch.randn(2, W, generator=g, dtype=F64), f"e{e}.up": torch.randn(2, W, generator=g, dtype=F64),
                  f"e{e}.down": torch.randn(W, 2, generator=g, dtype=F64)})
    h = torch.tensor([[1.0, 0.3, -0.2], [-0.5, 1.0, 2.0]], dtype=F64)
    got = plain.feed_forward(h, w, "", mlp)
    for t, e in ((0, 0), (1, 1)):  # the sign of the first value chooses
        s = 1 / (1 + math.exp(-abs(2.0 * float(h[t, 0]))))
        x = s * h[t]
        a = x @ w[f"e{e}.gate"].t()
        want = (a / (1 + torch.exp(-a)) * (x @ w[f"e{e}.up"].t())) @ w[f"e{e}.down"].t()
        assert torch.allclose(got[t], want, atol=1e-12)
        unscaled = h[t] @ w[f"e{e}.gate"].t()
        other = s * ((unscaled / (1 + torch.exp(-unscaled)) * (h[t] @ w[f"e{e}.up"].t())) @ w[f"e{e}.down"].t())
        assert float((got[t] - other).abs().max()) > 1e-3  # weighing the output instead is another function
    dense = plain.feed_forward(h, {"up": torch.eye(W, dtype=F64), "down": torch.eye(W, dtype=F64)}, "", {"kind": "dense", "ff": W})
    assert torch.allclose(dense, torch.relu(h) ** 2)


def test_loop_passes_add_their_step_and_the_embedding(tmp_path):
    """Zeroing the per-pass vectors or the re-added embedding changes the logits; a model whose loop runs once adds
    only its first vector."""
    config, seed = CONFIGS["x"]
    cfg, w = plain.read_model_folder(make_folder(str(tmp_path / "x"), config, seed))
    ids = [3, 14, 15, 92, 65]
    base = plain.forward_logits(cfg, w, ids)
    for row in range(3):
        changed = dict(w)
        changed["loop.step"] = w["loop.step"].clone()
        changed["loop.step"][row] = 0
        assert float((plain.forward_logits(cfg, changed, ids) - base).abs().max()) > 1e-3
    layers = []
    plain.forward(cfg, w, ids, layers_out=layers)
    assert len(layers) == 9
    once = copy.deepcopy(cfg)
    once["loop"]["times"] = 1
    short = dict(w)
    short["loop.step"] = w["loop.step"][:1]
    a = []
    plain.forward(once, short, ids, layers_out=a)
    assert len(a) == 5 and torch.equal(a[0], layers[0]) and torch.equal(a[2], layers[2])
