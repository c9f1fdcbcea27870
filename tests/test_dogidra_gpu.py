"""Dogidra on the GPU against the plain implementation (tests/plain_dogidra.py): the small kernels against float32
torch, each mechanism alone, then whole models in every cut, batches, reuse of pages and slots, keys made to show
at every edge of the window and of the pooled blocks, long decoding and greedy generation through the engine's
entry point."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_dogidra as plain
from dogidra_models import CONFIGS, make_folder
from harness import Replayer, assert_close
from test_binupel_gpu import MixerBench, part_weights

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
F64 = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(str(tmp_path_factory.mktemp(f"dogidra_{key}")), config, seed)
            for key, (config, seed) in CONFIGS.items()}


def tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close(got, want, dtype, what="", tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)
    bound = TOL[dtype] if tol is None else tol
    assert err <= bound, f"{what}: relative error {err:.3g} > {bound:g}"


# ---------------------------------------------------------------------- the small kernels against float32 torch
@pytest.mark.parametrize("out32", [True, False])
@pytest.mark.parametrize("W,T", [(48, 5), (64, 33), (200, 7), (1024, 19), (50, 4), (201, 6), (5000, 3)])
def test_layer_norm_with_the_sum_in_front(W, T, out32):
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    from qwen3_from_scratch_b200.registry import create_part
    dtype = "float32" if out32 else "bfloat16"
    part = create_part("norm", PartSpec("layer_norm", {"dim": W, "eps": 1e-5, "suffix": ".w", "bias_suffix": ".b"}), name="n")
    dev, ref = part_weights(part, dtype, seed=W)
    part.setup(Runtime(torch.device("cuda:0"), DT[dtype], 64, 2), dict(dev))
    g = torch.Generator().manual_seed(W + T)
    stream = (3 + 2 * torch.randn(T, W, generator=g)).cuda()      # a mean far from zero: the variance is of deviations
    delta = torch.randn(T, W, generator=g).to(DT[dtype]).cuda()
    total = stream.double() + delta.double()
    want = plain.layer_norm(total.cpu(), ref["w"], ref["b"], 1e-5)
    got = part.add_norm(stream, delta)
    close(got, want, dtype, "norm of the sum", tol=1e-5 if out32 else 8e-3)
    close(stream, total, "float32", "the sum stays in the stream", tol=1e-6)
    close(part.add_norm_float32(stream, None), want, "float32", "float32 rows", tol=1e-5)


@pytest.mark.parametrize("K", [1, 2, 3, 4, 7])
def test_input_convolution_through_portions_and_slots(K):
    """h + conv(h) per request over a batch of unequal portions; what lies before a portion comes from the request's
    slot, zeros for a new request; two tokens, one token and portions shorter than the taps."""
    from qwen3_from_scratch_b200.kernels import ops
    C, slots = 70, 3
    g = torch.Generator().manual_seed(K)
    w = torch.randn(C, K, generator=g)
    h_of = {"a": torch.randn(23, C, generator=g), "b": torch.randn(11, C, generator=g)}
    want = {r: plain.input_conv(h.double(), w.double(), torch.zeros(K - 1, C, dtype=F64))[0] for r, h in h_of.items()}
    state = torch.full((slots, max(K - 1, 1), C), float("nan")).cuda()
    state[2].zero_(); state[0].zero_()
    slot_of, fed, got = {"a": 2, "b": 0}, {"a": 0, "b": 0}, {"a": [], "b": []}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in ([("a", 1)], [("a", 2), ("b", 1)], [("b", 2), ("a", 1)], [("a", 9), ("b", 5)], [("a", 1)], [("b", 3), ("a", 9)]):
        rows = torch.cat([h_of[r][fed[r]:fed[r] + n] for r, n in step]).cuda()
        starts = [0]
        for _, n in step:
            starts.append(starts[-1] + n)
        q_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
        tok_seq = torch.tensor([i for i, (_, n) in enumerate(step) for _ in range(n)], dtype=torch.int32, device="cuda")
        slot_ids = torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device="cuda")
        out = torch.empty(rows.shape[0], C, device="cuda")
        ops.input_conv(rows, w.cuda(), state if K > 1 else None, q_start, tok_seq, slot_ids, len(step), out, status)
        for i, (r, n) in enumerate(step):
            got[r].append(out[starts[i]:starts[i + 1]].cpu())
            fed[r] += n
    assert int(status.item()) == 0
    for r in h_of:
        close(torch.cat(got[r]), want[r][:fed[r]], "float32", f"taps {K} request {r}", tol=1e-6)


@pytest.mark.parametrize("K", [1, 2, 4, 8, 9])
def test_input_convolution_of_long_portions_beside_each_other(K):
    """Portions long enough for the kernel that walks runs of tokens (and, for taps it has no form for, the one that
    takes four channels at a time): requests that start and end inside a run, a portion after a single token."""
    from qwen3_from_scratch_b200.kernels import ops
    C, slots = 136, 4
    g = torch.Generator().manual_seed(K + 20)
    w = torch.randn(C, K, generator=g)
    h_of = {"a": torch.randn(150, C, generator=g), "b": torch.randn(77, C, generator=g)}
    want = {r: plain.input_conv(h.double(), w.double(), torch.zeros(K - 1, C, dtype=F64))[0] for r, h in h_of.items()}
    state = torch.zeros(slots, max(K - 1, 1), C).cuda()
    slot_of, fed, got = {"a": 3, "b": 1}, {"a": 0, "b": 0}, {"a": [], "b": []}
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in ([("a", 1)], [("a", 50), ("b", 37)], [("b", 40), ("a", 99)]):
        rows = torch.cat([h_of[r][fed[r]:fed[r] + n] for r, n in step]).cuda()
        starts = [0]
        for _, n in step:
            starts.append(starts[-1] + n)
        q_start = torch.tensor(starts, dtype=torch.int32, device="cuda")
        tok_seq = torch.tensor([i for i, (_, n) in enumerate(step) for _ in range(n)], dtype=torch.int32, device="cuda")
        slot_ids = torch.tensor([slot_of[r] for r, _ in step], dtype=torch.int32, device="cuda")
        out = torch.empty(rows.shape[0], C, device="cuda")
        ops.input_conv(rows, w.cuda(), state if K > 1 else None, q_start, tok_seq, slot_ids, len(step), out, status)
        for i, (r, n) in enumerate(step):
            got[r].append(out[starts[i]:starts[i + 1]].cpu())
            fed[r] += n
    assert int(status.item()) == 0
    for r in h_of:
        close(torch.cat(got[r]), want[r], "float32", f"taps {K} request {r}", tol=1e-6)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("W,K", [(48, 4), (200, 2), (2048, 3), (64, 1), (4100, 5)])
def test_norm_and_convolution_of_single_tokens_in_one_launch(W, K, dtype):
    """A step of single tokens: the fused kernel gives the bits of the norm and the convolution one after the other,
    for the output, the stream and the state, through slots in any order and a second step on the renewed state."""
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(W + K)
    B, slots = 5, 7
    weight, bias = (1 + 0.3 * torch.randn(W, generator=g)).cuda(), (0.2 * torch.randn(W, generator=g)).cuda()
    taps = (0.5 * torch.randn(W, K, generator=g)).cuda()
    slot_ids = torch.tensor([4, 0, 6, 2, 3], dtype=torch.int32).cuda()
    tok_seq = torch.arange(B, dtype=torch.int32).cuda()
    q_start = torch.arange(B + 1, dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    state = {k: (torch.randn(slots, K - 1, W, generator=g).cuda() if K > 1 else None) for k in ("two", "one")}
    if K > 1:
        state["one"].copy_(state["two"])
    stream = {k: torch.randn(B, W, generator=torch.Generator().manual_seed(3)).cuda() for k in ("two", "one")}
    for step in range(2):
        delta = torch.randn(B, W, generator=g).to(DT[dtype]).cuda() if step else None
        h = torch.empty(B, W, dtype=torch.float32).cuda()
        two, one = torch.empty(B, W, dtype=DT[dtype]).cuda(), torch.empty(B, W, dtype=DT[dtype]).cuda()
        ops.add_layernorm(stream["two"], delta, weight, bias, h, 1e-5)
        ops.input_conv(h, taps, state["two"], q_start, tok_seq, slot_ids, B, two, status)
        ops.add_layernorm_conv1(stream["one"], delta, weight, bias, taps, state["one"], tok_seq, slot_ids, one, 1e-5, status)
        assert torch.equal(one, two) and torch.equal(stream["one"], stream["two"])
        assert K == 1 or torch.equal(state["one"], state["two"])
        x = stream["two"].double()
        hh = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + 1e-5) * weight.double() \
            + bias.double()
        if step == 0 and K > 1:
            first = state["two"][slot_ids.long()].double().clone()  # after the step: the older entries moved up
            assert torch.equal(first[:, -1].float(), h)
        close(h, hh, "float32", "the normed rows")
    assert int(status.item()) == 0


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("W,E,top", [(40, 6, 2), (64, 5, 1), (100, 4, 4), (72, 33, 8), (2048, 64, 6)])
def test_router_choice_and_weights(W, E, top, dtype):
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(E)
    T = 50
    h = torch.randn(T, W, generator=g).to(DT[dtype])
    wr = torch.randn(E, W, generator=g) * (3.0 / W ** 0.5)
    bias = 0.3 * torch.randn(E, generator=g)
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    ops.moe_route(h.cuda(), wr.cuda(), bias.cuda(), ids, wts, 1.7)
    s = plain.sigmoid(h.double() @ wr.double().t())
    choice = s + bias.double()
    order = torch.sort(choice, dim=-1, descending=True)
    margin = (order.values[:, top - 1] - order.values[:, top]) if top < E else torch.ones(T, dtype=F64)
    inner = (order.values[:, :top - 1] - order.values[:, 1:top]).min(-1).values if top > 1 else torch.ones(T, dtype=F64)
    sure = (margin > 1e-4) & (inner > 1e-4)  # rows in which float32 rounding cannot turn the choice or its order
    assert int(sure.sum()) > T // 2
    assert torch.equal(ids.cpu().long()[sure], order.indices[:, :top][sure])
    close(wts.cpu()[sure], 1.7 * torch.gather(s, 1, order.indices[:, :top])[sure], "float32", "weights", tol=1e-5)


# ---------------------------------------------------------------------- each mechanism alone
def _attention(params):
    pos = params["position"].params
    m = {"heads": params["num_heads"], "kv_heads": params["num_kv_heads"], "dim": params["dim"], "vdim": params["vdim"],
         "scale": params["scale"], "softcap": params.get("softcap"), "mask": {"size": params["window"], "pool": params["pool"]},
         "rot": {"dims": pos["dims"], "base": pos["base"], "scaling": pos["scaling"]}}

    def fn(h, ref, _):
        G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
        cache = {"k": torch.zeros(0, G, D, dtype=F64), "v": torch.zeros(0, G, Dv, dtype=F64)}
        return plain.left_mixer(h, ref, "", m, params["norm_eps"], list(range(h.shape[0])), cache), None
    return fn


def _mingru(params):
    return lambda h, ref, _: plain.min_gru(h, ref, "", torch.zeros(params["width"], dtype=F64))


def _parallel(params):
    def fn(h, ref, _):
        total = 0
        for b in params["branches"]:
            sub = {k[len(b["label"]) + 1:]: v for k, v in ref.items() if k.startswith(b["label"] + ".")}
            one = (_attention if b["mixer"].kind == "pooled_window_attention" else _mingru)(b["mixer"].params)
            total = total + b["scale"] * one(h, sub, None)[0]
        return total, None
    return fn


def mixers():
    from qwen3_from_scratch_b200.parts.base import PartSpec

    def rot(dims, base, scaling=None):
        return PartSpec("rotary_stretched", {"dims": dims, "base": base, "scaling": scaling})

    stretch = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0, "magnitude": (0.1, 1.0)}
    att = {"hidden_size": 40, "num_heads": 6, "num_kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.3, "softcap": 4.0,
           "window": 9, "pool": 4, "norm_eps": 1e-5, "position": rot(16, 10000.0, stretch)}
    table = {
        "pooled_window_attention": att,
        # one head, blocks longer than the window, no cap, no stretching, the whole head rotated
        "pooled_window_attention, long blocks": dict(att, num_heads=1, num_kv_heads=1, dim=32, vdim=8, window=3, pool=7,
                                                     softcap=None, position=rot(32, 300.0)),
        # blocks of one token (every token before the window is read as a block of its own), a window of one, no rotation
        "pooled_window_attention, blocks of one": dict(att, num_heads=5, num_kv_heads=5, dim=8, vdim=16, window=1, pool=1,
                                                       position=rot(0, 10000.0)),
        # seventeen query heads on one key head (more than a tensor-core tile's sixteen rows), a page's worth of window
        "pooled_window_attention, many heads": dict(att, num_heads=17, num_kv_heads=1, dim=16, vdim=16, window=16, pool=5),
        # sizes that the tensor-core kernel takes: steps of single tokens cut the keys into ranges, most of them empty
        "pooled_window_attention, tensor cores": dict(att, num_heads=4, num_kv_heads=2, dim=32, vdim=64),
        "pooled_window_attention, tensor cores, wide heads": dict(att, num_heads=3, num_kv_heads=1, dim=128, vdim=32,
                                                                  window=5, pool=2, softcap=None),
        "mingru": {"hidden_size": 40, "width": 72},
        "mingru, odd": {"hidden_size": 40, "width": 37},
    }
    table["parallel"] = {"hidden_size": 40, "branches": [
        {"label": "left", "mixer": PartSpec("pooled_window_attention", att), "scale": 0.7},
        {"label": "right", "mixer": PartSpec("mingru", table["mingru"]), "scale": 1.3}]}
    fns = {"pooled_window_attention": _attention, "mingru": _mingru, "parallel": _parallel}
    return {k: (v, fns[k.split(",")[0]](v)) for k, v in table.items()}


MIXER_KINDS = ["pooled_window_attention", "pooled_window_attention, long blocks", "pooled_window_attention, blocks of one",
               "pooled_window_attention, many heads", "pooled_window_attention, tensor cores",
               "pooled_window_attention, tensor cores, wide heads", "mingru", "mingru, odd", "parallel"]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("kind", MIXER_KINDS)
def test_mixer_alone_whole_in_portions_and_beside_another_request(kind, dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params, plain_fn = mixers()[kind]
    bench = MixerBench(create_part("mixer", PartSpec(kind.split(",")[0], params), name="m"), dtype, seed=11)
    g = torch.Generator().manual_seed(12)
    x_of = {r: torch.randn(n, 40, generator=g).to(DT[dtype]) for r, n in (("a", 61), ("b", 19))}
    want = {r: plain_fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda x, ctx: bench.part.forward(x.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    for r in x_of:  # whole, each alone
        close(bench.run([(r, len(x_of[r]))], x_of, call)[r], want[r], dtype, f"{kind} whole {r}")
        bench.manager.close(r)
    # portions down to one and two tokens, the second request joining and leaving in between
    got = {r: [] for r in x_of}
    for step in ([("a", 7)], [("a", 1)], [("a", 2), ("b", 2)], [("b", 1), ("a", 1)], [("a", 13), ("b", 16)],
                 [("a", 2)], [("a", 1)], [("a", 14)], [("a", 2)], [("a", 1)], [("a", 1)], [("a", 16)]):
        for r, y in bench.run(step, x_of, call).items():
            got[r].append(y)
    for r in x_of:
        close(torch.cat(got[r]), want[r], dtype, f"{kind} portions {r}")


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows", [1, 3, 12, 40, 300])
@pytest.mark.parametrize("E,top,ff,shared", [(6, 2, 24, 40), (5, 1, 32, None), (4, 4, 16, 24), (16, 3, 64, 128)])
def test_routed_experts_few_rows_and_many(E, top, ff, shared, rows, dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    from qwen3_from_scratch_b200.registry import create_part
    W = 64
    sh = None if shared is None else PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": shared,
                                                            "activation": "relu_sq", "names": {"up": "up", "down": "down"}})
    part = create_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "experts": E, "top": top, "expert_ff": ff, "router_scale": 1.5, "activation": "relu_sq",
        "shared": sh}), name="f")
    dev, ref = part_weights(part, dtype, seed=rows + E, scale={"router": 6.0})
    part.setup(Runtime(torch.device("cuda:0"), DT[dtype], 512, 2), dict(dev))
    x = torch.randn(rows, W, generator=torch.Generator().manual_seed(rows + 1)).to(DT[dtype])
    mlp = {"router": {"experts": E, "top": top, "scale": 1.5}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_experts(x.double(), ref, "", mlp)
    got = part.forward(x.cuda()).double().cpu()
    # a row whose choice hangs on a difference that rounding can turn is left out (at most a few)
    s = plain.sigmoid(x.double() @ ref["router"].t()) + ref["correction"]
    order = torch.sort(s, dim=-1, descending=True).values
    sure = (order[:, top - 1] - order[:, top] > 1e-3) if top < E else torch.ones(rows, dtype=torch.bool)
    assert int(sure.sum()) >= rows * 0.9
    close(got[sure], want[sure], dtype, f"{rows} rows")


@pytest.mark.parametrize("W,E,top,ff,shared,rows", [(320, 8, 2, 264, 72, 900), (136, 3, 3, 520, None, 1500),
                                                     (64, 40, 5, 8, 16, 333)])
def test_routed_experts_grouped_products_over_several_tiles(W, E, top, ff, shared, rows):
    """bfloat16 and many rows: the sorted, grouped products with several tiles per expert, several tiles of columns, an
    inner size that is no multiple of a tile's 64, more experts than rows per tile; then a few rows through the same
    part (a pair at a time) while the sorted rows still hold the step before."""
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    from qwen3_from_scratch_b200.registry import create_part
    sh = None if shared is None else PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": shared,
                                                            "activation": "relu_sq", "names": {"up": "up", "down": "down"}})
    part = create_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": W, "experts": E, "top": top, "expert_ff": ff, "router_scale": 0.8, "activation": "relu_sq",
        "shared": sh}), name="f")
    dev, ref = part_weights(part, "bfloat16", seed=rows, scale={"router": 6.0})
    rt = Runtime(torch.device("cuda:0"), torch.bfloat16, 2048, 2)
    part.setup(rt, dict(dev))
    mlp = {"router": {"experts": E, "top": top, "scale": 0.8}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}
    for n, seed in ((rows, 1), (rows // 3, 2), (5, 3), (rows, 1)):
        x = torch.randn(n, W, generator=torch.Generator().manual_seed(rows + seed)).to(torch.bfloat16)
        want = plain.routed_experts(x.double(), ref, "", mlp)
        got = part.forward(x.cuda()).double().cpu()
        s = plain.sigmoid(x.double() @ ref["router"].t()) + ref["correction"]
        order = torch.sort(s, dim=-1, descending=True).values
        sure = (order[:, top - 1] - order[:, top] > 1e-3) if top < E else torch.ones(n, dtype=torch.bool)
        assert int(sure.sum()) >= int(n * 0.9)
        close(got[sure], want[sure], "bfloat16", f"{n} rows")
    assert int(rt.status.item()) == 0


def test_chunked_recurrence_of_long_portions_side_by_side():
    """bfloat16: two requests with portions long enough for the chunked scan in one step (lengths that are no multiple
    of a chunk), after a first portion each that left a state, and single tokens after; a width that fills no warp."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params = {"hidden_size": 32, "width": 37}
    part = create_part("mixer", PartSpec("mingru", params), name="m")
    bench = MixerBench(part, "bfloat16", page_size=8, pages=8, max_tokens=1024, seed=61)
    g = torch.Generator().manual_seed(62)
    x_of = {"a": torch.randn(420, 32, generator=g).to(torch.bfloat16), "b": torch.randn(391, 32, generator=g).to(torch.bfloat16)}
    fn = _mingru(params)
    want = {r: fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda rows, ctx: part.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    got = {r: [] for r in x_of}
    for step in ([("a", 3)], [("b", 70), ("a", 1)], [("a", 301), ("b", 257)], [("b", 1), ("a", 1)], [("a", 114), ("b", 63)]):
        for r, y in bench.run(step, x_of, call).items():
            got[r].append(y)
    for r in x_of:
        close(torch.cat(got[r]), want[r], "bfloat16", f"request {r}")


def _sharp_scores(x, ref, params):
    """(largest softmax weight [heads, n], what holds it: a token's distance back, or -1 - b for block b)."""
    n, H, G, D = x.shape[0], params["num_heads"], params["num_kv_heads"], params["dim"]
    pos = params["position"].params
    rot = {"dims": pos["dims"], "base": pos["base"], "scaling": pos["scaling"]}
    q = plain.rotate(plain.rms_norm(x @ ref["q"].t(), ref["q.norm"], params["norm_eps"]).view(n, H, D), range(n), rot)
    k = plain.rotate(plain.rms_norm(x @ ref["k"].t(), ref["k.norm"], params["norm_eps"]).view(n, G, D), range(n), rot)
    top, what = torch.zeros(H, n, dtype=F64), torch.zeros(H, n, dtype=torch.long)
    for i in range(n):
        toks, blocks = plain.visible(i, params["window"], params["pool"])
        P = params["pool"]
        for h in range(H):
            g = h // (H // G)
            keys = torch.stack([k[j, g] for j in toks] + [k[b * P:(b + 1) * P, g].mean(0) for b in blocks])
            p = torch.softmax(keys @ q[i, h] * params["scale"], 0)
            a = int(p.argmax())
            top[h, i] = p[a]
            what[h, i] = i - toks[a] if a < len(toks) else -1 - blocks[a - len(toks)]
    return top, what


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("dim,vdim", [(16, 24), (32, 64)])  # the second: sizes that the tensor-core kernel takes
def test_sharp_attention_reads_the_windows_edges_and_far_blocks(dim, vdim, dtype):
    """A scale so large that nearly every query gives all its weight to one key or one block, which random weights
    put anywhere: the window's oldest token, the query's own, the block that has just become visible, blocks
    hundreds of tokens back, the very first block, slots at a page's border.  A key that is lost, read one token
    too far or one block too early changes that query's output entirely.  As a whole prompt, then in portions and
    single tokens."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    W, n, page = 32, 330, 8
    params = {"hidden_size": W, "num_heads": 4, "num_kv_heads": 2, "dim": dim, "vdim": vdim, "scale": 7.0, "softcap": None,
              "window": 11, "pool": 3, "norm_eps": 1e-5,
              "position": PartSpec("rotary_stretched", {"dims": 8, "base": 10000.0, "scaling": None})}
    part = create_part("mixer", PartSpec("pooled_window_attention", params), name="m")
    bench = MixerBench(part, dtype, page_size=page, pages=64, max_tokens=512, seed=41)
    x = torch.randn(n, W, generator=torch.Generator().manual_seed(42)).to(DT[dtype])
    want = _attention(params)(x.double(), bench.ref, None)[0]
    top, what = _sharp_scores(x.double(), bench.ref, params)
    sharp = top > (0.9 if dtype == "float32" else 0.99)
    pos = torch.arange(n)[None, :].expand_as(what)
    newest_block = (pos - params["window"] - (params["pool"] - 1)) // params["pool"]  # the last block a position reads
    assert sharp.float().mean() > 0.3
    assert int((what[sharp] == params["window"] - 1).sum()) > 3, "the window's oldest token"
    assert int((what[sharp] == 0).sum()) > 3, "the query's own key"
    assert int(((-1 - what == newest_block) & sharp).sum()) > 3, "the block that has just become visible"
    assert int(((what == -1) & sharp & (pos > 200)).sum()) > 0, "the first block from far away"
    assert int(((what < 0) & sharp & (newest_block + 1 + what > 60)).sum()) > 3, "blocks far back"
    rows = sharp.all(0).nonzero()[:, 0] if dtype == "bfloat16" else torch.arange(n)
    assert rows.numel() > 40
    call = lambda r, ctx: part.forward(r.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    got = bench.run([("r", n)], {"r": x}, call)["r"]
    close(got[rows], want[rows], dtype, "whole prompt")
    bench.manager.close("r")
    cuts = [47, 1, 1, 100, 1] + [2] * 30 + [17, 15, 33] + [1] * (n - 47 - 103 - 60 - 65)
    pieces = torch.cat([bench.run([("r", c)], {"r": x}, call)["r"] for c in cuts])
    close(pieces[rows], want[rows], dtype, "portions and single tokens")


@pytest.mark.parametrize("dtype", list(DT))
def test_a_slow_gate_carries_the_first_token_to_the_end(dtype):
    """Update gates near zero after a first token that writes the state: what it wrote is still most of the output
    hundreds of tokens later, through portions and single tokens and beside another request's tokens."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params = {"hidden_size": 32, "width": 48}

    def tweak(dev, ref):
        for tensors, pre in ((dev, "m."), (ref, "")):
            tensors[pre + "z.b"].fill_(-7.0)  # sigmoid(-7 + small): the state keeps 999 thousandths per token

    part = create_part("mixer", PartSpec("mingru", params), name="m")
    bench = MixerBench(part, dtype, page_size=8, pages=8, max_tokens=512, seed=51, tweak=tweak)
    g = torch.Generator().manual_seed(52)
    n = 400
    x = 0.02 * torch.randn(n, 32, generator=g)
    x[0] = 6 * torch.randn(32, generator=g)  # gates of the first token are wide open where W_z x is large
    x_of = {"r": x.to(DT[dtype]), "o": torch.randn(9, 32, generator=g).to(DT[dtype])}
    fn = _mingru(params)
    want = fn(x_of["r"].double(), bench.ref, None)[0]
    quiet = x_of["r"].clone()
    quiet[0] = 0
    assert float((want[-1] - fn(quiet.double(), bench.ref, None)[0][-1]).abs().max()) > 0.3 * float(want[-1].abs().max())
    call = lambda rows, ctx: part.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    close(bench.run([("r", n)], x_of, call)["r"], want, dtype, "whole")
    bench.manager.close("r")
    got = []
    for step in ([("r", 1)], [("r", 2), ("o", 4)], [("r", 290)], [("o", 1), ("r", 1)], [("r", 2)], [("r", 64), ("o", 4)]) \
            + tuple([("r", 1)] for _ in range(40)):
        got.append(bench.run(list(step), x_of, call)["r"])
    close(torch.cat(got), want, dtype, "portions")


# ---------------------------------------------------------------------- whole models
def tolerance(dtype, cfg, w, seqs):
    """float32: the harness's bound.  bfloat16: three times what rounding alone does to these prompts in the plain
    implementation (projections' operands and results rounded to bfloat16), and no less than the harness's bound."""
    if dtype == "float32":
        return None
    return max(TOL[dtype], 3 * max(plain.rounding_error(cfg, w, ids) for ids in seqs.values()))


def replay(folder, dtype, seqs, schedule, **session_args):
    from qwen3_from_scratch_b200.engine.session import Session
    args = dict(page_size=8, num_pages=96, max_seqs=3, max_step_tokens=256)
    args.update(session_args)
    session = Session(folder, dtype=dtype, **args)
    r = Replayer(session, seqs)
    schedule(r)
    session.manager.check()
    assert session.manager.free_slots() == args["max_seqs"]
    return r.result()


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("key", list(CONFIGS))
def test_model_whole_decoded_and_in_portions(folders, key, dtype):
    """90 tokens: every window of the small models (1 to 16 tokens, 64 and 48 in the third) passes over prompt tokens
    and over decoded ones, blocks close inside portions and at single tokens."""
    cfg, w = plain.read_model_folder(folders[key])
    n = 90 if key != "z" else 150
    ids = tokens(cfg["vocab"], n, 51)
    want = {"a": plain.forward_logits(cfg, w, ids)}
    tol = tolerance(dtype, cfg, w, {"a": ids})

    def whole(r):
        r.step([("a", n)])

    def decoded(r):
        r.step([("a", n - 60)])
        for _ in range(60):
            r.step([("a", 1)])

    def portions(r):
        for c in [3, 2, 2, 1, 17, 2, 31, 1, 1, 2, 16, 2, 8, 2] + [n - 90] * (n > 90):
            r.step([("a", c)])

    for name, schedule in (("whole", whole), ("decoded", decoded), ("portions", portions)):
        assert_close(replay(folders[key], dtype, {"a": ids}, schedule), want, dtype, f"{key} {name}", tol=tol)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("key", ["x", "z"])
def test_unequal_requests_together_equal_each_alone_with_pages_and_slots_used_again(folders, key, dtype):
    """Five requests through two state slots and a pool that holds less than their sum: portions of some beside
    single tokens of others; a slot and its pages go to the next request as soon as one ends; pages that fall out of
    a window are given back while the request lives; freed pages are filled with NaN."""
    cfg, w = plain.read_model_folder(folders[key])
    lens = {"a": 61, "b": 7, "c": 33, "d": 1, "e": 40}
    seqs = {r: tokens(cfg["vocab"], n, 60 + i) for i, (r, n) in enumerate(lens.items())}
    want = {r: plain.forward_logits(cfg, w, ids) for r, ids in seqs.items()}

    def schedule(r):
        r.step([("a", 30), ("b", 5)])
        r.step([("a", 1), ("b", 2)])             # b ends: its slot is free
        r.step([("c", 2), ("a", 1)])             # c takes b's slot
        r.step([("a", 1), ("c", 20)])
        r.step([("c", 1)])                       # a is left out of a step
        r.step([("a", 28), ("c", 10)])           # both end
        r.step([("d", 1), ("e", 9)])             # a request of a single token
        for _ in range(31):
            r.step([("e", 1)])

    got = replay(folders[key], dtype, seqs, schedule, page_size=4, num_pages=26, max_seqs=2, poison_freed_pages=True)
    assert_close(got, want, dtype, f"{key} mixed", tol=tolerance(dtype, cfg, w, seqs))


def test_long_prompt_on_the_serving_kernels(folders):
    """bfloat16 at the serving kernels' sizes with pages of 16: a prompt of 700 tokens whole and cut into long and
    short portions with single tokens between them; then a batch of a long portion beside single tokens."""
    cfg, w = plain.read_model_folder(folders["z"])
    ids, other = tokens(cfg["vocab"], 700, 77), tokens(cfg["vocab"], 90, 78)
    want = {"a": plain.forward_logits(cfg, w, ids), "b": plain.forward_logits(cfg, w, other)}
    tol = tolerance("bfloat16", cfg, w, {"a": ids, "b": other})
    for name, cuts in (("whole", [700]), ("portions", [300, 1, 250, 1, 1, 130, 17])):
        got = replay(folders["z"], "bfloat16", {"a": ids}, lambda r, cuts=cuts: [r.step([("a", n)]) for n in cuts],
                     page_size=16, num_pages=64, max_seqs=2, max_step_tokens=1024)
        assert_close(got, {"a": want["a"]}, "bfloat16", f"z long {name}", tol=tol)

    def beside(r):
        r.step([("b", 70)])
        r.step([("a", 300), ("b", 1)])
        r.step([("b", 1), ("a", 399)])
        r.step([("a", 1), ("b", 18)])

    got = replay(folders["z"], "bfloat16", {"a": ids, "b": other}, beside, page_size=16, num_pages=64, max_seqs=2,
                 max_step_tokens=1024)
    assert_close(got, want, "bfloat16", "z long beside single tokens", tol=tol)


@pytest.mark.parametrize("dtype", list(DT))
def test_long_decoding_through_graphs(folders, dtype):
    """300 single tokens after a short prompt, replayed from CUDA graphs: the state, the tails and the pages are
    carried on the device from step to step, pages leave the window and are used again."""
    cfg, w = plain.read_model_folder(folders["x"])
    ids = tokens(cfg["vocab"], 310, 71)
    want = {"a": plain.forward_logits(cfg, w, ids)}

    def schedule(r):
        r.step([("a", 10)])
        for _ in range(300):
            r.step([("a", 1)])

    got = replay(folders["x"], dtype, {"a": ids}, schedule, page_size=4, num_pages=80, max_seqs=2)
    assert_close(got, want, dtype, "long decoding", tol=tolerance(dtype, cfg, w, {"a": ids}))


def test_float32_cuts_give_identical_bits(folders):
    """In float32 every sum has an order that depends only on the token, so a prompt whole, in portions and
    token by token gives the same bits."""
    cfg, _ = plain.read_model_folder(folders["x"])
    ids = tokens(cfg["vocab"], 45, 81)
    runs = [replay(folders["x"], "float32", {"a": ids}, s)["a"] for s in (
        lambda r: r.step([("a", 45)]),
        lambda r: [r.step([("a", n)]) for n in (7, 2, 1, 20, 15)],
        lambda r: [r.step([("a", 1)]) for _ in range(45)])]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])


# ---------------------------------------------------------------------- the engine's entry points
@pytest.mark.parametrize("key", ["x", "y"])
def test_greedy_generation_through_the_engine_equals_plain(folders, key):
    """Prompts of unequal length through SyncEngine.batch_generate: chunked prompts, continuous batching with
    fewer slots than requests, lookahead, CUDA graphs; float32, prompts chosen so that no step is a near tie."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    cfg, w = plain.read_model_folder(folders[key])
    prompts, expected = [], []
    for i, n in enumerate([1, 9, 33, 70]):
        for seed in range(100 * i, 100 * i + 50):
            prompt = tokens(cfg["vocab"], n, seed)
            out, margins = plain.greedy(cfg, w, prompt, 12)
            if min(margins) > 1e-3:
                break
        prompts.append(prompt)
        expected.append(out)
    engine = SyncEngine(folders[key], dtype="float32", block_size=8, num_pages=64, max_num_seqs=3, max_num_tokens=48,
                        chunked_prefill_size=16)
    results, batch = engine.batch_generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert batch.num_requests == 4
    for want, r in zip(expected, results):
        assert r.token_ids == want and r.finish_reason == "length"
    engine.session.manager.check()
    assert engine.session.manager.free_slots() == 3


def test_preempted_request_is_recomputed_from_a_clean_state(folders):
    """A pool too small for all requests at once: the one that loses its pages starts again in a zeroed slot and
    still generates what it generates alone."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    cfg, _ = plain.read_model_folder(folders["y"])
    prompts = [tokens(cfg["vocab"], n, 90 + i) for i, n in enumerate([30, 28, 26])]
    alone = SyncEngine(folders["y"], dtype="float32", block_size=4, num_pages=96, max_num_seqs=4, max_num_tokens=64)
    want = [alone.generate(p, max_new_tokens=24, ignore_eos=True) for p in prompts]
    tight = SyncEngine(folders["y"], dtype="float32", block_size=4, num_pages=34, max_num_seqs=4, max_num_tokens=64)
    results, _ = tight.batch_generate(prompts, max_new_tokens=24, ignore_eos=True)
    assert [r.token_ids for r in results] == want


@pytest.mark.parametrize("dtype", list(DT))
def test_trace_replay_program_and_command_line(folders, tmp_path, dtype):
    folder = folders["x"]
    cfg, w = plain.read_model_folder(folder)
    vocab = cfg["vocab"]
    a, b = tokens(vocab, 70, 31), tokens(vocab, 50, 32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]},
                                {"id": "b", "tokens": b[2:50], "want": [47, 0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[41:70], "want": list(range(29))}], "end": ["a"]},
    ]
    out = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
           "--max-tokens", "192", "--poison-freed-pages"]
    proc = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(4)]
    la, lb = plain.forward_logits(cfg, w, a), plain.forward_logits(cfg, w, b)
    tol = tolerance(dtype, cfg, w, {"a": a, "b": b}) or TOL[dtype]

    def check(step, rows):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")).view(len(rows), vocab)
        want = torch.stack(rows)
        assert float((got - want).abs().max()) <= tol * float(max(la.abs().max(), lb.abs().max()))

    check(0, [la[0], la[39]])
    check(2, [la[40], lb[49], lb[2]])
    check(3, [la[41 + i] for i in range(29)])
    if dtype == "float32":
        prompt = a[:9]
        want, margins = plain.greedy(cfg, w, prompt, 6)
        gen = [sys.executable, "-m", "qwen3_from_scratch_b200", "generate", "--model", folder, "--dtype", "float32",
               "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--ignore-eos",
               "--block-size", "4", "--num-pages", "32", "--max-num-seqs", "2", "--max-num-tokens", "32"]
        proc = subprocess.run(gen, capture_output=True, text=True, cwd=ROOT, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        if min(margins) > 1e-3:
            assert json.loads(proc.stdout.splitlines()[0])["token_ids"] == want
