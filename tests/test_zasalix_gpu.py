"""Zasalix on the GPU against the plain implementation (tests/plain_zasalix.py): the small kernels against float32
torch, each mechanism alone through portions and batches, keys made to show at every edge of the window and among the
kept first tokens, a memory that carries its first token to the end, then whole models in every cut, batches, reuse of
pages and slots, long decoding and greedy generation through the engine's entry point."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zasalix as plain
from harness import Replayer, assert_close
from test_binupel_gpu import MixerBench, part_weights
from zasalix_models import CONFIGS, make_folder

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
F64 = torch.float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(str(tmp_path_factory.mktemp(f"zasalix_{key}")), config, seed)
            for key, (config, seed) in CONFIGS.items()}


def tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close(got, want, dtype, what="", tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)
    bound = TOL[dtype] if tol is None else tol
    assert err <= bound, f"{what}: relative error {err:.3g} > {bound:g}"


def part(kind, name, params):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    return create_part(kind, PartSpec(name, params), name="m")


# ---------------------------------------------------------------------- the small kernels against float32 torch
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("W,T", [(48, 5), (64, 33), (200, 7), (1030, 19), (5000, 3)])
def test_dynamic_tanh_with_the_sums_in_front(W, T, dtype):
    """The norm after a sub-layer, the sum into the stream, what a pass of a loop adds, and the norm before the next
    sub-layer in one kernel; the same for chosen rows with the stream left alone; the sum alone."""
    from qwen3_from_scratch_b200.parts.base import PendingNormed, Runtime
    rt = Runtime(torch.device("cuda:0"), DT[dtype], 64, 2)
    before, after = part("norm", "dynamic_tanh", {"dim": W}), part("norm", "dynamic_tanh", {"dim": W})
    refs = []
    for p, seed in ((before, 1), (after, 2)):
        dev, ref = part_weights(p, dtype, seed=W + seed)
        p.setup(rt, dict(dev))
        refs.append({"n": ref["weight"], "n.b": ref["bias"], "n.alpha": ref["alpha"]})
    g = torch.Generator().manual_seed(W + T)
    stream0 = 2 * torch.randn(T, W, generator=g)
    delta = (1.5 * torch.randn(T, W, generator=g)).to(DT[dtype])
    rows_add, vec_add = torch.randn(T, W, generator=g), torch.randn(W, generator=g)
    tight = 1e-6 if dtype == "float32" else 8e-3
    # plain sum and norm
    stream = stream0.clone().cuda()
    got = before.add_norm(stream, delta.cuda())
    total = stream0.double() + delta.double()
    close(got, plain.dynamic_tanh(total, refs[0], "n"), dtype, "norm of the sum", tol=tight)
    close(stream, total, "float32", "the sum stays in the stream", tol=1e-6)
    # everything at once
    stream = stream0.clone().cuda()
    got = before.add_norm(stream, PendingNormed(delta.cuda(), after), extra_rows=rows_add.cuda(), extra_vec=vec_add.cuda())
    total = stream0.double() + plain.dynamic_tanh(delta.double(), refs[1], "n") + rows_add.double() + vec_add.double()
    close(stream, total, "float32", "stream", tol=1e-6)
    close(got, plain.dynamic_tanh(total, refs[0], "n"), dtype, "normed", tol=tight)
    # chosen rows, the stream untouched
    stream = stream0.clone().cuda()
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32).cuda()
    got = before.norm_rows(stream, PendingNormed(delta.cuda(), after), rows)
    total = stream0.double() + plain.dynamic_tanh(delta.double(), refs[1], "n")
    close(got, plain.dynamic_tanh(total, refs[0], "n")[rows.cpu().long()], dtype, "rows", tol=tight)
    assert torch.equal(stream.cpu(), stream0)
    # the sum alone, with a copy for the next product
    copy = after.close(stream, delta.cuda(), want_copy=True)
    close(stream, total, "float32", "closed", tol=1e-6)
    close(copy, total, dtype, "copy", tol=tight)


@pytest.mark.parametrize("dtype", list(DT))
def test_token_side_kernels_and_the_gate(dtype):
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    T, W, d = 9, 136, 24
    p = torch.randn(T, d, generator=g).to(DT[dtype])
    side = torch.randn(T, 5 * d, generator=g)
    out = torch.empty(T, d, dtype=DT[dtype], device="cuda")
    ops.side_gate(p.cuda(), side.cuda(), 2 * d, out)
    close(out, plain.gelu_tanh(p.double()) * side[:, 2 * d:3 * d].double(), dtype, "side gate", tol=1e-6 if dtype == "float32" else 8e-3)
    y = (3 * torch.randn(T, W, generator=g)).to(DT[dtype])
    weight, stream0 = 1 + 0.2 * torch.randn(W, generator=g), torch.randn(T, W, generator=g)
    stream = stream0.clone().cuda()
    ops.add_unit_rms(stream, y.cuda(), weight.cuda(), 1e-5)
    close(stream, stream0.double() + plain.rms_norm(y.double(), weight.double(), 1e-5), "float32", "unit rms", tol=1e-6)
    wide = torch.randn(T, 3 * W, generator=g).to(DT[dtype]).cuda()
    proj = torch.randn(T, 2 * W + 8, generator=g).to(DT[dtype])
    view = wide[:, W:2 * W]
    want = view.double().cpu() * plain.sigmoid(proj[:, 8:8 + W].double())
    keep = wide.clone()
    ops.sigmoid_gate(view, proj.cuda(), 8)
    close(view, want, dtype, "gate", tol=1e-6 if dtype == "float32" else 8e-3)
    assert torch.equal(wide[:, :W], keep[:, :W]) and torch.equal(wide[:, 2 * W:], keep[:, 2 * W:])


# ---------------------------------------------------------------------- each mechanism alone
LATENT = {"hidden_size": 40, "num_heads": 3, "dim": 24, "rot_dim": 8, "vdim": 16, "kv_rank": 40, "q_rank": 32, "scale": 0.3,
          "norm_eps": 1e-5, "gate": False, "sink": True, "pairing": "neighbours"}
WINDOW = {"hidden_size": 40, "num_heads": 4, "num_kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.25, "window": 7,
          "keep_first": 3, "gate": True}
MEMORY = {"hidden_size": 40, "num_heads": 3, "dim": 24, "vdim": 40, "gate_cap": 9.0, "norm_eps": 1e-5}


def rotation(dims, base=1000.0):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    return PartSpec("rotary_stretched", {"dims": dims, "base": base})


def plain_latent(p, dims, base=1000.0):
    m = {"heads": p["num_heads"], "dim": p["dim"], "rot_dim": p["rot_dim"], "vdim": p["vdim"], "kv_rank": p["kv_rank"],
         "q_rank": p["q_rank"], "scale": p["scale"], "rot": {"base": base, "dims": dims}}

    def fn(h, ref, st):
        st = st or {"c": torch.zeros(0, p["kv_rank"], dtype=F64), "r": torch.zeros(0, p["rot_dim"], dtype=F64)}
        start = st["c"].shape[0]
        return plain.latent_attention(h, ref, "", m, p["norm_eps"], list(range(start, start + h.shape[0])), st), st
    return fn


def plain_window(p, dims, base=1000.0):
    m = {"heads": p["num_heads"], "kv_heads": p["num_kv_heads"], "dim": p["dim"], "vdim": p["vdim"], "scale": p["scale"],
         "mask": {"size": p["window"], "keep_first": p["keep_first"]}, "rot": {"base": base, "dims": dims}}

    def fn(h, ref, st):
        st = st or {"k": torch.zeros(0, m["kv_heads"], m["dim"], dtype=F64), "v": torch.zeros(0, m["kv_heads"], m["vdim"], dtype=F64)}
        start = st["k"].shape[0]
        factor = 1.0
        if not p.get("gate", True):  # a part built without its gate: the plain function reads a zero matrix, a factor 1/2
            ref, factor = dict(ref, g=torch.zeros(m["heads"] * m["vdim"], h.shape[1], dtype=F64)), 2.0
        return factor * plain.window_attention(h, ref, "", m, list(range(start, start + h.shape[0])), st), st
    return fn


def plain_memory(p):
    m = {"heads": p["num_heads"], "dim": p["dim"], "vdim": p["vdim"], "gate_cap": p["gate_cap"]}

    def fn(h, ref, st):
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        st = st or {"S": torch.zeros(H, D, Dv, dtype=F64), "n": torch.zeros(H, D, dtype=F64), "m": torch.zeros(H, dtype=F64)}
        return plain.matrix_memory(h, ref, "", m, p["norm_eps"], st), st
    return fn


def mixer_cases():
    yield "latent", "latent_attention", dict(LATENT, position=rotation(8)), plain_latent(LATENT, 8)
    yield "latent, partly rotated, one head", "latent_attention", dict(LATENT, num_heads=1, rot_dim=16, position=rotation(6)), \
        plain_latent(dict(LATENT, num_heads=1, rot_dim=16), 6)
    yield "latent, nothing rotated", "latent_attention", dict(LATENT, rot_dim=0, position=rotation(0)), \
        plain_latent(dict(LATENT, rot_dim=0), 0)
    yield "latent of a size for the tensor cores", "latent_attention", \
        dict(LATENT, kv_rank=64, rot_dim=32, num_heads=5, position=rotation(32)), plain_latent(dict(LATENT, kv_rank=64, rot_dim=32, num_heads=5), 32)
    yield "window", "kept_window_attention", dict(WINDOW, position=rotation(12)), plain_window(WINDOW, 12)
    yield "window, none kept, nothing rotated", "kept_window_attention", dict(WINDOW, keep_first=0, position=rotation(0)), \
        plain_window(dict(WINDOW, keep_first=0), 0)
    yield "window of one, more kept than the window", "kept_window_attention", \
        dict(WINDOW, window=1, keep_first=6, num_heads=2, num_kv_heads=2, position=rotation(24)), \
        plain_window(dict(WINDOW, window=1, keep_first=6, num_heads=2, num_kv_heads=2), 24)
    yield "window of sizes for the tensor cores", "kept_window_attention", \
        dict(WINDOW, dim=32, vdim=64, window=19, keep_first=21, position=rotation(16)), \
        plain_window(dict(WINDOW, dim=32, vdim=64, window=19, keep_first=21), 16)
    yield "memory", "mlstm", MEMORY, plain_memory(MEMORY)
    yield "memory, one head, wide keys", "mlstm", dict(MEMORY, num_heads=1, dim=72, vdim=8), plain_memory(dict(MEMORY, num_heads=1, dim=72, vdim=8))
    yield "memory, keys of 160", "mlstm", dict(MEMORY, num_heads=2, dim=160, vdim=24), plain_memory(dict(MEMORY, num_heads=2, dim=160, vdim=24))


CASES = {name: rest for name, *rest in mixer_cases()}


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("case", list(CASES))
def test_mixer_alone_whole_in_portions_and_beside_another_request(case, dtype):
    """A mixer on random rows: a request whole; then the same in portions down to two tokens and single tokens, beside
    another request whose portions start and end elsewhere, in slots and pages that were used before."""
    kind, params, fn = CASES[case]
    p = part("mixer", kind, params)
    bench = MixerBench(p, dtype, page_size=4, pages=96, max_tokens=256, seed=11)
    g = torch.Generator().manual_seed(12)
    x_of = {r: torch.randn(n, params["hidden_size"], generator=g).to(DT[dtype]) for r, n in (("a", 75), ("b", 31), ("c", 9))}
    want = {r: fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda rows, ctx: p.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    tol = None if dtype == "float32" else 3e-2
    close(bench.run([("c", 9)], x_of, call)["c"], want["c"], dtype, f"{case}: short request", tol)
    bench.manager.close("c")  # its slot and pages go to the next ones
    close(bench.run([("a", 75)], x_of, call)["a"], want["a"], dtype, f"{case}: whole", tol)
    bench.manager.close("a")
    got = {"a": [], "b": []}
    steps = [[("a", 2)], [("b", 5), ("a", 1)], [("a", 30), ("b", 1)], [("a", 1), ("b", 2)], [("b", 20), ("a", 2)],
             [("a", 1)], [("a", 17), ("b", 3)]] + [[("a", 1)] for _ in range(21)]
    for step in steps:
        out = bench.run(step, x_of, call)
        for r, rows in out.items():
            got[r].append(rows)
    for r in got:
        close(torch.cat(got[r]), want[r], dtype, f"{case}: request {r} in portions", tol)


def _sharp_window_scores(x, ref, p, dims, base):
    """(largest softmax weight [heads, n], the position that holds it)."""
    n, H, G, D = x.shape[0], p["num_heads"], p["num_kv_heads"], p["dim"]
    q = plain.rotate_halves((x @ ref["q"].t()).view(n, H, D), range(n), base, dims)
    k = plain.rotate_halves((x @ ref["k"].t()).view(n, G, D), range(n), base, dims)
    top, where = torch.zeros(H, n, dtype=F64), torch.zeros(H, n, dtype=torch.long)
    for i in range(n):
        read = [j for j in range(i + 1) if i - j < p["window"] or j < p["keep_first"]]
        for h in range(H):
            w = torch.softmax(k[read, h // (H // G)] @ q[i, h] * p["scale"], 0)
            a = int(w.argmax())
            top[h, i], where[h, i] = w[a], read[a]
    return top, where


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("dim,vdim", [(16, 24), (32, 64)])  # the second: sizes that the tensor-core kernel takes
def test_sharp_attention_reads_the_windows_edges_and_the_kept_tokens(dim, vdim, dtype):
    """A scale so large that nearly every query gives all its weight to one key, which random weights put anywhere:
    the window's oldest token, the query's own, the last kept token hundreds of tokens back, the very first token,
    slots at a page's border.  A key that is lost or read one token too far changes that query's output entirely.
    As a whole prompt, then in portions and single tokens."""
    n, page = 330, 8
    params = dict(WINDOW, hidden_size=32, dim=dim, vdim=vdim, scale=7.0, window=11, keep_first=5, gate=False)
    p = part("mixer", "kept_window_attention", dict(params, position=rotation(8, 10000.0)))
    bench = MixerBench(p, dtype, page_size=page, pages=64, max_tokens=512, seed=41)
    x = torch.randn(n, 32, generator=torch.Generator().manual_seed(42)).to(DT[dtype])
    want = plain_window(params, 8, 10000.0)(x.double(), bench.ref, None)[0]
    top, where = _sharp_window_scores(x.double(), bench.ref, params, 8, 10000.0)
    sharp = top > (0.9 if dtype == "float32" else 0.99)
    pos = torch.arange(n)[None, :].expand_as(where)
    assert sharp.float().mean() > 0.3
    assert int(((pos - where == params["window"] - 1) & sharp).sum()) > 3, "the window's oldest token"
    assert int(((where == pos) & sharp).sum()) > 3, "the query's own key"
    assert int(((where == params["keep_first"] - 1) & sharp & (pos > 100)).sum()) > 0, "the last kept token from far away"
    assert int(((where == 0) & sharp & (pos > 200)).sum()) > 0, "the first token from far away"
    assert int(((where < params["keep_first"]) & sharp & (pos > 20)).sum()) > 10, "kept tokens"
    rows = sharp.all(0).nonzero()[:, 0] if dtype == "bfloat16" else torch.arange(n)
    assert rows.numel() > 40
    call = lambda r, ctx: p.forward(r.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    got = bench.run([("r", n)], {"r": x}, call)["r"]
    close(got[rows], want[rows], dtype, "whole prompt")
    bench.manager.close("r")
    cuts = [47, 1, 1, 100, 1] + [2] * 30 + [17, 15, 33] + [1] * (n - 47 - 103 - 60 - 65)
    pieces = torch.cat([bench.run([("r", c)], {"r": x}, call)["r"] for c in cuts])
    close(pieces[rows], want[rows], dtype, "portions and single tokens")


@pytest.mark.parametrize("dtype", list(DT))
def test_a_far_key_in_the_latent_attention_and_a_strong_sink(dtype):
    """One key among hundreds made to stand out for one head (its latent and the head's query scaled), read from far
    away in a prompt and in single tokens; another head's sink so large that the head gives almost nothing."""
    params = dict(LATENT, hidden_size=32, scale=0.5, position=rotation(8, 10000.0))

    def tweak(dev, ref):
        for tensors, pre in ((dev, "m."), (ref, "")):
            tensors[pre + "sink"][1] = 30.0      # the second head's weight goes to its sink
            tensors[pre + "sink"][0] = -30.0     # the first head's sink takes nothing

    p = part("mixer", "latent_attention", params)
    bench = MixerBench(p, dtype, page_size=8, pages=64, max_tokens=512, seed=43, tweak=tweak)
    g = torch.Generator().manual_seed(44)
    n = 300
    x = 0.3 * torch.randn(n, 32, generator=g)
    x[37] = 4 * torch.randn(32, generator=g)  # a token whose latent is large before the norm and so points one way
    x = x.to(DT[dtype])
    fn = plain_latent(LATENT | {"hidden_size": 32, "scale": 0.5}, 8, 10000.0)
    want = fn(x.double(), bench.ref, None)[0]
    quiet = x.clone()
    quiet[37] = 0
    moved = (want - fn(quiet.double(), bench.ref, None)[0]).abs().max(dim=1).values
    assert int((moved[200:] > 0.05 * float(want.abs().max())).sum()) > 5, "token 37 is read from far away"
    call = lambda rows, ctx: p.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    close(bench.run([("r", n)], {"r": x}, call)["r"], want, dtype, "whole")
    bench.manager.close("r")
    cuts = [36, 2, 150, 3, 2] + [1] * 40 + [n - 233]
    close(torch.cat([bench.run([("r", c)], {"r": x}, call)["r"] for c in cuts]), want, dtype, "portions and single tokens")


@pytest.mark.parametrize("dtype", list(DT))
def test_an_open_forget_gate_carries_the_first_token_to_the_end(dtype):
    """Forget gates wide open (log f near zero) and input gates shut after a first token that writes the memory: what
    it wrote is still most of the output hundreds of tokens later, through portions and single tokens and beside
    another request's tokens."""
    params = dict(MEMORY, hidden_size=32, gate_cap=12.0)

    def tweak(dev, ref):
        for tensors, pre in ((dev, "m."), (ref, "")):
            tensors[pre + "f.b"].fill_(11.0)
            tensors[pre + "i.b"].fill_(-6.0)

    p = part("mixer", "mlstm", params)
    bench = MixerBench(p, dtype, page_size=8, pages=8, max_tokens=512, seed=51, tweak=tweak)
    g = torch.Generator().manual_seed(52)
    n = 400
    x = 0.02 * torch.randn(n, 32, generator=g)
    x[0] = 6 * torch.randn(32, generator=g)
    x_of = {"r": x.to(DT[dtype]), "o": torch.randn(9, 32, generator=g).to(DT[dtype])}
    fn = plain_memory(params)
    want = fn(x_of["r"].double(), bench.ref, None)[0]
    quiet = x_of["r"].clone()
    quiet[0] = 0
    assert float((want[-1] - fn(quiet.double(), bench.ref, None)[0][-1]).abs().max()) > 0.3 * float(want[-1].abs().max())
    call = lambda rows, ctx: p.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    # float32: the running maximum, a number near 6, takes 400 decrements of 7e-6, each rounded to a float32 spacing of
    # 5e-7: a random walk of some 1e-5, which exp(-m) hands on to the output
    tol = 1e-4 if dtype == "float32" else 4e-2
    close(bench.run([("r", n)], x_of, call)["r"], want, dtype, "whole", tol)
    bench.manager.close("r")
    got = []
    for step in ([("r", 1)], [("r", 2), ("o", 4)], [("r", 290)], [("o", 1), ("r", 1)], [("r", 2)], [("r", 64), ("o", 4)]) \
            + tuple([("r", 1)] for _ in range(40)):
        got.append(bench.run(list(step), x_of, call)["r"])
    close(torch.cat(got), want, dtype, "portions", tol)


def test_long_portions_of_the_memory_in_segments_side_by_side():
    """bfloat16 portions long enough for the segmented scan (every segment from an empty memory, a carry through the
    segments, then the walk that writes): two requests of unequal length side by side whose segments end inside a
    portion, a single token between two long portions, and a request that enters with a state it built earlier.
    Against the single walk on the same rounded projections the segments differ by float32 rounding only; against the
    plain implementation both carry the projections' rounding, which the division by max(|n . q|, e^-m) enlarges
    where n . q is a small difference of large terms."""
    params = dict(MEMORY, hidden_size=32, num_heads=2, dim=40, vdim=24)
    g = torch.Generator().manual_seed(62)
    x_of = {"a": torch.randn(931, 32, generator=g).to(torch.bfloat16), "b": torch.randn(330, 32, generator=g).to(torch.bfloat16)}
    results = {}
    for form in ("walk", "segments"):
        p = part("mixer", "mlstm", params)
        bench = MixerBench(p, "bfloat16", page_size=8, pages=8, max_tokens=1024, seed=61)
        assert p._segments is not None
        if form == "walk":
            p._segments = None
        call = lambda rows, ctx, p=p: p.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
        got = {"a": [], "b": []}
        for step in ([("a", 3)], [("a", 600), ("b", 300)], [("a", 1), ("b", 1)], [("a", 327), ("b", 29)]):
            for r, rows in bench.run(step, x_of, call).items():
                got[r].append(rows)
        results[form] = {r: torch.cat(rows) for r, rows in got.items()}
    fn = plain_memory(params)
    for r, x in x_of.items():
        close(results["segments"][r], results["walk"][r], "bfloat16", f"request {r}: segments against the walk", tol=8e-3)
        close(results["walk"][r], fn(x.double(), bench.ref, None)[0], "bfloat16", f"request {r}: the walk", tol=6e-2)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("W,E,top,ff,shared,rows", [(40, 5, 2, 24, 32, 3), (40, 5, 2, 24, 32, 23), (64, 3, 3, 20, None, 40),
                                                     (128, 8, 2, 48, 64, 300), (136, 6, 1, 16, None, 700)])
def test_gated_experts_whose_router_weight_scales_the_input(W, E, top, ff, shared, rows, dtype):
    """A pair at a time (few tokens, float32, inner widths that are no multiple of 16) and as grouped products."""
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    sh = None if shared is None else PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": shared, "activation": "silu",
                                                           "names": {"gate": "gate", "up": "up", "down": "down"}})
    p = part("feed_forward", "routed_experts", {"hidden_size": W, "experts": E, "top": top, "expert_ff": ff, "activation": "silu",
                                                "correction": False, "gated": True, "weigh": "input", "shared": sh})
    dev, ref = part_weights(p, dtype, seed=W + rows, scale={"router": 4.0 / W ** 0.5})  # logits of order two: scores spread out
    p.setup(Runtime(torch.device("cuda:0"), DT[dtype], 1024, 2), dict(dev))
    x = torch.randn(rows, W, generator=torch.Generator().manual_seed(rows)).to(DT[dtype])
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    want = plain.feed_forward(x.double(), ref, "", mlp)
    got = p.forward(x.cuda())
    # a near tie of two scores may fall the other way (in float32 too, against float64); such rows are left out
    score = plain.sigmoid(x.double() @ ref["router"].t()).sort(dim=1, descending=True).values
    margin = 1e-5 if dtype == "float32" else 2e-2
    clear = (score[:, top - 1] - score[:, top]).abs() > margin if top < E else torch.ones(rows, dtype=torch.bool)
    assert clear.float().mean() > (0.99 if dtype == "float32" else 0.6)
    close(got[clear], want[clear], dtype, "experts", tol=None if dtype == "float32" else 3e-2)


# ---------------------------------------------------------------------- whole models
def tolerance(dtype, cfg, w, seqs):
    """float32: 5e-5 of the largest logit.  The harness's 1e-5 is made for a handful of pre-norm layers; here up to nine
    layer runs follow one another without a norm that would take a row back to unit size, and every matrix memory
    divides by max(|n . q|, e^-m), a sum with cancellation whose float32 rounding the division hands on (measured:
    up to 1.4e-5 on these models, the same for a prompt whole, in portions and decoded, whose bits are equal).
    bfloat16: three times what rounding alone does to these prompts in the plain implementation (projections'
    operands and results rounded to bfloat16), and no less than the harness's bound."""
    if dtype == "float32":
        return 5e-5
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
    """90 tokens (150 for the third model): every window of the small models (1 to 48 tokens) passes over prompt tokens
    and over decoded ones, the kept first tokens are read from beyond the window in portions and at single tokens."""
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
@pytest.mark.parametrize("key", ["x", "z", "w"])
def test_unequal_requests_together_equal_each_alone_with_pages_and_slots_used_again(folders, key, dtype):
    """Five requests through two state slots and a pool that holds less than their sum: portions of some beside
    single tokens of others; a slot and its pages go to the next request as soon as one ends; pages that fall out of
    a window are given back while the request lives (those of the kept first tokens stay); freed pages are filled
    with NaN."""
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

    got = replay(folders[key], dtype, seqs, schedule, page_size=4, num_pages=30, max_seqs=2, poison_freed_pages=True)
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
    """300 single tokens after a short prompt, replayed from CUDA graphs: the memories and the pages are carried on the
    device from step to step, pages leave the window and are used again."""
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
    tol = tolerance(dtype, cfg, w, {"a": a, "b": b})

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
