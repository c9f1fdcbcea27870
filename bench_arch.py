"""``bench.py --arch binupel|bikadra|dogidra|zasalix``: another design beside Qwen3 (Zasalix: beside Dogidra, the closest
of the other designs) at equal layer sizes (random weights drawn on
the device): a prompt step of 2,048 tokens and decode steps at two batch sizes, each replayed on the device
between CUDA events, and every kernel of one eagerly launched step timed by events of its own, with the bytes
or flops it must move and the fraction of the measured copy bandwidth or bf16 throughput that this makes.

A Binupel model of ``layers`` entries repeats the pattern selective scan, RG-LRU, attention; a Bikadra model
alternates the state-space mixer and attention through a latent, over four residual streams; a Dogidra model runs
windowed attention over pooled blocks beside a minGRU in every layer, routed experts with a shared one behind them,
and a span of two layers twice; a Zasalix model repeats the pattern latent attention with a dense feed-forward, windowed
attention that keeps the first tokens beside a matrix memory with routed gated experts, a matrix memory alone with
routed gated experts, the last two as a span that runs twice; the Qwen3 model has as many layer runs of the same width, heads, head size and
(active) feed-forward width.
"""

from __future__ import annotations

import json
import statistics
import sys
import tempfile
import time

SIZES = {
    # width, feed-forward, heads, kv heads, head size, vocabulary, layers
    "2k": dict(width=2048, ff=6144, heads=16, kv_heads=8, dim=128, vocab=32000, layers=12),
    "4k": dict(width=4096, ff=12288, heads=32, kv_heads=8, dim=128, vocab=32000, layers=6),
}
PAGE = 16


def binupel_config(s):
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"],
                                          "vdim": s["dim"], "scale": s["dim"] ** -0.5,
                                          "q_temp": {"coef": 0.3, "every": 256}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    rec = {"type": "rglru", "mixer": {"width": s["width"], "blocks": s["width"] // 256, "conv": 4},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    scan = {"type": "mamba1", "mixer": {"inner": 2 * s["width"], "state": 16, "dt_rank": s["width"] // 16, "conv": 4},
            "mlp": {"kind": "dense", "ff": s["ff"]}}
    pattern = [scan, rec, att]
    return {"architecture": "Binupel", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "postln_alpha": 2.0, "layers": [pattern[i % 3] for i in range(s["layers"])]}


def bikadra_config(s):
    """State-space mixer and latent attention in turn: heads of 64 channels over twice the width with a state of 128
    in eight groups; a latent of 512 with a rotated part of 64 and heads of 128 + 64 query and 128 value dimensions."""
    ssm = {"type": "mamba2", "mixer": {"heads": 2 * s["width"] // 64, "vdim": 64, "state": 128, "groups": 8,
                                       "norm_groups": 8, "conv": 4},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    att = {"type": "latent_attention",
           "mixer": {"heads": s["heads"], "dim": s["dim"], "rot_dim": 64, "vdim": s["dim"], "kv_rank": 512,
                     "q_rank": 3 * s["width"] // 4, "scale": (s["dim"] + 64) ** -0.5,
                     "rot": {"base": 10000.0, "dims": 64,
                             "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    pattern = [ssm, att]
    return {"architecture": "Bikadra", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0},
            "streams": 4, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [pattern[i % 2] for i in range(s["layers"])]}


def dogidra_config(s):
    """Every layer: attention over a window of 1,024 tokens and blocks of 16 beside a minGRU as wide as the stream; 16
    experts of a quarter of the dense feed-forward's width, three per token, and a shared one of the same width (as
    many active rows as the dense one); four taps.  Two of the listed layers run twice, so that the layer runs are as
    many as the other model's layers."""
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                                "scale": s["dim"] ** -0.5, "softcap": 50.0, "mask": {"size": 1024, "pool": 16},
                                "rot": {"base": 10000.0, "dims": s["dim"] // 2,
                                        "scaling": {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
                       "right": {"width": s["width"]}, "left_scale": 0.7, "right_scale": 0.7},
             "mlp": {"kind": "moe", "router": {"experts": 16, "top": 3, "scale": 1.0}, "expert": {"ff": s["ff"] // 4},
                     "shared": {"ff": s["ff"] // 4}}}
    return {"architecture": "Dogidra", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "canon": {"taps": 4}, "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [layer] * (s["layers"] - 2)}


def zasalix_config(s):
    """Layer runs as in the other models: latent attention (a latent of 512 with a rotated part of 64, as the Bikadra
    model's) with a dense feed-forward; windowed attention (1,024 tokens, the first 64 kept, as wide as the Dogidra
    model's) beside a matrix memory with keys of 128 and values of 256 per head; a matrix memory alone, twice as many
    heads; the last two kinds with 16 gated experts of a quarter of the dense width, three per token, and a shared
    one.  The listed layers are runs - 2; layers 1 and 2 run twice."""
    mem = lambda heads: {"heads": heads, "dim": 128, "vdim": 256, "gate_cap": 15.0}  # noqa: E731
    moe = {"kind": "moe", "router": {"experts": 16, "top": 3}, "expert": {"ff": s["ff"] // 4}, "shared": {"ff": s["ff"] // 4}}
    lat = {"type": "latent_attention",
           "mixer": {"heads": s["heads"], "dim": s["dim"], "rot_dim": 64, "vdim": s["dim"], "kv_rank": 512,
                     "q_rank": 3 * s["width"] // 4, "scale": (s["dim"] + 64) ** -0.5, "rot": {"base": 10000.0, "dims": 64}},
           "mlp": {"kind": "dense", "ff": s["ff"]}}
    par = {"type": "parallel",
           "mixer": {"left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                              "scale": s["dim"] ** -0.5, "mask": {"size": 1024, "keep_first": 64},
                              "rot": {"base": 10000.0, "dims": s["dim"] // 2}},
                     "right": mem(s["width"] // 512), "left_scale": 0.7, "right_scale": 0.7},
           "mlp": moe}
    rec = {"type": "mlstm", "mixer": mem(s["width"] // 256), "mlp": moe}
    pattern = [lat, par, rec]
    return {"architecture": "Zasalix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "token_side": {"dim": 64}, "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [pattern[i % 3] for i in range(s["layers"] - 2)]}


def qwen3_config(s):
    return dict(architectures=["Qwen3ForCausalLM"], vocab_size=s["vocab"], hidden_size=s["width"], hidden_act="silu",
                num_hidden_layers=s["layers"], max_position_embeddings=40960, num_key_value_heads=s["kv_heads"],
                num_attention_heads=s["heads"], head_dim=s["dim"], intermediate_size=s["ff"], rms_norm_eps=1e-6,
                rope_theta=1000000.0, tie_word_embeddings=False)


def make_session(config, max_seqs, pool_tokens, step_tokens):
    from qwen3_from_scratch_b200.engine.session import Session
    from qwen3_from_scratch_b200.registry import config_from_dict
    with tempfile.TemporaryDirectory(prefix="q3b200-arch-") as tmp:
        config_from_dict(config).save(tmp)
        return Session(tmp, dtype="bfloat16", page_size=PAGE, num_pages=pool_tokens // PAGE + max_seqs, max_seqs=max_seqs,
                       max_step_tokens=step_tokens, random_weights=0)


def time_replays(session, steps, warmup):
    """Median milliseconds of one replay of the session's last step (a CUDA graph once its shape has come
    twice), every replay between events of its own; a buffer larger than L2 is written between replays."""
    import torch
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        session.rerun_last()
    out = []
    for _ in range(steps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        session.rerun_last()
        end.record()
        torch.cuda.synchronize()
        out.append(start.elapsed_time(end))
    return statistics.median(out)


class KernelClock:
    """Wraps the launchers of ``kernels.ops`` (and the projections' library products) with CUDA events and the
    work each call must do, for one eagerly launched step."""

    def __init__(self, scenario):
        self.scenario = scenario
        self.rows = {}
        self.pending = []
        self.saved = []

    # what a call must move: ("bytes", n) against the copy bandwidth or ("flops", n) against the bf16 peak
    def work(self, name, a, k):
        sc = self.scenario
        size = lambda t: t.numel() * t.element_size()  # noqa: E731
        if name in ("add_rmsnorm", "scale_add_rmsnorm"):
            resid, delta, out = a[0], a[1], a[3]
            n = size(resid) * (2 if (delta is not None or name == "scale_add_rmsnorm") else 1)
            return "bytes", n + (size(delta) if delta is not None else 0) + (size(out) if out is not None else 0)
        if name == "add_rmsnorm_rows":
            return "bytes", size(a[4]) * 3
        if name == "token_shift":
            return "bytes", size(a[0]) + size(a[6])
        if name == "causal_conv":
            return "bytes", 2 * size(a[10])
        if name in ("gated_act", "swiglu"):
            return "bytes", size(a[0]) + size(a[1])
        if name == "qk_gate_post":
            proj, q_out, pages = a[0], a[1], a[2]
            return "bytes", size(proj) + size(q_out) + 2 * proj.shape[0] * pages.shape[1] * pages.shape[3] * proj.element_size()
        if name == "qkv_post":
            qkv, q_out, pages = a[0], a[1], a[2]
            return "bytes", size(qkv) + size(q_out) + 2 * qkv.shape[0] * pages.shape[1] * pages.shape[3] * qkv.element_size()
        if name == "gemm_tc_qkv":
            x, w = a[0], a[1]
            return "flops", 2 * x.shape[0] * w.shape[0] * w.shape[1]
        if name == "rglru_scan":
            u, gates, out = a[3], a[4], a[13]
            twice = 2 if k.get("scratch") is not None and sc["kind"] == "prefill" else 1
            return "bytes", twice * (size(gates) + size(u)) + size(u) + size(out)
        if name == "selective_scan":
            xc, bc, dt, out = a[0], a[3], a[4], a[12]
            twice = 2 if k.get("scratch") is not None and sc["kind"] == "prefill" else 1
            return "bytes", twice * (size(xc) + size(bc) + size(dt)) + size(xc) + size(out)
        if name in ("sigmoid_attention", "paged_attention"):
            q, pages = a[0], a[1]
            hq, d, hkv = q.shape[1], q.shape[2], pages.shape[1]
            if sc["kind"] == "prefill":
                return "flops", 4 * hq * d * sc["tokens"] * (sc["tokens"] + 1) // 2
            return "bytes", sc["batch"] * sc["context"] * hkv * d * 2 * pages.element_size() + 2 * size(q)
        if name == "block_diag":
            u, w = a[0], a[1]
            if u.shape[0] <= 16:
                return "bytes", size(w)
            return "flops", 2 * u.shape[0] * w.shape[0] * w.shape[1] * w.shape[2]
        if name in ("gemm_skinny", "gemm_skinny_normed", "gemm_skinny_into_stream"):
            w = a[1] if name != "gemm_skinny_normed" else a[4]
            return "bytes", size(w)
        if name == "gemm_tc":
            return "flops", 2 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
        if name == "library product":
            x, w = a
            if x.shape[0] <= 64:
                return "bytes", size(w)
            return "flops", 2 * x.shape[0] * w.shape[0] * w.shape[1]
        if name == "embed":
            return "bytes", size(a[2]) * 1.5
        if name == "embed_scaled":
            return "bytes", size(a[2]) * (1 + 0.5 / a[2].shape[1])
        if name == "hc_norm":
            streams, pending, out = a[0], a[1], a[4]
            return "bytes", size(streams) * (2 if pending is not None else 1) + size(out) * (2 if pending is not None else 1)
        if name == "act":
            return "bytes", size(a[0]) + size(a[1])
        if name == "latent_kv_post":
            proj, c_pages, r_pages, cq, gate = a[0], a[16], a[17], a[18], a[19]
            return "bytes", (size(proj) + size(cq) + (size(gate) if gate is not None else 0)
                             + proj.shape[0] * (c_pages.shape[3] + r_pages.shape[3]) * 2)
        if name == "add_dyt":
            stream, delta, out = a[0], a[1], a[4]
            n = size(stream) * (2 if (delta is not None or k.get("rows_add") is not None or k.get("vec_add") is not None) else 1)
            n += size(k["rows_add"]) if k.get("rows_add") is not None else 0
            return "bytes", n + (size(delta) if delta is not None else 0) + (size(out) if out is not None else 0)
        if name == "add_unit_rms":
            return "bytes", 2 * size(a[0]) + size(a[1])
        if name == "side_gate":
            return "bytes", 2 * size(a[0]) + a[0].numel() * 4
        if name == "sigmoid_gate":
            x = a[0]
            return "bytes", 3 * x.numel() * x.element_size()
        if name == "mlstm_scan":
            # what the walk must move: q, k, v and the result once, and the state in and out; against the copy bandwidth
            memory, out = a[9], a[15]
            H, D, Dv = memory.shape[1], memory.shape[2], memory.shape[3]
            seqs = 1 if sc["kind"] == "prefill" else sc["batch"]
            return "bytes", out.shape[0] * H * (2 * D + Dv) * a[0].element_size() + size(out) + 2 * seqs * H * D * Dv * 4
        if name == "mlstm_out":
            o, out = a[0], a[5]
            return "bytes", size(o) + 2 * out.numel() * out.element_size()
        if name == "latent_q_post":
            return "bytes", 2 * size(a[0])
        if name == "gate_heads":
            return "bytes", size(a[0]) + (size(a[1]) if a[1] is not None else 0) + size(a[2])
        if name == "latent_attention":
            q_abs, q_rot, c_pages = a[0], a[1], a[2]
            H, _, rank = q_abs.shape
            rot = q_rot.shape[2]
            if sc["kind"] == "prefill":
                return "flops", 2 * H * (2 * rank + rot) * sc["tokens"] * (sc["tokens"] + 1) // 2
            return "bytes", sc["batch"] * sc["context"] * (rank + rot) * c_pages.element_size() + size(q_abs) + size(a[6])
        if name == "ssd_scan":
            xbc, y = a[0], a[10]
            twice = 2 if k.get("scratch") is not None and sc["kind"] == "prefill" else 1
            return "bytes", twice * size(xbc) + size(y)
        if name == "gated_group_norm":
            y, out = a[0], a[4]
            return "bytes", size(y) + 2 * size(out)
        if name == "add_layernorm":
            stream, delta, out = a[0], a[1], a[4]
            return "bytes", size(stream) * (2 if delta is not None else 1) + (size(delta) if delta is not None else 0) + size(out)
        if name == "add_layernorm_conv1":
            stream, delta, state, out = a[0], a[1], a[5], a[8]
            n = size(stream) * (2 if delta is not None else 1) + (size(delta) if delta is not None else 0) + size(out)
            return "bytes", n + (2 * stream.shape[0] * state.shape[1] * state.shape[2] * 4 if state is not None else 0)
        if name == "input_conv":
            return "bytes", size(a[0]) + size(a[7])
        if name == "stream_concat":
            return "bytes", size(a[0]) + size(a[2]) + size(a[3]) + (size(a[1]) if a[1] is not None else 0)
        if name == "pw_qkv_post":
            proj, heads, kv_heads, dim, vdim = a[0], a[4], a[5], a[6], a[7]
            n = proj.shape[0] * proj.element_size()
            return "bytes", n * (2 * heads * dim + 2 * kv_heads * (dim + vdim))
        if name == "pool_blocks":
            k_pages, v_pages = a[0], a[1]
            n = sc["tokens"] if sc["kind"] == "prefill" else sc["batch"]
            return "bytes", n * k_pages.shape[1] * (k_pages.shape[3] + v_pages.shape[3]) * k_pages.element_size() * (1 + 1 / a[10])
        if name == "pooled_window_attention":
            q, k_pages, v_pages, window, pool = a[0], a[1], a[2], a[9], a[10]
            H, D = q.shape[1], q.shape[2]
            G, Dv = k_pages.shape[1], v_pages.shape[3]
            limit = k.get("block_limit", -1)
            blocks = lambda i: max(0, i + 1 - window) // pool  # noqa: E731
            seen = lambda i: min(i + 1, window) + (blocks(i) if limit < 0 else min(blocks(i), limit))  # noqa: E731
            if sc["kind"] == "prefill":
                return "flops", 2 * H * (D + Dv) * sum(seen(i) for i in range(sc["tokens"]))
            return "bytes", sc["batch"] * seen(sc["context"] - 1) * G * (D + Dv) * k_pages.element_size() + 2 * size(q)
        if name == "mingru_scan":
            out = a[10]
            return "bytes", 4 * out.numel() * out.element_size()
        if name == "moe_route":
            return "bytes", size(a[0]) + size(a[1])
        if name == "routed_experts":
            h, up, down, ids = a[0], a[1], a[2], a[3]
            pairs = ids.numel()
            # the experts' matrices that the step touches (at most all of them) or the products, whichever takes
            # longer at 240 bf16 flops per byte of HBM (about the ratio of the two measured peaks)
            touched = min(pairs, up.shape[0]) * (size(up) + size(down)) // up.shape[0]
            flops = (6 if k.get("gate_block") else 4) * pairs * down.shape[2] * up.shape[2]
            return ("bytes", touched) if touched * 240 > flops else ("flops", flops)
        return "bytes", 0

    def wrap(self, owner, attr, name):
        import torch
        real = getattr(owner, attr)

        def timed(*a, **k):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = real(*a, **k)
            end.record()
            self.pending.append((name, start, end, self.work(name, a, k)))
            return out

        self.saved.append((owner, attr, real))
        setattr(owner, attr, timed)

    def __enter__(self):
        import torch
        from qwen3_from_scratch_b200.kernels import ops
        for name in ("embed", "add_rmsnorm", "add_rmsnorm_rows", "scale_add_rmsnorm", "token_shift", "causal_conv",
                     "gated_act", "swiglu", "qk_gate_post", "qkv_post", "gemm_tc_qkv", "rglru_scan", "selective_scan",
                     "sigmoid_attention", "paged_attention", "block_diag", "gemm_skinny", "gemm_skinny_normed",
                     "gemm_skinny_into_stream", "gemm_tc", "embed_scaled", "hc_norm", "act", "latent_kv_post",
                     "latent_q_post", "gate_heads", "latent_attention", "ssd_scan", "gated_group_norm", "add_layernorm",
                     "add_layernorm_conv1", "input_conv", "stream_concat", "pw_qkv_post", "pool_blocks", "pooled_window_attention",
                     "mingru_scan", "moe_route", "routed_experts", "add_dyt", "add_unit_rms", "side_gate", "sigmoid_gate",
                     "mlstm_scan", "mlstm_out"):
            self.wrap(ops, name, name)
        real_mm = torch.mm
        clock = self

        def mm(x, wt, **k):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = real_mm(x, wt, **k)
            end.record()
            clock.pending.append(("library product", start, end, clock.work("library product", (x, wt.t()), {})))
            return out

        self.saved.append((torch, "mm", real_mm))
        torch.mm = mm
        return self

    def __exit__(self, *exc):
        import torch
        for owner, attr, real in self.saved:
            setattr(owner, attr, real)
        torch.cuda.synchronize()
        for name, start, end, (kind, amount) in self.pending:
            row = self.rows.setdefault((name, kind), {"calls": 0, "us": 0.0, "work": 0.0})
            row["calls"] += 1
            row["us"] += start.elapsed_time(end) * 1e3
            row["work"] += amount

    def table(self, peaks):
        out = {}
        for (name, kind), row in sorted(self.rows.items(), key=lambda kv: -kv[1]["us"]):
            rate = row["work"] / (row["us"] * 1e-6) if row["us"] > 0 else 0.0
            peak = peaks["hbm_gbs"] * 1e9 if kind == "bytes" else peaks["bf16_tflops"] * 1e12
            out[f"{name} ({'HBM' if kind == 'bytes' else 'bf16'})"] = {
                "calls": row["calls"], "us": round(row["us"], 1), "fraction_of_measured_peak": round(rate / peak, 3)}
        return out


def run_scenario(config, scenario, steps, warmup, peaks):
    """One model in one scenario: the step's time replayed, and its kernels' times in an eager launch."""
    import torch
    from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
    vocab = config.get("vocab", config.get("vocab_size"))
    g = torch.Generator().manual_seed(5)
    ids = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()  # noqa: E731
    if scenario["kind"] == "prefill":
        T = scenario["tokens"]
        session = make_session(config, 2, T + 64, T)
        entries = [Entry("p", ids(T), [T - 1])]
        session.prepare(entries)
        for _ in range(3):  # the shape's second appearance records its graph
            session._run(entries)
        tokens = T
    else:
        B, C = scenario["batch"], scenario["context"]
        session = make_session(config, B, B * (C + PAGE), 2048)
        for b in range(B):
            left = C - 1
            while left > 0:
                n = min(left, 2048)
                session.step([Entry(b, ids(n), [])])
                left -= n
        entries = [Entry(b, ids(1), [0]) for b in range(B)]
        session.prepare(entries)
        for _ in range(3):
            session._run(entries)
        tokens = B
    torch.cuda.synchronize()
    ms = time_replays(session, steps, warmup)
    with KernelClock(scenario) as clock:
        ctx = BatchContext(session.manager, session.storage, session.rt).build(entries, session.vocab_size)
        session.model.step(ctx)
    session.check_status()
    result = {"ms_per_step": round(ms, 4), "tokens_per_s": round(tokens / (ms * 1e-3), 1),
              "graph": session.last_graph is not None, "kernels": clock.table(peaks)}
    del session
    torch.cuda.empty_cache()
    return result


def compare(args, peaks, sample_clocks):
    size = SIZES[args.arch_size]
    scenarios = {"prefill_2048": {"kind": "prefill", "tokens": 2048},
                 "decode_b8_ctx2048": {"kind": "decode", "batch": 8, "context": 2048},
                 "decode_b64_ctx2048": {"kind": "decode", "batch": 64, "context": 2048}}
    sampler = sample_clocks()
    t0 = time.time()
    other = {"binupel": binupel_config, "bikadra": bikadra_config, "dogidra": dogidra_config,
             "zasalix": zasalix_config}[args.arch]
    # what the design stands beside: Qwen3, or for Zasalix the closest of the other designs (a windowed attention
    # beside a recurrence, routed experts, a span of layers that runs twice)
    beside, beside_config = ("dogidra", dogidra_config) if args.arch == "zasalix" else ("qwen3", qwen3_config)
    out = {"arch": args.arch, "beside": beside, "sizes": dict(size, name=args.arch_size), "dtype": "bf16",
           "data": "synthetic tokens, random weights drawn on the device", "steps": args.steps, "warmup": args.warmup,
           "peaks": peaks, "timing": "CUDA events around each replay of the step; 256 MB written between replays",
           args.arch: {}, beside: {}}
    for name, scenario in scenarios.items():
        for model, config in ((args.arch, other(size)), (beside, beside_config(size))):
            out[model][name] = run_scenario(config, scenario, args.steps, args.warmup, peaks)
            print(f"[bench] {model} {name}: {out[model][name]['ms_per_step']} ms", file=sys.stderr, flush=True)
    out["clocks"] = sampler.stop()
    # the sampler runs from before the models are made: where making them takes long most samples see an idle GPU, so the
    # median of the samples taken under load (at half of the top clock or more) is given beside the median of all
    busy = [s[0] for s in getattr(sampler, "samples", []) if s[1] and s[0] >= 0.5 * s[1]]
    out["clocks"]["sm_mhz_under_load"] = statistics.median(busy) if busy else None
    out["clocks"]["samples_under_load"] = len(busy)
    out["seconds"] = round(time.time() - t0, 1)
    print(json.dumps(out))
    return 0
