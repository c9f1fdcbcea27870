"""The arrangements of norms, mixer and feed-forward around the residual stream: the norm before each
sub-layer (``pre_norm``), the norm after each sub-layer's sum (``post_norm``), the norm before each sub-layer
of a model that keeps several residual streams per token (``hyper_pre_norm``), and a norm on both sides of each
sub-layer (``sandwich_norm``, at the end of the file).

Pre-norm residual block: h = x + mixer(norm1(x)); y = h + feed_forward(norm2(h)).

Reference: models/transformer_block.py:38-46.  The residual stream is float32 and the sums are
fused into the norms: a block receives the previous sub-layer's output as ``pending`` and hands
its own feed-forward output on in the same way.  With a few rows in bfloat16 (decoding) the sums
and the norms move into the projections instead (``PreNormBlock.fuses``): the last projection of a
sub-layer adds into the stream, the first one of the next applies the norm, and no norm kernel runs.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..registry import create_part, register_part
from ..kernels import ops
from .base import (EMBEDDING_OUTPUT, EMBEDDING_SIDE, LAYER_REPEAT, NEXT_NORM_WEIGHT, STREAM_SUMSQ, Block, PartSpec, PendingNormed,
                   PendingStreamWrite, Runtime, StateSpec, StepContext, WeightSpec)
from .linear import Linear


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """x <- x + mixer(norm1(x)); x <- x + feed_forward(norm2(x)).  Options, all off by default:

    ``feed_forward`` (and ``norm2``) None: the block is the mixer alone.
    ``conv_taps`` = K: what each sub-layer reads, h, is first replaced by h + conv(h), a causal convolution over time
    on each channel with the tensors ``<name>.<conv1>`` (mixer) and ``<name>.<conv2>`` (feed-forward) of shape
    [width, K]: conv(h)_t = sum_j w[:, j] h_(t - K + 1 + j), zeros before the sequence's start.  The last K - 1
    inputs of both are kept per request in state slots of the block's own (``conv1``, ``conv2`` in its cache needs).
    The norm's result stays float32 until the convolution has run.
    ``reentry``: the full name of a tensor [width, 2 width]; before its first norm the block replaces the stream by
    W [stream | embedding output] (the model keeps the embedding's output for it)."""

    def __init__(self, name: str, norm1: PartSpec, mixer: PartSpec, norm2: Optional[PartSpec] = None,
                 feed_forward: Optional[PartSpec] = None, names: Optional[Dict[str, str]] = None,
                 conv_taps: Optional[int] = None, reentry: Optional[str] = None, width: int = 0):
        super().__init__(name)
        n = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feed_forward": "feed_forward", "conv1": "conv1",
             "conv2": "conv2"}
        n.update(names or {})
        self.norm1 = create_part("norm", norm1, name=f"{name}.{n['norm1']}")
        self.mixer = create_part("mixer", mixer, name=f"{name}.{n['mixer']}")
        self.norm2 = self.feed_forward = None
        if feed_forward is not None:
            if norm2 is None:
                raise ValueError(f"block {name}: a feed-forward needs the norm before it")
            self.norm2 = create_part("norm", norm2, name=f"{name}.{n['norm2']}")
            self.feed_forward = create_part("feed_forward", feed_forward, name=f"{name}.{n['feed_forward']}")
        self.conv_taps = None if conv_taps is None else int(conv_taps)
        self.reentry = reentry
        self.width = int(width)
        self.conv_tensors = [f"{name}.{n['conv1']}", f"{name}.{n['conv2']}"]
        if self.conv_taps is not None and not 1 <= self.conv_taps <= ops.INPUT_CONV_MAX_TAPS:
            raise ValueError(f"block {name}: between 1 and {ops.INPUT_CONV_MAX_TAPS} taps, got {self.conv_taps}")
        if (self.conv_taps is not None or self.reentry) and self.width <= 0:
            raise ValueError(f"block {name}: needs the stream's width")
        if self.conv_taps is not None and not hasattr(self.norm1, "add_norm_float32"):
            raise ValueError(f"block {name}: the convolution reads a norm that can leave float32 rows (add_norm_float32)")
        self.needs_embedding_output = bool(self.reentry)

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in self._parts())

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self._parts() for s in p.weight_specs()]
        if self.conv_taps is not None:
            for tensor in self.conv_tensors[: 2 if self.feed_forward is not None else 1]:
                specs.append(WeightSpec(tensor, (self.width, self.conv_taps), kind="vector", init="normal"))
        if self.reentry:
            specs.append(WeightSpec(self.reentry, (self.width, 2 * self.width)))
        return specs

    def cache_spec(self):
        need = self.mixer.cache_spec()
        if self.conv_taps is None or self.conv_taps == 1:
            return need
        needs = dict(need) if isinstance(need, dict) else ({} if need is None else {"": need})
        for label in ["conv1", "conv2"][: 2 if self.feed_forward is not None else 1]:
            if label in needs:
                raise ValueError(f"block {self.name}: its mixer already keeps something called '{label}'")
            needs[label] = StateSpec((self.conv_taps - 1, self.width), "float32")
        return needs

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        for part in self._parts():
            part.setup(rt, weights)
        if self.conv_taps is not None:
            self.conv_weights = [weights[t] for t in self.conv_tensors[: 2 if self.feed_forward is not None else 1]]
            self._conv_out = rt.shared("block.conv_out", rt.max_tokens, self.width)
        if self.reentry:
            # layers that run again (a looped span) share the tensor: every block that names it takes the same one
            self.reentry_proj = Linear(weights[self.reentry], rt, tag="block.reentry", out_dtype=torch.float32)
            self._both = rt.shared("block.reentry_in", rt.max_tokens, 2 * self.width)

    keeps_stream_stats = True

    @property
    def first_norm_weight(self) -> Optional[torch.Tensor]:
        """The weight of the norm this block applies to the stream first, if the block before may prepare
        the stream for it (see StreamStats.scaled)."""
        return self.norm1.weight if hasattr(self.norm1, "lazy") and not self.reentry else None

    def fuses(self, rows: int) -> bool:
        """A few rows (decoding) in bfloat16: the mixer's and the feed-forward's last projections add into
        the stream themselves and their first ones apply the norm, so that no norm kernel runs."""
        return (self.rt.dtype == torch.bfloat16 and self.feed_forward is not None and self.conv_taps is None
                and not self.reentry and hasattr(self.norm1, "lazy") and hasattr(self.norm2, "lazy")
                and getattr(self.mixer, "fuses_stream", False) and getattr(self.feed_forward, "fuses_stream", False)
                and self.mixer.can_fuse_stream(rows) and self.feed_forward.can_fuse_stream(rows))

    def _read(self, which: int, norm, stream: torch.Tensor, pending, ctx: StepContext, cache_id) -> torch.Tensor:
        """What sub-layer ``which`` reads: the normed stream, through the convolution if the block has one."""
        if self.conv_taps is None:
            return norm.add_norm(stream, pending)
        out = self._conv_out[: stream.shape[0]]
        state = ctx.state(cache_id, ("conv1", "conv2")[which]) if self.conv_taps > 1 else None
        if ctx.max_q_len == 1 and hasattr(norm, "add_norm_conv1"):  # single tokens: norm, convolution, state at once
            norm.add_norm_conv1(stream, pending, self.conv_weights[which], state, ctx, out)
            return out
        h = norm.add_norm_float32(stream, pending)
        ops.input_conv(h, self.conv_weights[which], state, ctx.q_start, ctx.tok_seq, ctx.slot_ids, ctx.num_seqs, out,
                       self.rt.status)
        return out

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_id: Optional[int], write_cache: bool) -> Optional[torch.Tensor]:
        shared = ctx.__dict__.setdefault("per_step", {})
        stats = shared.pop(STREAM_SUMSQ, None)  # of the stream as the block before left it
        if self.fuses(stream.shape[0]):
            x = self.norm1.lazy(stream, stats) if pending is None else None
            if x is None:  # the first block of a step, or one that nobody prepared the stream for
                x = self.norm1.add_norm(stream, pending)
            stats = self.mixer.forward(x, ctx, cache_id, write_cache, into_stream=stream,
                                       next_norm_weight=self.norm2.weight)
            shared[STREAM_SUMSQ] = self.feed_forward.forward(self.norm2.lazy(stream, stats), into_stream=stream,
                                                             next_norm_weight=shared.get(NEXT_NORM_WEIGHT))
            return None
        if self.reentry:
            both = self._both[: stream.shape[0]]
            ops.stream_concat(stream, pending, shared[EMBEDDING_OUTPUT], both)
            stream.copy_(self.reentry_proj(both))
            pending = None
        x = self._read(0, self.norm1, stream, pending, ctx, cache_id)
        a = self.mixer.forward(x, ctx, cache_id, write_cache)
        if self.feed_forward is None:
            return a
        x = self._read(1, self.norm2, stream, a, ctx, cache_id)
        return self.feed_forward.forward(x)


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """The norm after the sum: x <- norm1(alpha * x + mixer(h)); x <- norm2(alpha * x + feed_forward(x)).  The
    sub-layers read the stream itself, which the norms keep normed.  With ``token_shift`` the mixer reads

        h_t = x_t + (x_{t-1} - x_t) * mu        (mu: the tensor ``<name>.<shift>``, one value per feature)

    instead of x_t, x_{-1} = 0; the last x of a request is kept in a state slot of the block's own (``shift``
    in its cache needs) beside whatever the mixer keeps.  ``feed_forward`` may be None: the block is then the
    mixer and its norm alone.  The stream stays float32; the operands of the projections are the compute dtype.
    """

    def __init__(self, name: str, norm1: PartSpec, mixer: PartSpec, norm2: Optional[PartSpec] = None,
                 feed_forward: Optional[PartSpec] = None, alpha: float = 1.0, token_shift: bool = False,
                 width: int = 0, names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        n = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feed_forward": "feed_forward", "shift": "shift"}
        n.update(names or {})
        self.alpha = float(alpha)
        self.norm1 = create_part("norm", norm1, name=f"{name}.{n['norm1']}")
        self.mixer = create_part("mixer", mixer, name=f"{name}.{n['mixer']}")
        self.feed_forward = self.norm2 = None
        if feed_forward is not None:
            if norm2 is None:
                raise ValueError(f"block {name}: a feed-forward needs the norm that follows it")
            self.norm2 = create_part("norm", norm2, name=f"{name}.{n['norm2']}")
            self.feed_forward = create_part("feed_forward", feed_forward, name=f"{name}.{n['feed_forward']}")
        self.token_shift = bool(token_shift)
        self.shift_tensor = f"{name}.{n['shift']}"
        self.width = int(width)
        if self.width <= 0:
            raise ValueError(f"block {name}: needs the stream's width")

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in self._parts())

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self._parts() for s in p.weight_specs()]
        if self.token_shift:
            specs.append(WeightSpec(self.shift_tensor, (self.width,), kind="vector", init="normal"))
        return specs

    def cache_spec(self):
        need = self.mixer.cache_spec()
        if not self.token_shift:
            return need
        needs = dict(need) if isinstance(need, dict) else {"": need}
        if "shift" in needs:
            raise ValueError(f"block {self.name}: its mixer already keeps something called 'shift'")
        needs["shift"] = StateSpec((self.width,), "float32")
        return needs

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        for part in self._parts():
            part.setup(rt, weights)
        if self.token_shift:
            self.mu = weights[self.shift_tensor]
        self._shifted = rt.shared("block.shifted", rt.max_tokens, self.width)

    def forward(self, stream: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache_id: Optional[int], write_cache: bool) -> Optional[torch.Tensor]:
        if pending is not None:  # a block before this one left a sum open: close it without a norm
            stream.add_(pending.to(stream.dtype))
        T = stream.shape[0]
        if self.token_shift:
            h = self._shifted[:T]
            ops.token_shift(stream, self.mu, ctx.state(cache_id, "shift"), ctx.q_start, ctx.tok_seq, ctx.slot_ids, h,
                            self.rt.status)
        elif self.rt.dtype == torch.float32:
            h = stream
        else:
            h = self._shifted[:T]
            h.copy_(stream)
        a = self.mixer.forward(h, ctx, cache_id, write_cache)
        x = self.norm1.scale_add_norm(stream, a, self.alpha, want_copy=self.feed_forward is not None)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(x)
            self.norm2.scale_add_norm(stream, f, self.alpha, want_copy=False)
        return None


@register_part("block", "hyper_pre_norm")
class HyperPreNormBlock(Block):
    """Pre-norm sub-layers over S residual streams per token (hyper-connections).  Sub-layer q (1: the mixer, 2: the
    feed-forward) has three small tensors, ``<name>.hc<q>.in`` [S], ``.out`` [S] and ``.mix`` [S, S]:

        u = sum_s in[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

    The streams are one float32 tensor [T, S, W].  A sub-layer's write stays open (``PendingStreamWrite``) until the
    next norm kernel, which closes it, reads for the next sub-layer and norms in one pass over the streams; the block
    hands its last write on to the block after it (or to the model's last norm) in the same way.  ``feed_forward``
    may be None: the block is then the mixer alone."""

    def __init__(self, name: str, norm1: PartSpec, mixer: PartSpec, streams: int, width: int,
                 norm2: Optional[PartSpec] = None, feed_forward: Optional[PartSpec] = None,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        n = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feed_forward": "feed_forward", "hc1": "hc1", "hc2": "hc2"}
        n.update(names or {})
        self.streams, self.width = int(streams), int(width)
        if not 1 <= self.streams <= ops.HC_MAX_STREAMS:
            raise ValueError(f"block {name}: between 1 and {ops.HC_MAX_STREAMS} residual streams, got {self.streams}")
        self.norm1 = create_part("norm", norm1, name=f"{name}.{n['norm1']}")
        self.mixer = create_part("mixer", mixer, name=f"{name}.{n['mixer']}")
        self.feed_forward = self.norm2 = None
        if feed_forward is not None:
            if norm2 is None:
                raise ValueError(f"block {name}: a feed-forward needs the norm before it")
            self.norm2 = create_part("norm", norm2, name=f"{name}.{n['norm2']}")
            self.feed_forward = create_part("feed_forward", feed_forward, name=f"{name}.{n['feed_forward']}")
        self.hc = [f"{name}.{n['hc1']}", f"{name}.{n['hc2']}"]

    def _parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in self._parts())

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self._parts() for s in p.weight_specs()]
        S = self.streams
        for prefix in self.hc[: 2 if self.feed_forward is not None else 1]:
            specs += [WeightSpec(f"{prefix}.in", (S,), kind="vector", init="one_plus_normal"),
                      WeightSpec(f"{prefix}.out", (S,), kind="vector", init="one_plus_normal"),
                      WeightSpec(f"{prefix}.mix", (S, S), kind="vector", init="identity_plus_normal")]
        return specs

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        for part in self._parts():
            part.setup(rt, weights)
        self.coef = [(weights[f"{p}.in"], weights[f"{p}.out"], weights[f"{p}.mix"].contiguous())
                     for p in self.hc[: 2 if self.feed_forward is not None else 1]]
        self._normed = rt.shared("normed", rt.max_tokens, self.width)

    def _read_norm(self, streams: torch.Tensor, pending: Optional[PendingStreamWrite], q: int, norm) -> torch.Tensor:
        out = self._normed[: streams.shape[0]]
        ops.hc_norm(streams, None if pending is None else (pending.delta, pending.mix, pending.write), self.coef[q][0],
                    norm.weight, out, norm.eps, self.rt.status)
        return out

    def forward(self, stream: torch.Tensor, pending, ctx: StepContext, cache_id: Optional[int],
                write_cache: bool) -> Optional[PendingStreamWrite]:
        if stream.dim() != 3 or stream.shape[1] != self.streams:
            raise ValueError(f"block {self.name}: expects {self.streams} residual streams per token, got a stream of "
                             f"shape {tuple(stream.shape)}")
        if pending is not None and not isinstance(pending, PendingStreamWrite):
            raise ValueError(f"block {self.name}: the block before it left a plain sum open, not a write into streams")
        x = self._read_norm(stream, pending, 0, self.norm1)
        y = self.mixer.forward(x, ctx, cache_id, write_cache)
        pending = PendingStreamWrite(y, self.coef[0][2], self.coef[0][1])
        if self.feed_forward is not None:
            x = self._read_norm(stream, pending, 1, self.norm2)
            y = self.feed_forward.forward(x)
            pending = PendingStreamWrite(y, self.coef[1][2], self.coef[1][1])
        return pending


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after each sub-layer:

        x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(feed_forward(norm2(x)))

    The norms are parts with ``add_norm(stream, delta, extra_rows, extra_vec)`` and ``close(stream, delta, want_copy)``
    (``dynamic_tanh``): the norm after a sub-layer, the sum into the float32 stream and the norm before the next
    sub-layer are one pass over the stream.  ``feed_forward`` may be None (the block is then the mixer between its two
    norms).  Two options, both off by default:

    ``entry``: ``{"step": name of a tensor [times, width], "embedding": bool}``.  The block is the first of a span of
    layers that runs ``times`` times; at the start of run t (``ctx.per_step[LAYER_REPEAT]``) the stream takes
    ``step[t]`` and, from the second run on and if ``embedding`` is set, the embedding's output once more.  Both ride on
    the block's first norm.
    ``side``: ``{"column": c, "dim": d, "eps": e}`` and the tensors ``<name>.<side>.gate`` [d, width], ``.proj``
    [width, d] and ``.norm`` [width].  After the block's last sub-layer the stream takes a term made from a second
    embedding of the token, of whose row (``ctx.per_step[EMBEDDING_SIDE]``, looked up by the embedding part) the block
    reads the columns c .. c + d - 1:

        g = gelu_tanh(W_gate x) * row;   y = W_proj g;   x <- x + y / sqrt(mean(y^2) + e) * w_norm

    Without ``side`` the block hands its last sub-layer's output on as ``PendingNormed`` (the next block's first norm,
    or the model's last one, brings it through the norm after the sub-layer and into the stream)."""

    def __init__(self, name: str, width: int, norm1: PartSpec, norm1b: PartSpec, mixer: PartSpec,
                 norm2: Optional[PartSpec] = None, norm2b: Optional[PartSpec] = None, feed_forward: Optional[PartSpec] = None,
                 entry: Optional[dict] = None, side: Optional[dict] = None, names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        n = {"norm1": "norm1", "norm1b": "norm1b", "mixer": "mixer", "norm2": "norm2", "norm2b": "norm2b",
             "feed_forward": "feed_forward", "side": "side"}
        n.update(names or {})
        self.width = int(width)
        if self.width <= 0:
            raise ValueError(f"block {name}: needs the stream's width")
        self.norm1 = create_part("norm", norm1, name=f"{name}.{n['norm1']}")
        self.norm1b = create_part("norm", norm1b, name=f"{name}.{n['norm1b']}")
        self.mixer = create_part("mixer", mixer, name=f"{name}.{n['mixer']}")
        self.norm2 = self.norm2b = self.feed_forward = None
        if feed_forward is not None:
            if norm2 is None or norm2b is None:
                raise ValueError(f"block {name}: a feed-forward needs the norms before and after it")
            self.norm2 = create_part("norm", norm2, name=f"{name}.{n['norm2']}")
            self.norm2b = create_part("norm", norm2b, name=f"{name}.{n['norm2b']}")
            self.feed_forward = create_part("feed_forward", feed_forward, name=f"{name}.{n['feed_forward']}")
        for norm in self._norms():
            if not (hasattr(norm, "close") and hasattr(norm, "add_norm")):
                raise ValueError(f"block {name}: {type(norm).__name__} cannot stand on both sides of a sub-layer")
        self.entry = dict(entry) if entry else None
        self.side = dict(side) if side else None
        self.side_prefix = f"{name}.{n['side']}"
        if self.side and (int(self.side["dim"]) <= 0 or int(self.side["column"]) < 0):
            raise ValueError(f"block {name}: the token-side slice needs a width and a column")
        self.needs_embedding_output = bool(self.entry and self.entry.get("embedding"))

    def _norms(self):
        return [p for p in (self.norm1, self.norm1b, self.norm2, self.norm2b) if p is not None]

    def _parts(self):
        return self._norms() + [p for p in (self.mixer, self.feed_forward) if p is not None]

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in self._parts())

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self._parts() for s in p.weight_specs()]
        if self.side:
            d = int(self.side["dim"])
            specs += [WeightSpec(f"{self.side_prefix}.gate", (d, self.width)),
                      WeightSpec(f"{self.side_prefix}.proj", (self.width, d)),
                      WeightSpec(f"{self.side_prefix}.norm", (self.width,), kind="vector", init="one_plus_normal")]
        if self.entry:
            specs.append(WeightSpec(self.entry["step"], (int(self.entry["times"]), self.width), kind="vector", init="normal"))
        return specs

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        for part in self._parts():
            part.setup(rt, weights)
        if self.side:
            d = int(self.side["dim"])
            self.side_gate = Linear(weights.pop(f"{self.side_prefix}.gate"), rt, tag="block.side_gate")
            self.side_proj = Linear(weights.pop(f"{self.side_prefix}.proj"), rt, tag="block.side_proj")
            self.side_norm = weights[f"{self.side_prefix}.norm"]
            self._side_g = rt.shared("block.side_g", rt.max_tokens, d)
        if self.entry:
            self.entry_steps = weights[self.entry["step"]]  # [times, width], float32

    def forward(self, stream: torch.Tensor, pending, ctx: StepContext, cache_id: Optional[int],
                write_cache: bool):
        shared = ctx.__dict__.setdefault("per_step", {})
        extra_rows = extra_vec = None
        if self.entry:
            run = int(shared.get(LAYER_REPEAT, 0))
            if not 0 <= run < self.entry_steps.shape[0]:
                raise ValueError(f"block {self.name}: run {run} of a span that runs {self.entry_steps.shape[0]} times")
            extra_vec = self.entry_steps[run]
            if run > 0 and self.entry.get("embedding"):
                extra_rows = shared[EMBEDDING_OUTPUT]
        x = self.norm1.add_norm(stream, pending, extra_rows=extra_rows, extra_vec=extra_vec)
        a = self.mixer.forward(x, ctx, cache_id, write_cache)
        last, after = a, self.norm1b
        if self.feed_forward is not None:
            x = self.norm2.add_norm(stream, PendingNormed(a, self.norm1b))
            last, after = self.feed_forward.forward(x), self.norm2b
        if not self.side:
            return PendingNormed(last, after)
        x = after.close(stream, last, want_copy=True)
        g = self._side_g[: stream.shape[0]]
        ops.side_gate(self.side_gate(x), shared[EMBEDDING_SIDE], int(self.side["column"]), g)
        ops.add_unit_rms(stream, self.side_proj(g), self.side_norm, float(self.side["eps"]))
        return None
