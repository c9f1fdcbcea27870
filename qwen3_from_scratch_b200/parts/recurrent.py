"""Mixers that carry a state of fixed size from token to token instead of a cache of keys.

``rglru``           the recurrent block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with
                    Local Attention for Efficient Language Models"): two branches of ``width`` channels,
                    y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x); block-diagonal gates
                    r = sigmoid(R_b u_b + b), i = sigmoid(I_b u_b + b); a = exp(-decay * softplus(lam) * r);
                    S_t = a S_{t-1} + sqrt(1 - a^2) (i * u); out = W_o (S * y).
``selective_scan``  the mixer of Mamba (Gu and Dao, "Mamba: Linear-Time Sequence Modeling with Selective State
                    Spaces"): [x | z] = W_in h; x = silu(conv(x)); [dt | B | C] = W_x x;
                    step = softplus(W_dt dt + b); S[c, n] = exp(step_c A[c, n]) S[c, n] + step_c x_c B_n;
                    y_c = sum_n S[c, n] C_n + D_c x_c; out = W_o (y * silu(z)).

``mlstm``           the matrix memory of the xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory"): per head a
                    memory S [dim, vdim] with exponential input and forget gates kept stable by a running maximum
                    (see the class).

The first two keep two things per request, named in ``cache_spec()``: ``state`` (float32) and ``conv`` (the last
taps - 1 inputs of the short convolution, float32).  A new request's slot is zero.  The projections are
``Linear``s (the compute dtype, float32 accumulation); decays, step sizes, gates and the state are float32 in
every run; a portion of a prompt is walked token by token in the same order as the whole prompt.
The names of the tensors are parameters (``names``), with the defaults below.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import Mixer, Runtime, StateSpec, StepContext, WeightSpec
from .linear import Linear


class _NamedTensors:
    def _name_tensors(self, name: str, defaults: Dict[str, str], names: Optional[Dict[str, str]]) -> None:
        n = dict(defaults)
        n.update(names or {})
        self.tensors = {k: f"{name}.{v}" for k, v in n.items()}


@register_part("mixer", "rglru")
class RGLRU(Mixer, _NamedTensors):
    graph_capturable = True
    NAMES = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
             "gate_a": "ra", "gate_a_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "out": "o"}

    def __init__(self, name: str, hidden_size: int, width: int, blocks: int, conv: int, decay: float = 8.0,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.width, self.blocks, self.taps = int(hidden_size), int(width), int(blocks), int(conv)
        if self.width % self.blocks:
            raise ValueError(f"{self.width} channels are not a multiple of {self.blocks} blocks")
        self.block_width = self.width // self.blocks
        self.decay = float(decay)
        self._name_tensors(name, self.NAMES, names)

    def weight_specs(self) -> List[WeightSpec]:
        t, h, c, nb, bw = self.tensors, self.hidden_size, self.width, self.blocks, self.block_width
        return [WeightSpec(t["y"], (c, h)), WeightSpec(t["y_bias"], (c,), kind="vector", init="normal"),
                WeightSpec(t["x"], (c, h)), WeightSpec(t["x_bias"], (c,), kind="vector", init="normal"),
                WeightSpec(t["conv"], (c, self.taps), kind="vector", init="normal"),
                WeightSpec(t["conv_bias"], (c,), kind="vector", init="normal"),
                WeightSpec(t["gate_a"], (nb, bw, bw)), WeightSpec(t["gate_a_bias"], (nb, bw), kind="vector", init="normal"),
                WeightSpec(t["gate_i"], (nb, bw, bw)), WeightSpec(t["gate_i_bias"], (nb, bw), kind="vector", init="normal"),
                WeightSpec(t["lam"], (c,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["out"], (h, c))]

    def cache_spec(self):
        return {"state": StateSpec((self.width,), "float32"),
                "conv": StateSpec((self.taps - 1, self.width), "float32")}

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        t, c = self.tensors, self.width
        y, x = weights.pop(t["y"]), weights.pop(t["x"])
        dtype = torch.float32 if torch.float32 in (y.dtype, x.dtype) else y.dtype
        self.proj = Linear(torch.cat([y.to(dtype), x.to(dtype)], dim=0), rt, tag="rglru.proj")  # columns: y, then x
        del y, x
        self.y_bias, self.x_bias = weights[t["y_bias"]], weights[t["x_bias"]]
        self.conv_weight, self.conv_bias = weights[t["conv"]], weights[t["conv_bias"]]
        ga, gi = weights.pop(t["gate_a"]), weights.pop(t["gate_i"])
        # per block the rows of the recurrence gate, then those of the input gate: one product gives both
        self.gate_weight = torch.cat([ga, gi], dim=1).to(rt.dtype).contiguous()
        del ga, gi
        self.gate_a_bias = weights[t["gate_a_bias"]].reshape(-1).contiguous()
        self.gate_i_bias = weights[t["gate_i_bias"]].reshape(-1).contiguous()
        self.lam = weights[t["lam"]]
        self.out_proj = Linear(weights.pop(t["out"]), rt, tag="rglru.out")
        self._u = rt.shared("rglru.u", rt.max_tokens, c)
        self._gates = rt.shared("rglru.gates", rt.max_tokens * 2 * c, dtype=torch.float32)
        self._gated = rt.shared("rglru.gated", rt.max_tokens, c)
        self._chunks = None
        if rt.dtype == torch.bfloat16:
            self._chunks = rt.shared("rglru.chunks", ops.scan_chunk_records(rt.max_tokens, rt.max_seqs) * 2 * c,
                                     dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        T, c, bw = x.shape[0], self.width, self.block_width
        status = self.rt.status
        proj = self.proj(x)
        u = self._u[:T]
        ops.causal_conv(proj, c, self.x_bias, self.conv_weight, self.conv_bias, ctx.state(cache_id, "conv"), ctx.q_start,
                        ctx.tok_seq, ctx.slot_ids, ctx.num_seqs, u, "none", status)
        gates = self._gates[: T * 2 * c].view(self.blocks, T, 2 * bw)
        ops.block_diag(u, self.gate_weight, gates)
        gated = self._gated[:T]
        ops.rglru_scan(proj, 0, self.y_bias, u, gates, self.gate_a_bias, self.gate_i_bias, self.lam, self.decay,
                       ctx.state(cache_id, "state"), ctx.q_start, ctx.slot_ids, ctx.num_seqs, gated, status,
                       max_q_len=ctx.max_q_len, scratch=self._chunks)
        return self.out_proj(gated)


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer, _NamedTensors):
    graph_capturable = True
    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b",
             "a_log": "A_log", "d": "D", "out": "o"}

    def __init__(self, name: str, hidden_size: int, inner: int, state: int, dt_rank: int, conv: int,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.inner, self.state_size = int(hidden_size), int(inner), int(state)
        self.dt_rank, self.taps = int(dt_rank), int(conv)
        self._name_tensors(name, self.NAMES, names)

    def weight_specs(self) -> List[WeightSpec]:
        t, h, i, n, r = self.tensors, self.hidden_size, self.inner, self.state_size, self.dt_rank
        return [WeightSpec(t["in"], (2 * i, h)),
                WeightSpec(t["conv"], (i, self.taps), kind="vector", init="normal"),
                WeightSpec(t["conv_bias"], (i,), kind="vector", init="normal"),
                WeightSpec(t["x"], (r + 2 * n, i)),
                WeightSpec(t["dt"], (i, r)), WeightSpec(t["dt_bias"], (i,), kind="vector", init="normal"),
                WeightSpec(t["a_log"], (i, n), kind="vector", init="normal"),
                WeightSpec(t["d"], (i,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["out"], (h, i))]

    def cache_spec(self):
        return {"state": StateSpec((self.state_size, self.inner), "float32"),
                "conv": StateSpec((self.taps - 1, self.inner), "float32")}

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        t, i, n, r = self.tensors, self.inner, self.state_size, self.dt_rank
        self.in_proj = Linear(weights.pop(t["in"]), rt, tag="scan.in")  # columns: x, then z
        self.conv_weight, self.conv_bias = weights[t["conv"]], weights[t["conv_bias"]]
        wx = weights.pop(t["x"])
        # the low-rank step sizes feed another product, so they come out in the compute dtype; B and C enter the
        # recurrence and come out in float32
        self.dt_low = Linear(wx[:r].contiguous(), rt, tag="scan.dt_low")
        self.bc_proj = Linear(wx[r:].contiguous(), rt, tag="scan.bc", out_dtype=torch.float32)
        del wx
        self.dt_proj = Linear(weights.pop(t["dt"]), rt, tag="scan.dt", out_dtype=torch.float32)
        self.dt_bias, self.a_log, self.d_skip = weights[t["dt_bias"]], weights[t["a_log"]], weights[t["d"]]
        self.out_proj = Linear(weights.pop(t["out"]), rt, tag="scan.out")
        self._xc = rt.shared("scan.xc", rt.max_tokens, i)
        self._y = rt.shared("scan.y", rt.max_tokens, i)
        self._chunks = None
        if rt.dtype == torch.bfloat16:
            self._chunks = rt.shared("scan.chunks", ops.scan_chunk_records(rt.max_tokens, rt.max_seqs) * (n + 1) * i,
                                     dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        T, i = x.shape[0], self.inner
        status = self.rt.status
        proj = self.in_proj(x)
        xc = self._xc[:T]
        ops.causal_conv(proj, 0, None, self.conv_weight, self.conv_bias, ctx.state(cache_id, "conv"), ctx.q_start,
                        ctx.tok_seq, ctx.slot_ids, ctx.num_seqs, xc, "silu", status)
        bc = self.bc_proj(xc)
        dt = self.dt_proj(self.dt_low(xc))
        y = self._y[:T]
        ops.selective_scan(xc, proj, i, bc, dt, self.dt_bias, self.a_log, self.d_skip, ctx.state(cache_id, "state"),
                           ctx.q_start, ctx.slot_ids, ctx.num_seqs, y, status, max_q_len=ctx.max_q_len,
                           scratch=self._chunks)
        return self.out_proj(y)


@register_part("mixer", "ssd")
class SSD(Mixer, _NamedTensors):
    """The mixer of Mamba-2 (Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms Through
    Structured State Space Duality"): a state-space recurrence with one scalar decay per head.  With inner =
    heads * vdim, N = state, G = groups:

        W_in h = [z: inner | x: inner | B: G N | C: G N | dt: heads];   [x | B | C] <- silu(conv([x | B | C]))
        step = softplus(dt + dt_bias);   S_h <- exp(-exp(A_log_h) step) S_h + step B_g x_h^T   (S_h: N x vdim)
        y_h = S_h^T C_g + D_h x_h;   out = W_o (unit_rms_per_part(y * silu(z)) * norm)

    (head h reads group h // (heads / G); the gated y is cut into ``norm_groups`` equal parts, each divided by its
    own root mean square).  Per request it keeps ``state`` (float32 [heads, N, vdim]) and ``conv`` (the last taps - 1
    inputs of the convolution, float32); a new request's slot is zero.  Step sizes, decays, the state and the norm
    are float32 in every run."""

    graph_capturable = True
    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D",
             "norm": "norm", "out": "o"}

    def __init__(self, name: str, hidden_size: int, num_heads: int, vdim: int, state: int, groups: int, norm_groups: int,
                 conv: int, norm_eps: float, names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.num_heads, self.vdim = int(hidden_size), int(num_heads), int(vdim)
        self.state_size, self.groups, self.norm_groups, self.taps = int(state), int(groups), int(norm_groups), int(conv)
        self.norm_eps = float(norm_eps)
        self.inner = self.num_heads * self.vdim
        if self.num_heads % self.groups or self.inner % self.norm_groups:
            raise ValueError(f"{self.num_heads} heads / {self.groups} groups / {self.norm_groups} norm groups do not divide")
        self.channels = self.inner + 2 * self.groups * self.state_size  # what the convolution runs over
        self._name_tensors(name, self.NAMES, names)

    def weight_specs(self) -> List[WeightSpec]:
        t, w, H = self.tensors, self.hidden_size, self.num_heads
        return [WeightSpec(t["in"], (self.inner + self.channels + H, w)),
                WeightSpec(t["conv"], (self.channels, self.taps), kind="vector", init="normal"),
                WeightSpec(t["conv_bias"], (self.channels,), kind="vector", init="normal"),
                WeightSpec(t["dt_bias"], (H,), kind="vector", init="normal"),
                WeightSpec(t["a_log"], (H,), kind="vector", init="normal"),
                WeightSpec(t["d"], (H,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["norm"], (self.inner,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["out"], (w, self.inner))]

    def cache_spec(self):
        return {"state": StateSpec((self.num_heads, self.state_size, self.vdim), "float32"),
                "conv": StateSpec((self.taps - 1, self.channels), "float32")}

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        t = self.tensors
        w_in = weights.pop(t["in"])
        pad = torch.zeros((-w_in.shape[0]) % 8, w_in.shape[1], dtype=w_in.dtype, device=w_in.device)
        self.in_proj = Linear(torch.cat([w_in, pad], dim=0), rt, tag="ssd.in")  # columns: z, x, B, C, dt
        del w_in
        self.conv_weight, self.conv_bias = weights[t["conv"]], weights[t["conv_bias"]]
        self.dt_bias, self.a_log, self.d_skip = weights[t["dt_bias"]], weights[t["a_log"]], weights[t["d"]]
        self.norm_weight = weights[t["norm"]]
        self.out_proj = Linear(weights.pop(t["out"]), rt, tag="ssd.out")
        self._xbc = rt.shared("ssd.xbc", rt.max_tokens, self.channels)
        self._y = rt.shared("ssd.y", rt.max_tokens, self.inner, dtype=torch.float32)
        self._gated = rt.shared("ssd.gated", rt.max_tokens, self.inner)
        self._chunks = None
        if rt.dtype == torch.bfloat16 and ops.ssd_chunked_pays(rt.dtype, rt.max_tokens):
            self._chunks = rt.shared("ssd.chunks", ops.ssd_scratch_numel(rt.max_tokens, rt.max_seqs, self.num_heads,
                                                                         self.vdim, self.state_size), dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        T, inner = x.shape[0], self.inner
        status = self.rt.status
        proj = self.in_proj(x)
        xbc = self._xbc[:T]
        ops.causal_conv(proj, inner, None, self.conv_weight, self.conv_bias, ctx.state(cache_id, "conv"), ctx.q_start,
                        ctx.tok_seq, ctx.slot_ids, ctx.num_seqs, xbc, "silu", status)
        y = self._y[:T]
        ops.ssd_scan(xbc, proj, inner + self.channels, self.dt_bias, self.a_log, self.d_skip, ctx.state(cache_id, "state"),
                     ctx.q_start, ctx.slot_ids, ctx.num_seqs, y, self.num_heads, self.vdim, self.state_size, self.groups,
                     status, max_q_len=ctx.max_q_len, scratch=self._chunks)
        gated = self._gated[:T]
        ops.gated_group_norm(y, proj, 0, self.norm_weight, gated, self.norm_groups, self.norm_eps)
        return self.out_proj(gated)


@register_part("mixer", "mingru")
class MinGRU(Mixer, _NamedTensors):
    """A gated recurrence whose gates read only the current token (the minGRU of Feng et al., "Were RNNs All We
    Needed?", with the candidate's activation continued linearly above zero).  With h the input and C channels:

        z = sigmoid(W_z h + b_z);  u = W_x h + b_x;  candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0
        S_t = (1 - z) S_(t-1) + z candidate      element by element, S float32, zero for a new request
        out = W_o (S_t silu(W_g h))

    Everything but the projections is float32.  ``names``: the tensors' names after the part's own."""

    graph_capturable = True
    splittable = True
    NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "gate": "g", "out": "o"}

    def __init__(self, name: str, hidden_size: int, width: int, names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.width = int(hidden_size), int(width)
        self._name_tensors(name, self.NAMES, names)

    def weight_specs(self) -> List[WeightSpec]:
        t, h, c = self.tensors, self.hidden_size, self.width
        return [WeightSpec(t["z"], (c, h)), WeightSpec(t["z_bias"], (c,), kind="vector", init="normal"),
                WeightSpec(t["x"], (c, h)), WeightSpec(t["x_bias"], (c,), kind="vector", init="normal"),
                WeightSpec(t["gate"], (c, h)), WeightSpec(t["out"], (h, c))]

    def cache_spec(self):
        return StateSpec((self.width,), "float32")

    def input_weight(self, weights: Dict[str, torch.Tensor]) -> torch.Tensor:
        t = self.tensors
        z, x, g = weights.pop(t["z"]), weights.pop(t["x"]), weights.pop(t["gate"])
        dtype = torch.float32 if torch.float32 in (z.dtype, x.dtype, g.dtype) else z.dtype
        return torch.cat([z.to(dtype), x.to(dtype), g.to(dtype)], dim=0)  # columns of the product: z, u, g

    def output_weight(self, weights: Dict[str, torch.Tensor]) -> torch.Tensor:
        return weights.pop(self.tensors["out"])

    @property
    def input_rows(self) -> int:
        return 3 * self.width

    @property
    def output_columns(self) -> int:
        return self.width

    def setup_core(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        self.rt = rt
        self.z_bias, self.x_bias = weights[self.tensors["z_bias"]], weights[self.tensors["x_bias"]]
        self._chunks = None
        if rt.dtype == torch.bfloat16:
            self._chunks = rt.shared("mingru.chunks", ops.mingru_scratch_numel(rt.max_tokens, rt.max_seqs, self.width),
                                     dtype=torch.float32)

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.in_proj = Linear(self.input_weight(weights), rt, tag="mingru.in")
        self.out_proj = Linear(self.output_weight(weights), rt, tag="mingru.out")
        self.setup_core(rt, weights)
        self._gated = rt.shared("mingru.gated", rt.max_tokens, self.width)

    def core(self, proj: torch.Tensor, column: int, ctx: StepContext, cache_id: Optional[int], write_cache: bool,
             out: torch.Tensor, out_scale: float) -> None:
        c = self.width
        ops.mingru_scan(proj, column, column + c, column + 2 * c, self.z_bias, self.x_bias, ctx.state(cache_id),
                        ctx.q_start, ctx.slot_ids, ctx.num_seqs, out, out_scale, self.rt.status, max_q_len=ctx.max_q_len,
                        scratch=self._chunks)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        gated = self._gated[: x.shape[0]]
        self.core(self.in_proj(x), 0, ctx, cache_id, write_cache, gated, 1.0)
        return self.out_proj(gated)


@register_part("mixer", "mlstm")
class MLSTM(Mixer, _NamedTensors):
    """The mLSTM cell.  With h the input, H heads, keys of ``dim`` and values of ``vdim`` values:

        q = W_q h * dim^-1/2;  k = W_k h;  v = W_v h
        i = cap tanh((W_i h + b_i) / cap);   f = logsigmoid(cap tanh((W_f h + b_f) / cap))        (log gates, per head)
        m' = max(f + m, i);   S' = exp(f + m - m') S + exp(i - m') k v^T;   n' = exp(f + m - m') n + exp(i - m') k
        o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
        out = W_o (unit_rms_per_head(o) * norm * sigmoid(W_g h))

    S, n and m start at zero for a new request and are float32 (``memory``, kept as S^T, ``normaliser``, ``maximum`` in
    the cache needs); gates, decays and the division are float32 in every run.  ``names``: the tensors' names after the part's
    own."""

    graph_capturable = True
    splittable = True
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b", "norm": "norm",
             "out": "o"}

    def __init__(self, name: str, hidden_size: int, num_heads: int, dim: int, vdim: int, gate_cap: float, norm_eps: float,
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.num_heads, self.dim, self.vdim = int(hidden_size), int(num_heads), int(dim), int(vdim)
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        if self.gate_cap <= 0:
            raise ValueError(f"mixer {name}: the gates' cap must be positive, got {self.gate_cap}")
        self._name_tensors(name, self.NAMES, names)

    def weight_specs(self) -> List[WeightSpec]:
        t, w, H, D, Dv = self.tensors, self.hidden_size, self.num_heads, self.dim, self.vdim
        return [WeightSpec(t["q"], (H * D, w)), WeightSpec(t["k"], (H * D, w)), WeightSpec(t["v"], (H * Dv, w)),
                WeightSpec(t["gate"], (H * Dv, w)), WeightSpec(t["i"], (H, w)), WeightSpec(t["f"], (H, w)),
                WeightSpec(t["i_bias"], (H,), kind="vector", init="normal"),
                WeightSpec(t["f_bias"], (H,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["norm"], (H * Dv,), kind="vector", init="one_plus_normal"),
                WeightSpec(t["out"], (w, H * Dv))]

    def cache_spec(self):
        H, D, Dv = self.num_heads, self.dim, self.vdim
        # the memory column by column ([vdim, dim]): the lanes that share a column read consecutive floats
        return {"memory": StateSpec((H, Dv, D), "float32"), "normaliser": StateSpec((H, D), "float32"),
                "maximum": StateSpec((H,), "float32")}

    def input_weight(self, weights: Dict[str, torch.Tensor]) -> torch.Tensor:
        t = self.tensors
        parts = [weights.pop(t[k]) for k in ("q", "k", "v", "gate", "i", "f")]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        rows = sum(p.shape[0] for p in parts)
        pad = torch.zeros((-rows) % 8, parts[0].shape[1], dtype=dtype, device=parts[0].device)  # whole groups of eight rows
        return torch.cat([p.to(dtype) for p in parts] + [pad], dim=0)  # columns of the product: q, k, v, g, i, f

    def output_weight(self, weights: Dict[str, torch.Tensor]) -> torch.Tensor:
        return weights.pop(self.tensors["out"])

    @property
    def output_columns(self) -> int:
        return self.num_heads * self.vdim

    def setup_core(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        self.rt = rt
        if self.dim > ops.mlstm_max_dim():
            raise ValueError(f"mixer {self.name}: keys of {self.dim} values exceed the {ops.mlstm_max_dim()} the scan takes")
        t = self.tensors
        self.i_bias, self.f_bias, self.norm_weight = weights[t["i_bias"]], weights[t["f_bias"]], weights[t["norm"]]
        self._h = rt.shared("mlstm.h", rt.max_tokens, self.output_columns, dtype=torch.float32)
        self._segments = None
        if ops.mlstm_segmented_pays(rt.dtype, rt.max_tokens):
            self._segments = ops.MlstmScratch(rt.shared, rt.max_tokens, rt.max_seqs, self.num_heads, self.dim, self.vdim)

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.in_proj = Linear(self.input_weight(weights), rt, tag="mlstm.in")
        self.out_proj = Linear(self.output_weight(weights), rt, tag="mlstm.out")
        self.setup_core(rt, weights)
        self._gated = rt.shared("mlstm.gated", rt.max_tokens, self.output_columns)

    def core(self, proj: torch.Tensor, column: int, ctx: StepContext, cache_id: Optional[int], write_cache: bool,
             out: torch.Tensor, out_scale: float) -> None:
        H, D, Dv = self.num_heads, self.dim, self.vdim
        q_col, k_col, v_col = column, column + H * D, column + 2 * H * D
        g_col = v_col + H * Dv
        i_col = g_col + H * Dv
        h = self._h[: proj.shape[0]]
        ops.mlstm_scan(proj, q_col, k_col, v_col, i_col, i_col + H, self.i_bias, self.f_bias, self.gate_cap,
                       ctx.state(cache_id, "memory"), ctx.state(cache_id, "normaliser"), ctx.state(cache_id, "maximum"),
                       ctx.q_start, ctx.slot_ids, ctx.num_seqs, h, self.rt.status, max_q_len=ctx.max_q_len,
                       scratch=self._segments)
        ops.mlstm_out(h, proj, g_col, self.norm_weight, self.norm_eps, out, out_scale, H)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        gated = self._gated[: x.shape[0]]
        self.core(self.in_proj(x), 0, ctx, cache_id, write_cache, gated, 1.0)
        return self.out_proj(gated)
