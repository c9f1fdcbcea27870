"""Gated feed-forward: y = (up(x) * act(gate(x))) W_down^T, no biases.  ``swiglu`` is the form with the SiLU
gate and the checkpoint's ``gate_proj`` / ``up_proj`` / ``down_proj`` names; ``gated_mlp`` takes the gate's
activation (``silu``, ``relu``, ``gelu_tanh``) and the tensors' names as parameters.

Reference: models/feedback.py:14-34.  The gate and up weights are merged into one [2I, H] weight at load, so
one product feeds the gate kernel.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import create_part, register_part
from .base import FeedForward, PartSpec, Runtime, StreamNorm, WeightSpec
from .linear import Linear

_DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_capturable = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: Optional[Dict[str, str]] = None):
        """``names``: what follows the part's name (and a dot) in the names of its gate, up and down tensors."""
        super().__init__(name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        ops.activation_code(activation, gate=True)
        self.activation = activation
        n = dict(_DEFAULT_NAMES)
        n.update(names or {})
        self.tensors = {k: f"{name}.{v}" for k, v in n.items()}

    def weight_specs(self) -> List[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.tensors["gate"], (i, h)),
                WeightSpec(self.tensors["up"], (i, h)),
                WeightSpec(self.tensors["down"], (h, i))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        gate = weights.pop(self.tensors["gate"])
        up = weights.pop(self.tensors["up"])
        dtype = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        h, i = self.hidden_size, self.intermediate_size
        # bfloat16: gate and up rows alternate in blocks of eight, so that the decode kernel has a
        # gate value and its up value in one thread and applies the activation before storing
        self.blocks_of_eight = dtype == torch.bfloat16 and i % 8 == 0
        if self.blocks_of_eight:
            merged = torch.cat([gate.view(i // 8, 8, h), up.view(i // 8, 8, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            merged = torch.cat([gate.to(dtype), up.to(dtype)], dim=0)
        del gate, up
        self.gate_up = Linear(merged, rt, tag="ffn.gate_up")
        self.down = Linear(weights.pop(self.tensors["down"]), rt, tag="ffn.down")
        self._act = rt.shared("ffn.act", rt.max_tokens, self.intermediate_size)
        # the few-rows product applies any gate in its epilogue, the tcgen05 product those of ops.GEMM_TC_GATES; the
        # product that also applies a norm that was never computed is built for the SiLU gate
        self.fused_gate = self.blocks_of_eight

    fuses_stream = True

    def can_fuse_stream(self, rows: int) -> bool:
        return (self.fused_gate and self.activation == "silu" and self.gate_up.takes_stream_norm(rows)
                and self.down.can_add_into_stream(rows))

    def forward(self, x, into_stream=None, next_norm_weight=None):
        act = self._act[: x.shape[0]]
        rows = x.shape[0]
        if isinstance(x, StreamNorm):
            # decoding without norm kernels: the norm is applied inside the gate/up product
            ops.gemm_skinny_normed(x.scaled, x.sumsq, x.parts, x.eps, self.gate_up.weight, act, swiglu_blocks=True)
        elif self.fused_gate and ops.gemm_skinny_takes(rows, self.gate_up.weight):
            # decoding: stream the weight once, activation applied before the store
            ops.gemm_skinny(x, self.gate_up.weight, act, swiglu_blocks=True, activation=self.activation)
        elif (self.fused_gate and self.activation in ops.GEMM_TC_GATES
              and ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight) and ops.gemm_tc_takes(x, self.gate_up.weight)):
            # prompt portions: the engine's tcgen05 product with the activation in its epilogue, so the
            # [T, 2I] gate/up product never goes to memory
            ops.gemm_tc(x, self.gate_up.weight, act, self.rt.status, swiglu_blocks=True,
                        pair=ops.gemm_tc_swiglu_pays(rows, self.gate_up.weight) == "pair", activation=self.activation)
        else:
            ops.gated_act(self.gate_up(x), act, interleave8=self.blocks_of_eight, activation=self.activation)
        if into_stream is not None:
            return self.down.into_stream(act, into_stream, next_norm_weight)
        return self.down(act)


@register_part("feed_forward", "swiglu")
class SwiGLU(GatedMLP):
    def __init__(self, name: str, hidden_size: int, intermediate_size: int):
        super().__init__(name, hidden_size, intermediate_size, activation="silu")


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """Feed-forward without a gate: y = W_down act(W_up x), no biases.  ``names``: what follows the part's name (and
    a dot) in the names of its up and down tensors."""

    graph_capturable = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "gelu_tanh",
                 names: Optional[Dict[str, str]] = None):
        super().__init__(name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        ops.activation_code(activation, gate=True)
        self.activation = activation
        n = {"up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.tensors = {k: f"{name}.{v}" for k, v in n.items()}

    def weight_specs(self) -> List[WeightSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return [WeightSpec(self.tensors["up"], (i, h)), WeightSpec(self.tensors["down"], (h, i))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.up = Linear(weights.pop(self.tensors["up"]), rt, tag="ffn.up")
        self.down = Linear(weights.pop(self.tensors["down"]), rt, tag="ffn.down")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.shape[0]
        if (ops.gemm_skinny_takes(rows, self.up.weight) and x.dtype == torch.bfloat16
                and self.up.out_dtype == torch.bfloat16):
            # decoding: the weight is streamed once and the activation applied before the store
            h = self.up._buffer("_out", rows, self.up.out_dtype)
            ops.gemm_skinny(x, self.up.weight, h, plain_activation=self.activation)
            return self.down(h)
        h = self.up(x)
        ops.act(h, h, self.activation)
        return self.down(h)


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of experts: ``experts`` small feed-forwards W_down act(W_up h) without biases, of which every token
    uses ``top``.

        s = sigmoid(W_router h)                  float32 (h may be its rounding to the compute dtype)
        chosen: the ``top`` experts with the largest s + correction (ties: the lower index)
        y = sum_chosen s_e * router_scale * expert_e(h)  [+ shared(h)]

    ``gated=True``: the experts are gated, W_down (act(W_gate h) * (W_up h)), with a further tensor
    ``<name>.<expert><e>.<gate>`` [ff, width].  ``weigh="input"``: the router's weight multiplies what the expert reads
    instead of what it returns, y = sum_chosen expert_e(s_e * router_scale * h).

    The correction takes part in the choice only; the weights are not renormalised.  ``shared``: a feed-forward
    (any registered one) that every token goes through, added to the sum, or None.  Tensors: ``<name>.<router>``
    [E, width], ``<name>.<correction>`` [E] (absent with ``correction=False``), ``<name>.<expert><e>.<up>`` [ff, width]
    and ``.<down>`` [width, ff], and the shared part's under ``<name>.<shared>``."""

    graph_capturable = True
    NAMES = {"router": "router", "correction": "correction", "expert": "e", "up": "up", "down": "down", "gate": "gate",
             "shared": "shared"}

    def __init__(self, name: str, hidden_size: int, experts: int, top: int, expert_ff: int, router_scale: float = 1.0,
                 activation: str = "relu_sq", correction: bool = True, shared: Optional[PartSpec] = None,
                 names: Optional[Dict[str, str]] = None, gated: bool = False, weigh: str = "output"):
        super().__init__(name)
        if weigh not in ("output", "input"):
            raise ValueError(f"feed-forward {name}: the router's weight goes to an expert's 'input' or 'output', got {weigh!r}")
        self.gated, self.weigh_input = bool(gated), weigh == "input"
        self.hidden_size, self.experts, self.top, self.expert_ff = int(hidden_size), int(experts), int(top), int(expert_ff)
        if not 1 <= self.top <= min(self.experts, ops.MOE_MAX_TOP):
            raise ValueError(f"feed-forward {name}: top {self.top} of {self.experts} experts (at most {ops.MOE_MAX_TOP})")
        self.router_scale = float(router_scale)
        ops.activation_code(activation, gate=True)
        self.activation = activation
        self.has_correction = bool(correction)
        n = dict(self.NAMES)
        n.update(names or {})
        self.n = n
        self.shared = None if shared is None else create_part("feed_forward", shared, name=f"{name}.{n['shared']}")

    def _expert(self, e: int, which: str) -> str:
        return f"{self.name}.{self.n['expert']}{e}.{self.n[which]}"

    def weight_specs(self) -> List[WeightSpec]:
        w, f = self.hidden_size, self.expert_ff
        specs = [WeightSpec(f"{self.name}.{self.n['router']}", (self.experts, w), kind="vector", init="normal")]
        if self.has_correction:
            specs.append(WeightSpec(f"{self.name}.{self.n['correction']}", (self.experts,), kind="vector", init="normal"))
        for e in range(self.experts):
            if self.gated:
                specs.append(WeightSpec(self._expert(e, "gate"), (f, w)))
            specs += [WeightSpec(self._expert(e, "up"), (f, w)), WeightSpec(self._expert(e, "down"), (w, f))]
        return specs + (self.shared.weight_specs() if self.shared is not None else [])

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.router = weights[f"{self.name}.{self.n['router']}"]
        self.correction = weights[f"{self.name}.{self.n['correction']}"] if self.has_correction else None
        # the experts' matrices in two stacks, in the compute dtype: up [E, ff, width], down [E, width, ff]
        self.gate_block = ops.moe_gate_block(self.expert_ff) if self.gated else 0
        if self.gated:
            # gate and up rows of an expert alternate in blocks of gate_block rows: [E, 2 ff, width]
            gb, f, w = self.gate_block, self.expert_ff, self.hidden_size
            self.up = torch.stack([
                torch.cat([weights.pop(self._expert(e, "gate")).to(rt.dtype).view(f // gb, gb, w),
                           weights.pop(self._expert(e, "up")).to(rt.dtype).view(f // gb, gb, w)], dim=1).reshape(2 * f, w)
                for e in range(self.experts)]).contiguous()
        else:
            self.up = torch.stack([weights.pop(self._expert(e, "up")).to(rt.dtype) for e in range(self.experts)]).contiguous()
        self.down = torch.stack([weights.pop(self._expert(e, "down")).to(rt.dtype) for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.setup(rt, weights)
        T = rt.max_tokens
        self._ids = rt.shared("moe.ids", T, self.top, dtype=torch.int32)
        self._weights = rt.shared("moe.weights", T, self.top, dtype=torch.float32)
        self._act = rt.shared("moe.act", T * self.top, self.expert_ff)
        self._out = rt.shared("moe.out", T, self.hidden_size)
        self._status = rt.status
        self._grouped = None
        # a design that weighs the experts' input adds their outputs up as they are
        self._ones = torch.ones(T, self.top, dtype=torch.float32, device=rt.device) if self.weigh_input else None
        if ops.moe_grouped_takes(rt.dtype, self.hidden_size, self.expert_ff, gated=self.gated):
            self._grouped = ops.MoeScratch(rt.shared, T, self.top, self.experts, self.hidden_size, self.expert_ff)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        ids, wts = self._ids[:T], self._weights[:T]
        ops.moe_route(x, self.router, self.correction, ids, wts, self.router_scale)
        base = self.shared.forward(x) if self.shared is not None else None
        out = self._out[:T]
        ops.routed_experts(x, self.up, self.down, ids, self._ones[:T] if self.weigh_input else wts, base,
                           self._act[: T * self.top], out, self.activation, scratch=self._grouped, status=self._status,
                           gate_block=self.gate_block, in_weights=wts if self.weigh_input else None)
        return out
