"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, and layer norm with weight and bias; statistics in float32.  And Dynamic
Tanh, which stands where a norm stands but computes no statistics: y = tanh(alpha x) w + b.

Reference: models/norm.py:11-22 (weight multiplies directly, eps from the configuration),
csrc/rms_norm/rms_norm.cpp:13-31.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import Norm, PendingNormed, Runtime, StreamNorm, StreamStats, WeightSpec


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    graph_capturable = True

    def __init__(self, name: str, dim: int, eps: float, suffix: str = ".weight"):
        """``suffix``: what follows the part's name in its tensor's name ("" where the tensor bears the
        part's name itself)."""
        super().__init__(name)
        self.dim, self.eps = int(dim), float(eps)
        self.tensor = f"{name}{suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor, (self.dim,), kind="vector", init="one_plus_normal")]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight = weights[self.tensor]
        self._out = rt.shared("normed", rt.max_tokens, self.dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        ops.rmsnorm(x, self.weight, out, self.eps)
        return out

    def add_norm(self, stream: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = self._out[: stream.shape[0]]
        ops.add_rmsnorm(stream, delta, self.weight, out, self.eps)
        return out

    def scale_add_norm(self, stream: torch.Tensor, delta: Optional[torch.Tensor], alpha: float,
                       want_copy: bool = True) -> Optional[torch.Tensor]:
        """The norm after the sum: stream = norm(alpha * stream + delta) in place; returns the new rows in the
        compute dtype for the next projection (``want_copy``; in a float32 run the stream itself)."""
        if self.rt.dtype == torch.float32 or not want_copy:
            ops.scale_add_rmsnorm(stream, delta, self.weight, None, alpha, self.eps)
            return stream if want_copy else None
        out = self._out[: stream.shape[0]]
        ops.scale_add_rmsnorm(stream, delta, self.weight, out, alpha, self.eps)
        return out

    def lazy(self, stream: torch.Tensor, stats: StreamStats) -> Optional[StreamNorm]:
        """This norm of the stream for a projection that applies it itself, if the projection that last
        added into the stream prepared the stream for this norm's weight; else None."""
        if stats is None or stats.scaled is None or stats.scaled_for is not self.weight:
            return None
        return StreamNorm(stream, self.weight, self.eps, stats.sumsq, stats.parts, stats.scaled)

    def norm_rows(self, stream: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.numel(), self.dim, dtype=self.rt.dtype, device=stream.device)
        ops.add_rmsnorm_rows(stream, delta, self.weight, rows, out, self.eps)
        return out


@register_part("norm", "stream_sum_rms_norm")
class StreamSumRMSNorm(Norm):
    """The last norm of a model with several residual streams per token: y = rmsnorm(sum of the streams) * w, for
    chosen rows of ``streams`` [T, S, W].  What the last sub-layer left open (``PendingStreamWrite``: its output and
    the coefficients that bring it into the streams) is applied to those rows on the way; the streams are not changed."""

    graph_capturable = True

    def __init__(self, name: str, dim: int, eps: float, streams: int, suffix: str = ".weight"):
        super().__init__(name)
        self.dim, self.eps, self.streams = int(dim), float(eps), int(streams)
        self.tensor = f"{name}{suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor, (self.dim,), kind="vector", init="one_plus_normal")]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight = weights[self.tensor]

    def norm_rows(self, stream: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.numel(), self.dim, dtype=self.rt.dtype, device=stream.device)
        pending = None if delta is None else (delta.delta, delta.mix, delta.write)
        ops.hc_sum_norm_rows(stream, pending, self.weight, rows, out, self.eps, self.rt.status)
        return out


@register_part("norm", "layer_norm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b over the last axis, var the mean of the squared deviations; statistics
    in float32.  The weight is the tensor ``<name><suffix>``, the bias ``<name><bias_suffix>``.  ``add_norm`` returns
    the compute dtype; ``add_norm_float32`` the same rows in float32, for a block that works on the normed rows
    before it hands them to a projection."""

    graph_capturable = True

    def __init__(self, name: str, dim: int, eps: float, suffix: str = ".weight", bias_suffix: str = ".bias"):
        super().__init__(name)
        self.dim, self.eps = int(dim), float(eps)
        self.tensor, self.bias_tensor = f"{name}{suffix}", f"{name}{bias_suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor, (self.dim,), kind="vector", init="one_plus_normal"),
                WeightSpec(self.bias_tensor, (self.dim,), kind="vector", init="normal")]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight, self.bias = weights[self.tensor], weights[self.bias_tensor]
        self._out = rt.shared("normed", rt.max_tokens, self.dim)
        self._out32 = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        stream = x.to(torch.float32).contiguous()
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.add_layernorm(stream, None, self.weight, self.bias, out, self.eps)
        return out

    def add_norm(self, stream: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        out = self._out[: stream.shape[0]]
        ops.add_layernorm(stream, delta, self.weight, self.bias, out, self.eps)
        return out

    def add_norm_float32(self, stream: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        if self._out32 is None:
            self._out32 = self.rt.shared("normed.float32", self.rt.max_tokens, self.dim, dtype=torch.float32)
        out = self._out32[: stream.shape[0]]
        ops.add_layernorm(stream, delta, self.weight, self.bias, out, self.eps)
        return out

    def add_norm_conv1(self, stream: torch.Tensor, delta: Optional[torch.Tensor], conv_weight: torch.Tensor,
                       state: Optional[torch.Tensor], ctx, out: torch.Tensor) -> None:
        """For a step of single tokens: the sum, the norm, the short convolution over the normed rows from the
        requests' states and the states' renewal in one launch."""
        ops.add_layernorm_conv1(stream, delta, self.weight, self.bias, conv_weight, state, ctx.tok_seq, ctx.slot_ids, out,
                                self.eps, self.rt.status)

    def norm_rows(self, stream: torch.Tensor, delta: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.numel(), self.dim, dtype=self.rt.dtype, device=stream.device)
        ops.add_layernorm(stream, delta, self.weight, self.bias, out, self.eps, rows=rows)
        return out


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha x) w + b over the last axis, with one learned scalar alpha, a weight and a bias per feature: the
    stand-in for a norm of Zhu et al., "Transformers without Normalization".  Nothing is reduced over the row.  The
    weight is the tensor ``<name><suffix>``, the bias ``<name><bias_suffix>``, alpha ``<name><alpha_suffix>`` (no
    dimensions).  All float32.

    ``delta`` may be a tensor (added as it is) or a ``PendingNormed`` (a sub-layer's output that first goes through the
    Dynamic Tanh that follows the sub-layer): both in the same pass over the stream as this norm.  ``extra_rows``
    (float32 [T, dim]) and ``extra_vec`` (float32 [dim]) are added to the stream on the same pass."""

    graph_capturable = True

    def __init__(self, name: str, dim: int, suffix: str = ".weight", bias_suffix: str = ".bias", alpha_suffix: str = ".alpha"):
        super().__init__(name)
        self.dim = int(dim)
        self.tensor, self.bias_tensor, self.alpha_tensor = f"{name}{suffix}", f"{name}{bias_suffix}", f"{name}{alpha_suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor, (self.dim,), kind="vector", init="one_plus_normal"),
                WeightSpec(self.bias_tensor, (self.dim,), kind="vector", init="normal"),
                WeightSpec(self.alpha_tensor, (), kind="vector", init="one_plus_normal")]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight, self.bias = weights[self.tensor], weights[self.bias_tensor]
        self.alpha = weights[self.alpha_tensor].reshape(1)
        self._out = rt.shared("normed", rt.max_tokens, self.dim)

    @property
    def params(self):
        return (self.alpha, self.weight, self.bias)

    @staticmethod
    def _open(delta):
        """(tensor or None, the Dynamic Tanh it still has to go through or None)."""
        if isinstance(delta, PendingNormed):
            if not isinstance(delta.norm, DynamicTanh):
                raise ValueError(f"the open sub-layer output waits for {type(delta.norm).__name__}, which this norm's kernel "
                                 f"does not apply")
            return delta.delta, delta.norm.params
        return delta, None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        stream = x.to(torch.float32).contiguous()
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.add_dyt(stream.view(-1, self.dim), None, None, self.params, out.view(-1, self.dim))
        return out

    def add_norm(self, stream: torch.Tensor, delta, extra_rows: Optional[torch.Tensor] = None,
                 extra_vec: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = self._out[: stream.shape[0]]
        d, after = self._open(delta)
        ops.add_dyt(stream, d, after, self.params, out, rows_add=extra_rows, vec_add=extra_vec)
        return out

    def close(self, stream: torch.Tensor, delta: torch.Tensor, want_copy: bool = False) -> Optional[torch.Tensor]:
        """stream += this(delta), with no norm after it; ``want_copy``: the new rows in the compute dtype (in a float32
        run the stream itself)."""
        out = None
        if want_copy and self.rt.dtype != torch.float32:
            out = self._out[: stream.shape[0]]
        ops.add_dyt(stream, delta, self.params, None, out)
        return (stream if out is None else out) if want_copy else None

    def norm_rows(self, stream: torch.Tensor, delta, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.numel(), self.dim, dtype=self.rt.dtype, device=stream.device)
        d, after = self._open(delta)
        ops.add_dyt(stream, d, after, self.params, out, rows=rows)
        return out
