"""Token embedding and the output head.

Reference: models/qwen3.py:17-19,45 (lookup, no scaling), models/qwen3.py:63-74,83-84
(head = Linear without bias, tied to the embedding table when the configuration says so).
The embedding writes the float32 residual stream; the head returns float32 logits.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..registry import register_part
from .base import Part, Runtime, WeightSpec
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_capturable = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, suffix: str = ".weight", scale: float = 1.0,
                 copies: Optional[int] = None, side_table: Optional[str] = None, side_width: int = 0):
        """``suffix``: what follows the part's name in its tensor's name ("" for a tensor named like the part).
        ``scale`` multiplies the looked-up rows.  With ``copies`` (a number, 1 included) the model's blocks keep that
        many residual streams per token: the result is [T, copies, hidden], every stream starting as the same row;
        None: the single stream [T, hidden] of the other blocks.  ``side_table``: the full name of a second table
        [vocab, side_width] of the token, whose rows ``side_rows`` looks up once per step for the layers that read
        their slice of it."""
        super().__init__(name)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tensor = f"{name}{suffix}"
        self.scale, self.copies = float(scale), None if copies is None else int(copies)
        self.side_table, self.side_width = side_table, int(side_width)
        self.has_side_table = bool(side_table)
        if self.has_side_table and self.side_width <= 0:
            raise ValueError(f"embedding {name}: the second table needs its width")
        if self.copies is not None and not 1 <= self.copies <= ops.HC_MAX_STREAMS:
            raise ValueError(f"embedding {name}: between 1 and {ops.HC_MAX_STREAMS} residual streams, got {self.copies}")

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size))]
        if self.has_side_table:
            specs.append(WeightSpec(self.side_table, (self.vocab_size, self.side_width)))
        return specs

    def side_rows(self, token_ids: torch.Tensor) -> torch.Tensor:
        """float32 [T, side_width]: the tokens' rows of the second table."""
        rows = self._side[: token_ids.numel()]
        ops.embed(self.side_weight, token_ids, rows, self.rt.status)
        return rows

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        self.weight = weights[self.tensor]
        if self.has_side_table:
            self.side_weight = weights[self.side_table]
            self._side = rt.shared("embedding.side", rt.max_tokens, self.side_width, dtype=torch.float32)
        self.plain = self.copies is None and self.scale == 1.0
        shape = (rt.max_tokens, self.hidden_size) if self.copies is None else (rt.max_tokens, self.copies, self.hidden_size)
        self._stream = rt.shared("stream", *shape, dtype=torch.float32)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        stream = self._stream[: token_ids.numel()]
        if self.plain:
            ops.embed(self.weight, token_ids, stream, self.rt.status)
        elif self.copies is None:
            ops.embed_scaled(self.weight, token_ids, stream.unsqueeze(1), self.scale, self.rt.status)
        else:
            ops.embed_scaled(self.weight, token_ids, stream, self.scale, self.rt.status)
        return stream


@register_part("head", "lm_head")
class LMHead(Part):
    graph_capturable = True

    """logits = x W^T in float32.  ``tied_to``: name of the embedding tensor it shares, or None.
    ``softcap``: logits <- softcap * tanh(logits / softcap), or None for the logits as they are."""

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None,
                 suffix: str = ".weight", softcap: Optional[float] = None):
        super().__init__(name)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tied_to = tied_to
        self.softcap = None if softcap is None else float(softcap)
        self.tensor = f"{name}{suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        if self.tied_to:
            return []
        return [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size))]

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        weight = weights[self.tied_to] if self.tied_to else weights[self.tensor]
        self.proj = Linear(weight, rt, out_dtype=torch.float32, reuse_output=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.proj(x)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits
