"""Several mixers side by side on the same input: y = sum_i scale_i mixer_i(h).

Every branch is a mixer of the kind that is one product of its input, a core and one product to its output
(``Mixer.splittable``).  The branches' input matrices are stacked into one, so that h is read by one product, and
their output matrices are laid side by side, so that one product over the cores' results (each times its scale)
gives the sum.  What a branch keeps per request is filed under the branch's label: a branch asks the context as if it
were alone, and the context it is handed puts the label in front.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..registry import create_part, register_part
from .base import Mixer, PartSpec, Runtime, StepContext, WeightSpec
from .linear import Linear


class ScopedContext:
    """A step context as one branch of a composite part sees it: everything as in the context itself, the names of
    pages and states under the branch's label."""

    def __init__(self, ctx: StepContext, label: str):
        self._ctx, self._label = ctx, label

    def __getattr__(self, name):
        return getattr(self._ctx, name)

    def _scoped(self, name: str) -> str:
        return f"{self._label}.{name}" if name else self._label

    def pages(self, cache_id: int, name: str = ""):
        return self._ctx.pages(cache_id, self._scoped(name))

    def kv(self, cache_id: int, name: str = ""):
        return self._ctx.kv(cache_id, self._scoped(name))

    def state(self, cache_id: int, name: str = ""):
        return self._ctx.state(cache_id, self._scoped(name))


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """``branches``: a list of ``{"label": str, "mixer": PartSpec, "scale": float}``; a branch's tensors are named
    ``<name>.<label>.*``."""

    def __init__(self, name: str, hidden_size: int, branches: Sequence[dict]):
        super().__init__(name)
        self.hidden_size = int(hidden_size)
        if not branches:
            raise ValueError(f"mixer {name}: needs at least one branch")
        self.labels = [str(b["label"]) for b in branches]
        if len(set(self.labels)) != len(self.labels) or any("." in label or not label for label in self.labels):
            raise ValueError(f"mixer {name}: branch labels must be distinct, non-empty and without dots: {self.labels}")
        self.scales = [float(b.get("scale", 1.0)) for b in branches]
        self.branches: List[Mixer] = [create_part("mixer", b["mixer"], name=f"{name}.{b['label']}") for b in branches]
        for label, branch in zip(self.labels, self.branches):
            if not branch.splittable:
                raise ValueError(f"mixer {name}: branch '{label}' ({type(branch).__name__}) cannot run on merged products")

    @property
    def graph_capturable(self) -> bool:
        return all(b.graph_capturable for b in self.branches)

    def weight_specs(self) -> List[WeightSpec]:
        return [s for b in self.branches for s in b.weight_specs()]

    def cache_spec(self):
        needs = {}
        for label, branch in zip(self.labels, self.branches):
            need = branch.cache_spec()
            if need is None:
                continue
            for sub, spec in (need.items() if isinstance(need, dict) else [("", need)]):
                if spec is not None:
                    needs[f"{label}.{sub}" if sub else label] = spec
        return needs or None

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        super().setup(rt, weights)
        ins = [b.input_weight(weights) for b in self.branches]
        outs = [b.output_weight(weights) for b in self.branches]
        dtype = torch.float32 if any(m.dtype == torch.float32 for m in ins + outs) else ins[0].dtype
        self.in_columns, self.out_columns = [0], [0]
        for m in ins:
            self.in_columns.append(self.in_columns[-1] + m.shape[0])
        for m in outs:
            self.out_columns.append(self.out_columns[-1] + m.shape[1])
        self.in_proj = Linear(torch.cat([m.to(dtype) for m in ins], dim=0), rt, tag="parallel.in")
        self.out_proj = Linear(torch.cat([m.to(dtype) for m in outs], dim=1), rt, tag="parallel.out")
        del ins, outs
        for b in self.branches:
            b.setup_core(rt, weights)
        self._mid = rt.shared("parallel.mid", rt.max_tokens, self.out_columns[-1])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache_id: Optional[int], write_cache: bool) -> torch.Tensor:
        proj = self.in_proj(x)
        mid = self._mid[: x.shape[0]]
        for i, (label, branch) in enumerate(zip(self.labels, self.branches)):
            branch.core(proj, self.in_columns[i], ScopedContext(ctx, label), cache_id, write_cache,
                        mid[:, self.out_columns[i]:self.out_columns[i + 1]], self.scales[i])
        return self.out_proj(mid)
