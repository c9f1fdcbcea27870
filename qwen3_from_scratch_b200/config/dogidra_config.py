"""Configuration of the Dogidra architecture: a pre-norm decoder with layer norms, a short causal convolution in
front of every sub-layer, a mixer that runs windowed attention over pooled blocks beside a gated recurrence, a
feed-forward of routed experts, and a span of layers that may run several times.

config.json names the model with ``"architecture": "Dogidra"`` and carries::

    vocab, width                 sizes of the embedding and of the residual stream
    embedding: {scale}           what the looked-up rows are multiplied by
    norm: {eps}                  epsilon of every norm
    canon: {taps}                taps of the convolution in front of each sub-layer
    loop: {start, stop, times}   layers start .. stop - 1 run ``times`` times in a row on the same tensors, each pass
                                 with a cache and state of its own, each pass entered through the ``loop.in``
                                 projection (optional: without it every layer runs once and nothing is projected)
    layers: [ {type: "parallel", mixer: {left, right, left_scale, right_scale}, mlp: {...} | null} ]

``mixer.left``: heads, kv_heads, dim, vdim, scale, softcap (optional), mask: {size, pool}, rot: {base, dims,
scaling: {factor, original, fast, slow} | absent}.  ``mixer.right``: width.  ``mlp``: kind "moe", expert: {ff},
router: {experts, top, scale}, shared: {ff} | absent.  Every number comes from the file; nothing is assumed about
the order or the count of the layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .bikadra_config import RotaryScaling
from .binupel_config import _int, _number
from .model_config import ConfigError, ModelConfig

ARCHITECTURE = "Dogidra"


def _object(where: str, data: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    value = data.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}: '{key}' must be an object")
    return value


@dataclass(frozen=True)
class PooledWindowAttention:
    """The left mixer: grouped-query attention over the last ``window`` tokens and one pooled key and value per
    block of ``pool`` tokens that lies wholly before them."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: int
    pool: int
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class RoutedExperts:
    experts: int
    top: int
    router_scale: float
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class DogidraLayer:
    type: str
    left: PooledWindowAttention
    left_scale: float
    right_width: int
    right_scale: float
    mlp: Optional[RoutedExperts]


def _left(where: str, m: Mapping[str, Any]) -> PooledWindowAttention:
    heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim, vdim = _int(where, m, "dim"), _int(where, m, "vdim")
    cap = m.get("softcap")
    if cap is not None:
        cap = _number(where, m, "softcap")
        if cap <= 0:
            raise ConfigError(f"config.json: {where}: softcap must be positive, got {cap!r}")
    mask = _object(where, m, "mask")
    window, pool = _int(f"{where}.mask", mask, "size"), _int(f"{where}.mask", mask, "pool")
    rot = _object(where, m, "rot")
    base = _number(f"{where}.rot", rot, "base")
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim or base <= 1:
        raise ConfigError(f"config.json: {where}.rot: base {base!r} must exceed 1 and dims {dims!r} be even and at "
                          f"most dim {dim}")
    scaling = None
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, Mapping):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object")
        scaling = RotaryScaling(*(_number(f"{where}.rot.scaling", sc, k) for k in ("factor", "original", "fast", "slow")))
        if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
            raise ConfigError(f"config.json: {where}.rot.scaling: every value must be positive")
    return PooledWindowAttention(heads, kv_heads, dim, vdim, _number(where, m, "scale"), cap, window, pool, base, dims,
                                 scaling)


def _mlp(where: str, mlp: Any) -> Optional[RoutedExperts]:
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}: mlp must be null or of kind 'moe', got {mlp!r}")
    router = _object(where, mlp, "router")
    experts, top = _int(f"{where}.router", router, "experts"), _int(f"{where}.router", router, "top")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: top {top} exceeds the {experts} experts")
    shared = mlp.get("shared")
    if shared is not None and not isinstance(shared, Mapping):
        raise ConfigError(f"config.json: {where}: 'shared' must be an object with 'ff', or absent")
    return RoutedExperts(experts, top, _number(f"{where}.router", router, "scale"),
                         _int(f"{where}.expert", _object(where, mlp, "expert"), "ff"),
                         None if shared is None else _int(f"{where}.shared", shared, "ff"))


@dataclass(frozen=True)
class DogidraConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    taps: int = 1
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    layers: Tuple[DogidraLayer, ...] = field(default_factory=tuple)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "DogidraConfig":
        vocab, width = _int("model", data, "vocab"), _int("model", data, "width")
        eps = _number("norm", _object("model", data, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        scale = _number("embedding", _object("model", data, "embedding"), "scale")
        taps = _int("canon", _object("model", data, "canon"), "taps")
        entries = data.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            if entry.get("type") != "parallel":
                raise ConfigError(f"config.json: {where}: mixer type {entry.get('type')!r} is not built (built: parallel)")
            m = entry["mixer"]
            right = _object(f"{where}.mixer", m, "right")
            layers.append(DogidraLayer("parallel", _left(f"{where}.mixer.left", _object(f"{where}.mixer", m, "left")),
                                       _number(f"{where}.mixer", m, "left_scale"),
                                       _int(f"{where}.mixer.right", right, "width"),
                                       _number(f"{where}.mixer", m, "right_scale"),
                                       _mlp(f"{where}.mlp", entry.get("mlp"))))
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            for key in ("start", "stop", "times"):
                v = loop.get(key)
                if isinstance(v, bool) or not isinstance(v, int) or v < 0:
                    raise ConfigError(f"config.json: loop.{key} must be a non-negative integer, got {v!r}")
            loop = (loop["start"], loop["stop"], loop["times"])
            if not 0 <= loop[0] < loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(layers)} layers")
        eos = data.get("eos_token_id")
        return cls(architecture=ARCHITECTURE, vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps, taps=taps,
                   loop=loop, layers=tuple(layers), eos_token_id=eos if isinstance(eos, int) else None)

    def run_order(self):
        """The layer index of every layer run: the looped span as often as it says, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_dict(self) -> dict:
        entries = []
        for layer in self.layers:
            a = layer.left
            rot = {"base": a.rot_base, "dims": a.rot_dims}
            if a.rot_scaling is not None:
                s = a.rot_scaling
                rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                    "mask": {"size": a.window, "pool": a.pool}, "rot": rot}
            if a.softcap is not None:
                left["softcap"] = a.softcap
            mlp = None
            if layer.mlp is not None:
                e = layer.mlp
                mlp = {"kind": "moe", "expert": {"ff": e.expert_ff},
                       "router": {"experts": e.experts, "top": e.top, "scale": e.router_scale}}
                if e.shared_ff is not None:
                    mlp["shared"] = {"ff": e.shared_ff}
            entries.append({"type": layer.type,
                            "mixer": {"left": left, "left_scale": layer.left_scale, "right": {"width": layer.right_width},
                                      "right_scale": layer.right_scale},
                            "mlp": mlp})
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}, "canon": {"taps": self.taps},
             "layers": entries}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
