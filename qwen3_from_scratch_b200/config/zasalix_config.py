"""Configuration of the Zasalix architecture: a decoder whose sub-layers stand between two norms without statistics
(tanh(alpha x) w + b), whose layers are listed one by one (attention through a latent with a sink, an mLSTM matrix
memory, or windowed attention that keeps the first tokens side by side with such a memory), each with a dense or a
routed feed-forward or none, each adding a gated slice of a second embedding of the token, and a span of layers that
may run several times.

config.json names the model with ``"architecture": "Zasalix"`` and carries::

    vocab, width                 sizes of the embedding and of the residual stream
    norm: {eps}                  epsilon of every RMS norm inside the mixers and of the token-side norm
    token_side: {dim}            width of a layer's slice of the second embedding (absent: no such input)
    loop: {start, stop, times}   layers start .. stop - 1 run ``times`` times in a row on the same tensors, each pass
                                 with a cache and state of its own (absent: every layer runs once)
    layers: [ {type, mixer: {...}, mlp: {...} | null} ]

``type`` "latent_attention": heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}.
``type`` "mlstm": heads, dim, vdim, gate_cap.
``type`` "parallel": left: {heads, kv_heads, dim, vdim, scale, mask: {size, keep_first}, rot: {base, dims}},
right: an mlstm's keys, left_scale, right_scale.
``mlp``: {kind: "dense", ff} or {kind: "moe", expert: {ff}, router: {experts, top}, shared: {ff} | absent}.
Every number comes from the file; nothing is assumed about the order or the count of the layers.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple, Union

from .binupel_config import _int, _number
from .model_config import ConfigError, ModelConfig

ARCHITECTURE = "Zasalix"


def _object(where: str, data: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    value = data.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}: '{key}' must be an object")
    return value


def _count(where: str, data: Mapping[str, Any], key: str) -> int:
    """A non-negative integer (``_int`` wants a positive one)."""
    v = data.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}: '{key}' must be a non-negative integer, got {v!r}")
    return v


def _rotation(where: str, m: Mapping[str, Any], most: int) -> Tuple[float, int]:
    rot = _object(where, m, "rot")
    base, dims = _number(f"{where}.rot", rot, "base"), _count(f"{where}.rot", rot, "dims")
    if dims % 2 or dims > most or base <= 1:
        raise ConfigError(f"config.json: {where}.rot: base {base!r} must exceed 1 and dims {dims!r} be even and at most {most}")
    return base, dims


@dataclass(frozen=True)
class SinkLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class KeptWindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelMixer:
    left: KeptWindowAttention
    right: MatrixMemory
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class ZasalixLayer:
    type: str
    mixer: Union[SinkLatentAttention, MatrixMemory, ParallelMixer]
    mlp: Union[DenseFF, RoutedFF, None]


def _latent(where: str, m: Mapping[str, Any]) -> SinkLatentAttention:
    rot_dim = _count(where, m, "rot_dim")
    base, dims = _rotation(where, m, rot_dim)
    return SinkLatentAttention(_int(where, m, "heads"), _int(where, m, "dim"), rot_dim, _int(where, m, "vdim"),
                               _int(where, m, "kv_rank"), _int(where, m, "q_rank"), _number(where, m, "scale"), base, dims)


def _memory(where: str, m: Mapping[str, Any]) -> MatrixMemory:
    cap = _number(where, m, "gate_cap")
    if cap <= 0:
        raise ConfigError(f"config.json: {where}: gate_cap must be positive, got {cap!r}")
    return MatrixMemory(_int(where, m, "heads"), _int(where, m, "dim"), _int(where, m, "vdim"), cap)


def _window(where: str, m: Mapping[str, Any]) -> KeptWindowAttention:
    heads, kv_heads = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = _int(where, m, "dim")
    base, dims = _rotation(where, m, dim)
    mask = _object(where, m, "mask")
    return KeptWindowAttention(heads, kv_heads, dim, _int(where, m, "vdim"), _number(where, m, "scale"),
                               _int(f"{where}.mask", mask, "size"), _count(f"{where}.mask", mask, "keep_first"), base, dims)


def _mlp(where: str, mlp: Any) -> Union[DenseFF, RoutedFF, None]:
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}: mlp must be null or of kind 'dense' or 'moe', got {mlp!r}")
    if mlp["kind"] == "dense":
        return DenseFF(_int(where, mlp, "ff"))
    router = _object(where, mlp, "router")
    experts, top = _int(f"{where}.router", router, "experts"), _int(f"{where}.router", router, "top")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: top {top} exceeds the {experts} experts")
    shared = mlp.get("shared")
    if shared is not None and not isinstance(shared, Mapping):
        raise ConfigError(f"config.json: {where}: 'shared' must be an object with 'ff', or absent")
    return RoutedFF(experts, top, _int(f"{where}.expert", _object(where, mlp, "expert"), "ff"),
                    None if shared is None else _int(f"{where}.shared", shared, "ff"))


MIXERS = ("latent_attention", "mlstm", "parallel")


@dataclass(frozen=True)
class ZasalixConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    side_dim: Optional[int] = None
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    layers: Tuple[ZasalixLayer, ...] = field(default_factory=tuple)
    eos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZasalixConfig":
        vocab, width = _int("model", data, "vocab"), _int("model", data, "width")
        eps = _number("norm", _object("model", data, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        side = data.get("token_side")
        side_dim = None if side is None else _int("token_side", _object("model", data, "token_side"), "dim")
        entries = data.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with 'type' and 'mixer'")
            kind, m = entry.get("type"), entry["mixer"]
            if kind == "latent_attention":
                mixer = _latent(f"{where}.mixer", m)
            elif kind == "mlstm":
                mixer = _memory(f"{where}.mixer", m)
            elif kind == "parallel":
                mixer = ParallelMixer(_window(f"{where}.mixer.left", _object(f"{where}.mixer", m, "left")),
                                      _memory(f"{where}.mixer.right", _object(f"{where}.mixer", m, "right")),
                                      _number(f"{where}.mixer", m, "left_scale"), _number(f"{where}.mixer", m, "right_scale"))
            else:
                raise ConfigError(f"config.json: {where}: mixer type {kind!r} is not built (built: {', '.join(MIXERS)})")
            layers.append(ZasalixLayer(kind, mixer, _mlp(f"{where}.mlp", entry.get("mlp"))))
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            loop = tuple(_count("loop", loop, key) for key in ("start", "stop", "times"))
            if not 0 <= loop[0] < loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(layers)} layers")
        eos = data.get("eos_token_id")
        return cls(architecture=ARCHITECTURE, vocab=vocab, width=width, norm_eps=eps, side_dim=side_dim, loop=loop,
                   layers=tuple(layers), eos_token_id=eos if isinstance(eos, int) else None)

    def run_order(self):
        """(layer index, pass of the loop or 0, first layer of a pass?) of every layer run: the looped span as often
        as it says, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, 0, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, 0, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t, i == start) for i in range(start, stop)]
        return runs + [(i, 0, False) for i in range(stop, n)]

    def to_dict(self) -> dict:
        def rot(a):
            return {"base": a.rot_base, "dims": a.rot_dims}

        def memory(a):
            return {"heads": a.heads, "dim": a.dim, "vdim": a.vdim, "gate_cap": a.gate_cap}

        entries = []
        for layer in self.layers:
            a = layer.mixer
            if layer.type == "latent_attention":
                mixer = {"heads": a.heads, "dim": a.dim, "rot_dim": a.rot_dim, "vdim": a.vdim, "kv_rank": a.kv_rank,
                         "q_rank": a.q_rank, "scale": a.scale, "rot": rot(a)}
            elif layer.type == "mlstm":
                mixer = memory(a)
            else:
                left = a.left
                mixer = {"left": {"heads": left.heads, "kv_heads": left.kv_heads, "dim": left.dim, "vdim": left.vdim,
                                  "scale": left.scale, "mask": {"size": left.window, "keep_first": left.keep_first},
                                  "rot": rot(left)},
                         "left_scale": a.left_scale, "right": memory(a.right), "right_scale": a.right_scale}
            e, mlp = layer.mlp, None
            if isinstance(e, DenseFF):
                mlp = {"kind": "dense", "ff": e.ff}
            elif isinstance(e, RoutedFF):
                mlp = {"kind": "moe", "expert": {"ff": e.expert_ff}, "router": {"experts": e.experts, "top": e.top}}
                if e.shared_ff is not None:
                    mlp["shared"] = {"ff": e.shared_ff}
            entries.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": entries}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
