"""Small Zasalix configurations and model folders for the tests: the configuration dicts, the tensors the design
names for them (names and shapes restated here from the design, not asked of the engine) and random weights strong
enough that every mechanism moves the logits."""

from __future__ import annotations

import json
import os
from typing import Dict

import torch
from safetensors.torch import save_file


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def parallel(heads, kv_heads, dim, vdim, scale, window, keep_first, base, dims, right, left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "keep_first": keep_first}, "rot": {"base": base, "dims": dims}}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": right["mixer"],
                                          "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def with_mlp(entry, mlp):
    return dict(entry, mlp=mlp)


# X: a loop of three passes over two layers in the middle; every layer with sizes of its own; a window of 9 tokens
# that keeps the first 4, two and three query heads per key head, a partly rotated head; a latent attention whose
# rotated part is only partly rotated; two experts of three chosen; a layer without feed-forward; a routed
# feed-forward without a shared expert.
ZASALIX_X = {
    "architecture": "Zasalix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [with_mlp(latent(4, 24, 8, 40, 48, 56, 0.2, 10000.0, dims=4), moe(5, 2, 24, 40)),
               with_mlp(parallel(4, 2, 24, 40, 0.2, 9, 4, 10000.0, 16, memory(3, 16, 24, 8.0), 0.7, 1.2), dense(96)),
               with_mlp(memory(2, 40, 24, 15.0), None),
               with_mlp(parallel(6, 2, 16, 8, 0.3, 5, 7, 500.0, 16, memory(2, 8, 40, 3.0), 1.1, 0.6), moe(3, 3, 32)),
               with_mlp(latent(2, 32, 16, 16, 24, 40, 0.15, 100.0), dense(72))]}
# Y: no loop and no token-side input at all; one head everywhere; a window of one token that keeps none, every
# expert chosen, no rotation in the windowed attention, a latent attention without a rotated part.
ZASALIX_Y = {
    "architecture": "Zasalix", "vocab": 173, "width": 48, "norm": {"eps": 1e-6},
    "layers": [with_mlp(parallel(1, 1, 32, 24, 0.18, 1, 0, 10000.0, 0, memory(1, 24, 16, 12.0)), moe(3, 3, 40, 56)),
               with_mlp(latent(1, 16, 0, 24, 32, 16, 0.25, 10000.0), dense(64)),
               with_mlp(memory(5, 8, 16, 6.0), moe(9, 1, 8, 16))]}
# Z: sizes in the manner of the serving kernels, small: heads of 64 and 128, a latent of 64 with a rotated part of 32,
# a window of 48 that keeps 16, experts in multiples of 16; the loop is the whole model, starts at the first layer and
# runs twice; more first tokens kept than the window is long in the second layer.
ZASALIX_Z = {
    "architecture": "Zasalix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "token_side": {"dim": 16},
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [with_mlp(parallel(8, 2, 64, 64, 0.11, 48, 16, 1000000.0, 64, memory(4, 64, 64, 10.0), 0.8, 1.1),
                        moe(8, 2, 48, 96)),
               with_mlp(parallel(4, 1, 128, 32, 0.09, 20, 33, 10000.0, 32, memory(2, 128, 32, 12.0)), dense(256)),
               with_mlp(latent(4, 32, 32, 64, 64, 96, 0.12, 50000.0), moe(12, 4, 32, 64))]}
# W: sizes that are multiples of 8 but not of 16 or 32: five heads, keys of 80 and values of 112, a latent of 128 (a
# size the tensor-core kernel takes) with a rotated part of 24, a window of 40 that keeps 12, experts of 80; the loop is
# the first two layers, the model ends with two latent attentions of different sizes.
ZASALIX_W = {
    "architecture": "Zasalix", "vocab": 400, "width": 160, "norm": {"eps": 1e-6}, "token_side": {"dim": 24},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [with_mlp(parallel(5, 5, 80, 112, 0.1, 40, 12, 20000.0, 40, memory(5, 24, 56, 12.0), 1.2, 0.5), moe(6, 2, 80, 48)),
               with_mlp(memory(3, 56, 40, 9.0), dense(200)),
               with_mlp(latent(5, 48, 24, 40, 128, 96, 0.12, 500000.0), moe(4, 1, 48)),
               with_mlp(latent(3, 64, 8, 56, 72, 104, 0.11, 10000.0, dims=8), None)]}
CONFIGS = {"x": (ZASALIX_X, 3), "y": (ZASALIX_Y, 4), "z": (ZASALIX_Z, 5), "w": (ZASALIX_W, 6)}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "head": (V, W)}

    def norm(name):
        shapes.update({name: (W,), name + ".b": (W,), name + ".alpha": ()})

    def mem(p, m):
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        shapes.update({p + "q": (H * D, W), p + "k": (H * D, W), p + "v": (H * Dv, W), p + "g": (H * Dv, W),
                       p + "o": (W, H * Dv), p + "norm": (H * Dv,), p + "i": (H, W), p + "i.b": (H,), p + "f": (H, W),
                       p + "f.b": (H,)})

    norm("final.norm")
    side = config.get("token_side")
    if side:
        shapes["side.embed"] = (V, len(config["layers"]) * side["dim"])
    if config.get("loop"):
        shapes["loop.step"] = (config["loop"]["times"], W)
    for i, entry in enumerate(config["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        norm(p + "norm1"), norm(p + "norm1b")
        if entry["type"] == "latent_attention":
            H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            shapes.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],),
                           p + "mix.uq": (H * (D + R), m["q_rank"]), p + "mix.dkv": (m["kv_rank"] + R, W),
                           p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * D, m["kv_rank"]),
                           p + "mix.uv": (H * Dv, m["kv_rank"]), p + "mix.sink": (H,), p + "mix.o": (W, H * Dv)})
        elif entry["type"] == "mlstm":
            mem(p + "mix.", m)
        else:
            a = m["left"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            shapes.update({p + "mix.left.q": (H * D, W), p + "mix.left.k": (G * D, W), p + "mix.left.v": (G * Dv, W),
                           p + "mix.left.g": (H * Dv, W), p + "mix.left.o": (W, H * Dv)})
            mem(p + "mix.right.", m["right"])
        mlp = entry["mlp"]
        if mlp is not None:
            norm(p + "norm2"), norm(p + "norm2b")
            if mlp["kind"] == "dense":
                shapes.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
                shapes[p + "mlp.router"] = (E, W)
                names = [f"e{e}" for e in range(E)] + (["shared"] if mlp.get("shared") else [])
                for n in names:
                    f = mlp["shared"]["ff"] if n == "shared" else F
                    shapes.update({f"{p}mlp.{n}.gate": (f, W), f"{p}mlp.{n}.up": (f, W), f"{p}mlp.{n}.down": (W, f)})
        if side:
            shapes.update({p + "side.gate": (side["dim"], W), p + "side.proj": (W, side["dim"]), p + "side.norm": (W,)})
    return shapes


def random_tensor(name: str, shape: tuple, g: torch.Generator) -> torch.Tensor:
    r = lambda: torch.randn(shape, generator=g)  # noqa: E731
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "alpha":
        t = 0.6 + 0.1 * r()
    elif name.endswith(".b"):  # gate biases among them: forget gates a little open
        t = 0.4 * r() + (1.5 if name.endswith("f.b") else 0.0)
    elif leaf in ("norm1", "norm1b", "norm2", "norm2b", "norm") or name == "final.norm":
        t = 1.0 + 0.2 * r()
    elif leaf == "sink":  # of the size of the scores: it takes a visible share of the weight
        t = 1.0 + r()
    elif name in ("embed", "side.embed"):
        t = 0.7 * r()
    elif name == "loop.step":
        t = 0.3 * r()
    elif leaf == "router":  # scores spread between zero and one, so that few choices are near ties
        t = r() * (3.0 / shape[-1] ** 0.5)
    elif leaf == "down" and ".mlp.e" in name:  # a choice of experts that rounding turns over must not move a bfloat16
        t = r() * (0.2 / shape[-1] ** 0.5)     # run's logits by more than other rounding does
    else:  # a matrix [out, in]: outputs of order one for inputs of order one
        t = r() * (1.3 / shape[-1] ** 0.5)
    return t.to(torch.bfloat16)


def make_folder(folder: str, config: dict, seed: int, tweak=None) -> str:
    """config.json and model.safetensors (bfloat16) in ``folder``.  ``tweak(tensors)`` may change them first."""
    os.makedirs(folder, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    tensors = {name: random_tensor(name, shape, g) for name, shape in sorted(tensor_shapes(config).items())}
    if tweak is not None:
        tweak(tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder
