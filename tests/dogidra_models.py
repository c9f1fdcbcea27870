"""Small Dogidra configurations and model folders for the tests: the configuration dicts, the tensors the design
names for them (names and shapes restated here from the design, not asked of the engine) and random weights strong
enough that every mechanism moves the logits."""

from __future__ import annotations

import json
import os
from typing import Dict

import torch
from safetensors.torch import save_file


def layer(heads, kv_heads, dim, vdim, scale, window, pool, base, dims, right, left_scale=1.0, right_scale=1.0,
          softcap=None, scaling=None, moe=None):
    """``moe``: (experts, top, expert ff, router scale, shared ff or None) or None for a layer without feed-forward."""
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "pool": pool}, "rot": rot}
    if softcap is not None:
        left["softcap"] = softcap
    mlp = None
    if moe is not None:
        experts, top, ff, rscale, shared = moe
        mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": rscale}}
        if shared is not None:
            mlp["shared"] = {"ff": shared}
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "left_scale": left_scale, "right": {"width": right}, "right_scale": right_scale}}


# X: a loop of three passes over the middle; every layer with sizes of its own; windows of 9, 5 and 16 tokens with
# blocks of 4, 7 (longer than its window) and 3; two and three query heads per key head; a partly rotated head with
# stretched frequencies; a layer without feed-forward; one without a shared expert; one without a cap.
DOGIDRA_X = {
    "architecture": "Dogidra", "vocab": 211, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "canon": {"taps": 4}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [layer(4, 2, 24, 40, 0.2, 9, 4, 10000.0, 16, 72, 0.7, 1.2, softcap=5.0, scaling=(4.0, 64, 8.0, 1.0),
                     moe=(6, 2, 24, 1.5, 40)),
               layer(6, 2, 16, 8, 0.3, 5, 7, 500.0, 16, 40, 1.1, 0.6, moe=None),
               layer(3, 3, 8, 24, 0.4, 16, 3, 100.0, 4, 56, 0.9, 0.8, softcap=50.0, moe=(5, 1, 32, 2.5, None)),
               layer(2, 1, 32, 16, 0.15, 7, 2, 10000.0, 32, 24, 1.0, 1.0, softcap=8.0, scaling=(16.0, 32, 4.0, 0.5),
                     moe=(4, 4, 16, 0.5, 24))]}
# Y: no loop at all, a single tap (no tail to keep), one head, blocks of one token, a window of one, every expert
# chosen, no rotation in the second layer.
DOGIDRA_Y = {
    "architecture": "Dogidra", "vocab": 173, "width": 48, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "canon": {"taps": 1},
    "layers": [layer(1, 1, 32, 24, 0.18, 6, 1, 10000.0, 8, 40, moe=(3, 3, 40, 1.0, 56)),
               layer(5, 5, 8, 16, 0.25, 1, 5, 200000.0, 0, 88, 0.5, 1.5, softcap=3.0, moe=(9, 2, 8, 3.0, 16))]}
# Z: sizes in the manner of the serving kernels, small: heads of 64 and 128, a window of 64 with blocks of 16, widths
# in multiples of 64; the loop is the whole model and starts at the first layer; two taps.
DOGIDRA_Z = {
    "architecture": "Dogidra", "vocab": 300, "width": 128, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
    "canon": {"taps": 2}, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [layer(8, 2, 64, 64, 0.11, 64, 16, 1000000.0, 64, 128, 0.8, 1.1, softcap=20.0,
                     scaling=(6.0, 256, 16.0, 2.0), moe=(8, 2, 72, 1.75, 192)),
               layer(4, 1, 128, 128, 0.09, 48, 32, 10000.0, 64, 256, 1.0, 1.0, moe=(12, 4, 48, 1.0, 64))]}
CONFIGS = {"x": (DOGIDRA_X, 3), "y": (DOGIDRA_Y, 4), "z": (DOGIDRA_Z, 5)}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V, K = config["width"], config["vocab"], config["canon"]["taps"]
    shapes = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    if config.get("loop"):
        shapes["loop.in"] = (W, 2 * W)
    for i, entry in enumerate(config["layers"]):
        p, m = f"l{i}.", entry["mixer"]
        a, C = m["left"], m["right"]["width"]
        H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        shapes.update({p + "norm1": (W,), p + "norm1.b": (W,), p + "canon1": (W, K),
                       p + "mix.left.q": (H * D, W), p + "mix.left.k": (G * D, W), p + "mix.left.v": (G * Dv, W),
                       p + "mix.left.q.norm": (H * D,), p + "mix.left.k.norm": (G * D,), p + "mix.left.o": (W, H * Dv),
                       p + "mix.right.z": (C, W), p + "mix.right.z.b": (C,), p + "mix.right.x": (C, W),
                       p + "mix.right.x.b": (C,), p + "mix.right.g": (C, W), p + "mix.right.o": (W, C)})
        mlp = entry["mlp"]
        if mlp is not None:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            shapes.update({p + "norm2": (W,), p + "norm2.b": (W,), p + "canon2": (W, K), p + "mlp.router": (E, W),
                           p + "mlp.correction": (E,)})
            for e in range(E):
                shapes.update({f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            if mlp.get("shared"):
                S = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.up": (S, W), p + "mlp.shared.down": (W, S)})
    return shapes


def random_tensor(name: str, shape: tuple, g: torch.Generator) -> torch.Tensor:
    r = lambda: torch.randn(shape, generator=g)  # noqa: E731
    if name.endswith(("norm1", "norm2", ".norm")):
        t = 1.0 + 0.2 * r()
    elif name.endswith("correction"):  # of the size of the differences between scores: it changes who is chosen
        t = 0.3 * r()
    elif name.endswith(".b"):
        t = 0.4 * r()
    elif name.endswith(("canon1", "canon2")):
        t = 0.5 * r()
    elif name == "embed":
        t = 0.5 * r()
    elif name.endswith("router"):  # scores spread between zero and one, so that few choices are near ties
        t = r() * (3.0 / shape[-1] ** 0.5)
    elif name.endswith(".down"):  # the square of relu grows quickly; and a choice of experts that rounding turns
        t = r() * (0.1 / shape[-1] ** 0.5)  # over must not move a bfloat16 run's logits by more than other rounding
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
