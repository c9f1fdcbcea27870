"""A plain, slow statement of the Dogidra design in float64 on the CPU: one function per mechanism, written
from the mechanism's equations, sharing no code with the engine.  Whatever is carried from token to token (the
keys and values of an attention, the state of the recurrence, the last inputs of the short convolutions) is taken
and returned explicitly, so that a prompt can run whole, in portions or token by token through the same
functions.

Notation: T tokens, W the stream's width.  ``w`` maps tensor names to float64 tensors.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open

F64 = torch.float64

# What a projection does to its operand and its result: nothing, or (inside ``bfloat16_projections()``) rounding
# both to bfloat16, which is where a bfloat16 run rounds.
_round = [lambda t: t]


class bfloat16_projections:
    def __enter__(self):
        _round.append(lambda t: t.to(torch.bfloat16).to(F64))

    def __exit__(self, *exc):
        _round.pop()


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x W^T for a weight stored [out, in]."""
    r = _round[-1]
    return r(r(x) @ weight.t())


def read_model_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            t = f.get_tensor(name)
            w[name] = t.to(F64) if t.is_floating_point() else t
    return config, w


# ---------------------------------------------------------------------- small functions
def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


# ---------------------------------------------------------------------- the convolution in front of a sub-layer
def input_conv(h: torch.Tensor, taps_w: torch.Tensor, tail: torch.Tensor):
    """h [T, W] -> (h + conv(h), new tail).  conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) with zeros before the
    sequence's start; ``tail`` [taps - 1, W] holds the inputs before this portion, oldest first."""
    taps = taps_w.shape[1]
    T = h.shape[0]
    ext = torch.cat([tail, h], dim=0)  # row i is the input at time i - (taps - 1)
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            out[t] = out[t] + taps_w[:, j] * ext[t + j]
    return out, ext[ext.shape[0] - (taps - 1):].clone()


# ---------------------------------------------------------------------- rotation with stretched frequencies
def stretched_frequencies(rot: dict):
    """(frequency per pair [dims / 2], factor on sines and cosines)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    s = rot.get("scaling")
    if not s:
        return torch.tensor(freq, dtype=F64), 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def pair(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(float(s["fast"]))), 0)
    hi = min(math.ceil(pair(float(s["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(freq[i] / factor * ramp + freq[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: Sequence[int], rot: dict) -> torch.Tensor:
    """x [T, heads, D]: the first rot.dims values of every head are rotated, pair (i, i + dims / 2)."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    freq, mag = stretched_frequencies(rot)
    ang = torch.tensor(list(positions), dtype=F64)[:, None] * freq[None, :]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------- the left mixer: attention
def visible(i: int, size: int, pool: int):
    """What position i reads: (positions j with 0 <= i - j < size, pooled blocks b with b pool + pool - 1 <= i - size)."""
    tokens = list(range(max(0, i - size + 1), i + 1))
    blocks = [b for b in range((i // pool) + 1) if b * pool + pool - 1 <= i - size]
    return tokens, blocks


def windowed_pooled_attention(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, positions: Sequence[int],
                              m: dict) -> torch.Tensor:
    """q [T, H, D] at ``positions``; keys [L, G, D], values [L, G, Dv] of positions 0 .. L - 1 as the cache holds
    them.  Returns [T, H * Dv]."""
    H, G = int(m["heads"]), int(m["kv_heads"])
    size, pool = int(m["mask"]["size"]), int(m["mask"]["pool"])
    scale, cap = float(m["scale"]), m.get("softcap")
    out = torch.zeros(q.shape[0], H, values.shape[-1], dtype=F64)
    for t, i in enumerate(positions):
        tokens, blocks = visible(i, size, pool)
        for h in range(H):
            g = h // (H // G)
            ks = [keys[j, g] for j in tokens] + [keys[b * pool:(b + 1) * pool, g].mean(dim=0) for b in blocks]
            vs = [values[j, g] for j in tokens] + [values[b * pool:(b + 1) * pool, g].mean(dim=0) for b in blocks]
            score = torch.stack(ks) @ q[t, h] * scale
            if cap:
                score = float(cap) * torch.tanh(score / float(cap))
            p = torch.softmax(score, dim=0)
            out[t, h] = p @ torch.stack(vs)
    return out.reshape(q.shape[0], -1)


def left_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, m: dict, eps: float, positions: Sequence[int],
               cache: dict) -> torch.Tensor:
    """``cache``: {"k": [L, G, D], "v": [L, G, Dv]} of the positions before this portion; grows in place."""
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = rms_norm(linear(h, w[pre + "q"]), w[pre + "q.norm"], eps)
    k = rms_norm(linear(h, w[pre + "k"]), w[pre + "k.norm"], eps)
    v = linear(h, w[pre + "v"])
    q = rotate(q.view(T, H, D), positions, m["rot"])
    k = rotate(k.view(T, G, D), positions, m["rot"])
    r = _round[-1]  # a bfloat16 run's cache holds rounded keys and values
    cache["k"] = torch.cat([cache["k"], r(k)], dim=0)
    cache["v"] = torch.cat([cache["v"], r(v.view(T, G, Dv))], dim=0)
    o = windowed_pooled_attention(q, cache["k"], cache["v"], positions, m)
    return linear(o, w[pre + "o"])


# ---------------------------------------------------------------------- the right mixer: a gated recurrence
def min_gru(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, state: torch.Tensor):
    """Returns (output [T, W], state after the portion [width])."""
    z = sigmoid(linear(h, w[pre + "z"]) + w[pre + "z.b"])
    u = linear(h, w[pre + "x"]) + w[pre + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(linear(h, w[pre + "g"]))
    rows = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        rows.append(state * gate[t])
    return linear(torch.stack(rows), w[pre + "o"]), state


# ---------------------------------------------------------------------- the feed-forward: routed experts
def expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return linear(torch.relu(linear(h, up)).pow(2), down)


def routed_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    E, top, rscale = int(r["experts"]), int(r["top"]), float(r["scale"])
    s = sigmoid(_round[-1](h) @ w[pre + "router"].t())  # the router's product is not rounded
    choice = s + w[pre + "correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(choice[t], top).indices.tolist()
        for e in chosen:
            out[t] = out[t] + s[t, e] * rscale * expert(h[t:t + 1], w[f"{pre}e{e}.up"], w[f"{pre}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + expert(h, w[pre + "shared.up"], w[pre + "shared.down"])
    return out


# ---------------------------------------------------------------------- a layer, the loop, the model
def run_order(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def new_state(config: dict) -> List[dict]:
    """One record per layer run (a looped layer has one per pass)."""
    W, taps = int(config["width"]), int(config["canon"]["taps"])
    state = []
    for i in run_order(config):
        m = config["layers"][i]["mixer"]
        left = m["left"]
        state.append({"tail1": torch.zeros(taps - 1, W, dtype=F64), "tail2": torch.zeros(taps - 1, W, dtype=F64),
                      "k": torch.zeros(0, int(left["kv_heads"]), int(left["dim"]), dtype=F64),
                      "v": torch.zeros(0, int(left["kv_heads"]), int(left["vdim"]), dtype=F64),
                      "s": torch.zeros(int(m["right"]["width"]), dtype=F64), "length": 0})
    return state


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, config: dict, st: dict, positions) -> torch.Tensor:
    spec, eps, pre = config["layers"][i], float(config["norm"]["eps"]), f"l{i}."
    if spec["type"] != "parallel":
        raise ValueError(spec["type"])
    m = spec["mixer"]
    h = layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps)
    h, st["tail1"] = input_conv(h, w[pre + "canon1"], st["tail1"])
    left = left_mixer(h, w, pre + "mix.left.", m["left"], eps, positions, st)
    right, st["s"] = min_gru(h, w, pre + "mix.right.", st["s"])
    x = x + float(m["left_scale"]) * left + float(m["right_scale"]) * right
    if spec.get("mlp"):
        h = layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps)
        h, st["tail2"] = input_conv(h, w[pre + "canon2"], st["tail2"])
        x = x + routed_experts(h, w, pre + "mlp.", spec["mlp"])
    return x


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], state: Optional[List[dict]] = None,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a portion; ``state`` (``new_state``) carries what earlier portions left."""
    if state is None:
        state = new_state(config)
    start = state[0]["length"]
    positions = list(range(start, start + len(tokens)))
    x0 = w["embed"][torch.tensor(list(tokens))] * float(config["embedding"]["scale"])
    x = x0
    loop = config.get("loop")
    for run, i in enumerate(run_order(config)):
        if loop and i == int(loop["start"]):
            x = linear(torch.cat([x, x0], dim=-1), w["loop.in"])
        x = layer(x, w, i, config, state[run], positions)
        state[run]["length"] = start + len(tokens)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], float(config["norm"]["eps"]))
    return linear(x, w["embed"])


def forward_logits(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    return forward(config, w, ids)


def rounding_error(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> float:
    """The largest difference that rounding every projection's operand and result (and the cached keys and values)
    to bfloat16 makes to a logit of this prompt, relative to the largest logit."""
    exact = forward(config, w, ids)
    with bfloat16_projections():
        rounded = forward(config, w, ids)
    return float((rounded - exact).abs().max()) / float(exact.abs().max())


def greedy(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], new_tokens: int):
    """(generated ids, gap between the two largest logits at every step), token by token through the states."""
    state = new_state(config)
    logits = forward(config, w, prompt, state)
    out, margins = [], []
    for _ in range(new_tokens):
        top = torch.topk(logits[-1], 2).values
        margins.append(float(top[0] - top[1]))
        out.append(int(torch.argmax(logits[-1])))
        logits = forward(config, w, [out[-1]], state)
    return out, margins
