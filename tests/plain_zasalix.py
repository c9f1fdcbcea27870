"""A plain, slow statement of the Zasalix design in float64 on the CPU: one function per mechanism, written from
the mechanism's equations, sharing no code with the engine.  Whatever is carried from token to token (the latents of
a latent attention, the keys and values of a windowed one, the matrix memory of an mLSTM) is taken and returned
explicitly, so that a prompt can run whole, in portions or token by token through the same functions.

Notation: T tokens, W the stream's width, H heads.  ``w`` maps tensor names to float64 tensors.
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


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -torch.logaddexp(torch.zeros_like(z), -z)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def dynamic_tanh(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """The design's norm: no statistics at all, tanh(alpha x) w + b with a scalar alpha."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


# ---------------------------------------------------------------------- rotations
def _angles(positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    return torch.tensor(list(positions), dtype=F64)[:, None] * freq[None, :]  # [T, dims / 2]


def rotate_neighbours(v: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """v [T, heads, D]: of the first ``dims`` values, value 2i turns with value 2i + 1."""
    if dims == 0:
        return v
    a = _angles(positions, base, dims)
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = v.clone()
    u, s = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - s * sin
    out[..., 1:dims:2] = s * cos + u * sin
    return out


def rotate_halves(v: torch.Tensor, positions: Sequence[int], base: float, dims: int) -> torch.Tensor:
    """v [T, heads, D]: of the first ``dims`` values, value i turns with value i + dims / 2."""
    if dims == 0:
        return v
    a = _angles(positions, base, dims)
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    half = dims // 2
    out = v.clone()
    u, s = v[..., :half], v[..., half:dims]
    out[..., :half] = u * cos - s * sin
    out[..., half:dims] = s * cos + u * sin
    return out


# ---------------------------------------------------------------------- attention through a latent, with a sink
def latent_attention(h: torch.Tensor, w, pre: str, m: dict, eps: float, positions: Sequence[int], st: dict) -> torch.Tensor:
    """``st["c"]`` [n, kv_rank] and ``st["r"]`` [n, rot_dim] hold the earlier tokens' latents and rotated key parts."""
    T = h.shape[0]
    H, D, R, Dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    r_ = _round[-1]
    cq = r_(rms_norm(linear(h, w[pre + "dq"]), w[pre + "dq.norm"], eps))
    q = linear(cq, w[pre + "uq"]).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], r_(rotate_neighbours(q[..., D:], positions, base, dims))
    down = linear(h, w[pre + "dkv"])
    c = r_(rms_norm(down[:, :rank], w[pre + "dkv.norm"], eps))
    r = r_(rotate_neighbours(down[:, None, rank:], positions, base, dims)[:, 0])
    st["c"], st["r"] = torch.cat([st["c"], c]), torch.cat([st["r"], r])
    k_plain = linear(st["c"], w[pre + "uk"]).view(-1, H, D)
    val = linear(st["c"], w[pre + "uv"]).view(-1, H, Dv)
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t, p in enumerate(positions):
        for n in range(H):
            s = (k_plain[: p + 1, n] @ q_plain[t, n] + st["r"][: p + 1] @ q_rot[t, n]) * float(m["scale"])
            sink = w[pre + "sink"][n]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[t, n] = (e[:, None] * val[: p + 1, n]).sum(0) / (e.sum() + torch.exp(sink - top))
    return linear(out.reshape(T, H * Dv), w[pre + "o"])


# ---------------------------------------------------------------------- windowed attention that keeps the first tokens
def window_attention(h: torch.Tensor, w, pre: str, m: dict, positions: Sequence[int], st: dict) -> torch.Tensor:
    """Grouped-query heads; a query at i reads j <= i with i - j < size or j < keep_first; the heads' outputs are
    gated element by element.  ``st["k"]`` [n, G, D], ``st["v"]`` [n, G, Dv]."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    size, first = int(m["mask"]["size"]), int(m["mask"]["keep_first"])
    r_ = _round[-1]
    q = r_(rotate_halves(linear(h, w[pre + "q"]).view(T, H, D), positions, base, dims))
    k = r_(rotate_halves(linear(h, w[pre + "k"]).view(T, G, D), positions, base, dims))
    v = linear(h, w[pre + "v"]).view(T, G, Dv)
    st["k"], st["v"] = torch.cat([st["k"], k]), torch.cat([st["v"], v])
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t, p in enumerate(positions):
        seen = [j for j in range(p + 1) if p - j < size or j < first]
        for n in range(H):
            g = n // (H // G)
            s = (st["k"][seen, g] @ q[t, n]) * float(m["scale"])
            out[t, n] = torch.softmax(s, dim=0) @ st["v"][seen, g]
    gate = sigmoid(linear(h, w[pre + "g"]))
    return linear(out.reshape(T, H * Dv) * gate, w[pre + "o"])


# ---------------------------------------------------------------------- matrix memory
def matrix_memory(h: torch.Tensor, w, pre: str, m: dict, eps: float, st: dict) -> torch.Tensor:
    """The mLSTM cell: per head a memory S [D, Dv], a normaliser n [D] and a running maximum m of the log gates,
    all starting at zero; ``st["S"]`` [H, D, Dv], ``st["n"]`` [H, D], ``st["m"]`` [H]."""
    T = h.shape[0]
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = linear(h, w[pre + "q"]).view(T, H, D) * D ** -0.5
    k = linear(h, w[pre + "k"]).view(T, H, D)
    v = linear(h, w[pre + "v"]).view(T, H, Dv)
    gi = cap * torch.tanh((linear(h, w[pre + "i"]) + w[pre + "i.b"]) / cap)                 # [T, H], log input gate
    gf = log_sigmoid(cap * torch.tanh((linear(h, w[pre + "f"]) + w[pre + "f.b"]) / cap))    # log forget gate
    S, n, mx = st["S"].clone(), st["n"].clone(), st["m"].clone()
    out = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    st["S"], st["n"], st["m"] = S, n, mx
    y = rms_norm(out, None, eps).reshape(T, H * Dv) * w[pre + "norm"] * sigmoid(linear(h, w[pre + "g"]))
    return linear(y, w[pre + "o"])


# ---------------------------------------------------------------------- feed-forwards
def gated_expert(h: torch.Tensor, w, pre: str) -> torch.Tensor:
    return linear(silu(linear(h, w[pre + "gate"])) * linear(h, w[pre + "up"]), w[pre + "down"])


def feed_forward(h: torch.Tensor, w, pre: str, mlp: dict) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return linear(torch.relu(linear(h, w[pre + "up"])) ** 2, w[pre + "down"])
    top = int(mlp["router"]["top"])
    score = sigmoid(_round[-1](h) @ w[pre + "router"].t())
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(score.shape[1]), key=lambda e: (-float(score[t, e]), e))[:top]
        for e in chosen:  # the score scales what the expert reads
            out[t] += gated_expert((score[t, e] * h[t])[None], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, pre + "shared.")
    return out


def token_side(x: torch.Tensor, tokens: Sequence[int], w, pre: str, index: int, dim: int, eps: float) -> torch.Tensor:
    """What a layer adds from a second table of the token: a gated slice of the token's row, projected and normed."""
    e = w["side.embed"][torch.tensor(list(tokens))][:, index * dim:(index + 1) * dim]
    y = linear(gelu_tanh(linear(x, w[pre + "gate"])) * e, w[pre + "proj"])
    return x + rms_norm(y, w[pre + "norm"], eps)


# ---------------------------------------------------------------------- layers and the model
def run_order(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def new_state(config: dict) -> List[dict]:
    def memory(m):
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        return {"S": torch.zeros(H, D, Dv, dtype=F64), "n": torch.zeros(H, D, dtype=F64), "m": torch.zeros(H, dtype=F64)}

    states = []
    for i in run_order(config):
        spec = config["layers"][i]
        m = spec["mixer"]
        st = {"length": 0}
        if spec["type"] == "latent_attention":
            st.update(c=torch.zeros(0, m["kv_rank"], dtype=F64), r=torch.zeros(0, m["rot_dim"], dtype=F64))
        elif spec["type"] == "mlstm":
            st.update(memory(m))
        else:
            a = m["left"]
            st["left"] = {"k": torch.zeros(0, a["kv_heads"], a["dim"], dtype=F64),
                          "v": torch.zeros(0, a["kv_heads"], a["vdim"], dtype=F64)}
            st["right"] = memory(m["right"])
        states.append(st)
    return states


def mixer(h, w, pre, spec, eps, positions, st):
    m = spec["mixer"]
    if spec["type"] == "latent_attention":
        return latent_attention(h, w, pre, m, eps, positions, st)
    if spec["type"] == "mlstm":
        return matrix_memory(h, w, pre, m, eps, st)
    left = window_attention(h, w, pre + "left.", m["left"], positions, st["left"])
    right = matrix_memory(h, w, pre + "right.", m["right"], eps, st["right"])
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def layer(x, tokens, w, i, config, st, positions):
    spec, pre, eps = config["layers"][i], f"l{i}.", float(config["norm"]["eps"])
    x = x + dynamic_tanh(mixer(dynamic_tanh(x, w, pre + "norm1"), w, pre + "mix.", spec, eps, positions, st), w, pre + "norm1b")
    if spec.get("mlp"):
        x = x + dynamic_tanh(feed_forward(dynamic_tanh(x, w, pre + "norm2"), w, pre + "mlp.", spec["mlp"]), w, pre + "norm2b")
    if config.get("token_side"):
        x = token_side(x, tokens, w, pre + "side.", i, int(config["token_side"]["dim"]), eps)
    return x


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], state: Optional[List[dict]] = None,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a portion; ``state`` (``new_state``) carries what earlier portions left."""
    if state is None:
        state = new_state(config)
    start = state[0]["length"]
    positions = list(range(start, start + len(tokens)))
    x0 = w["embed"][torch.tensor(list(tokens))]
    x = x0
    loop = config.get("loop")
    first, span = (int(loop["start"]), int(loop["stop"]) - int(loop["start"])) if loop else (-1, 1)
    seen_first = 0
    for run, i in enumerate(run_order(config)):
        if i == first:  # a pass of the loop begins
            if seen_first > 0:
                x = x + x0
            x = x + w["loop.step"][seen_first]
            seen_first += 1
        x = layer(x, tokens, w, i, config, state[run], positions)
        state[run]["length"] = start + len(tokens)
        if layers_out is not None:
            layers_out.append(x.clone())
    return linear(dynamic_tanh(x, w, "final.norm"), w["head"])


def forward_logits(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    return forward(config, w, ids)


def rounding_error(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> float:
    """The largest difference that rounding every projection's operand and result (and what the caches hold) to
    bfloat16 makes to a logit of this prompt, relative to the largest logit."""
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
