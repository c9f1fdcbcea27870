"""Zasalix as a model specification: blocks with a Dynamic Tanh (tanh(alpha x) w + b, no statistics) before and after
every sub-layer; per layer one of three mixers (attention through a latent with a sink in its softmax; an mLSTM matrix
memory; windowed attention that keeps a request's first tokens, gated, side by side with such a memory); a dense
feed-forward with the square of relu, a feed-forward of routed gated experts whose router weight scales what the
expert reads, or none; after each layer a term made from the layer's slice of a second embedding of the token.  A span
of layers may run several times: each pass starts by adding a vector of its own and, from the second pass on, the
embedding's output.

Tensor names: ``embed``, ``head``, ``side.embed``, ``loop.step``, ``final.norm`` / ``.b`` / ``.alpha``, per layer
``l<i>.norm1`` / ``norm1b`` / ``norm2`` / ``norm2b`` (each with ``.b`` and ``.alpha``), ``l<i>.mix.*`` (latent attention:
``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o``; mLSTM: ``q, k, v, g, i, i.b, f, f.b, norm, o``; parallel: ``left.{q,k,v,g,o}``
and ``right.*`` as an mLSTM), ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router, e<n>.{gate,up,down}, shared.{gate,up,down}}``,
``l<i>.side.{gate,proj,norm}``.  A looped span becomes further entries of the run order on the same layers, each with a
cache id (pages, state slots) of its own.
"""

from __future__ import annotations

from ..config.zasalix_config import ARCHITECTURE, DenseFF, MatrixMemory, RoutedFF, ZasalixConfig, ZasalixLayer
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..registry import register_architecture

# constants of the design (what config.json cannot change)
DENSE_ACTIVATION = "relu_sq"   # the dense feed-forward: W_down relu(W_up h)^2
EXPERT_ACTIVATION = "silu"     # routed and shared experts: W_down (silu(W_gate h) * (W_up h))
LATENT_PAIRING = "neighbours"  # the latent attention turns value 2i with value 2i + 1
LOOP_STEP_TENSOR = "loop.step"
SIDE_TABLE = "side.embed"
_BLOCK_NAMES = {"norm1": "norm1", "norm1b": "norm1b", "mixer": "mix", "norm2": "norm2", "norm2b": "norm2b",
                "feed_forward": "mlp", "side": "side"}


def _memory(m: MatrixMemory, cfg: ZasalixConfig) -> PartSpec:
    return PartSpec("mlstm", {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                              "gate_cap": m.gate_cap, "norm_eps": cfg.norm_eps})


def _mixer(layer: ZasalixLayer, cfg: ZasalixConfig) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
            "kv_rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "norm_eps": cfg.norm_eps, "gate": False, "sink": True,
            "pairing": LATENT_PAIRING, "position": PartSpec("rotary_stretched", {"dims": m.rot_dims, "base": m.rot_base})})
    if layer.type == "mlstm":
        return _memory(m, cfg)
    a = m.left
    left = PartSpec("kept_window_attention", {
        "hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
        "scale": a.scale, "window": a.window, "keep_first": a.keep_first, "gate": True,
        "position": PartSpec("rotary_stretched", {"dims": a.rot_dims, "base": a.rot_base})})
    return PartSpec("parallel", {"hidden_size": cfg.width, "branches": [
        {"label": "left", "mixer": left, "scale": m.left_scale},
        {"label": "right", "mixer": _memory(m.right, cfg), "scale": m.right_scale}]})


def _feed_forward(layer: ZasalixLayer, cfg: ZasalixConfig):
    e = layer.mlp
    if e is None:
        return None
    if isinstance(e, DenseFF):
        return PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": e.ff, "activation": DENSE_ACTIVATION,
                                      "names": {"up": "up", "down": "down"}})
    assert isinstance(e, RoutedFF)
    shared = None
    if e.shared_ff is not None:
        shared = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": e.shared_ff,
                                        "activation": EXPERT_ACTIVATION, "names": {"gate": "gate", "up": "up", "down": "down"}})
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "experts": e.experts, "top": e.top, "expert_ff": e.expert_ff,
                                       "router_scale": 1.0, "activation": EXPERT_ACTIVATION, "correction": False,
                                       "gated": True, "weigh": "input", "shared": shared})


@register_architecture(ARCHITECTURE, ZasalixConfig)
def zasalix_spec(cfg: ZasalixConfig) -> ModelSpec:
    def norm(_=None):
        return PartSpec("dynamic_tanh", {"dim": cfg.width, "suffix": "", "bias_suffix": ".b", "alpha_suffix": ".alpha"})

    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(layer, cfg)
        if ff is None:  # a folder may still carry the norms around a feed-forward that is not there
            ignorable += [f"l{i}.{n}{s}" for n in ("norm2", "norm2b") for s in ("", ".b", ".alpha")]
        entry = None
        if cfg.loop is not None and i == cfg.loop[0]:
            entry = {"step": LOOP_STEP_TENSOR, "times": cfg.loop[2], "embedding": True}
        side = None
        if cfg.side_dim is not None:
            side = {"column": i * cfg.side_dim, "dim": cfg.side_dim, "eps": cfg.norm_eps}
        layers.append((f"l{i}", PartSpec("sandwich_norm", {
            "width": cfg.width, "norm1": norm(), "norm1b": norm(), "mixer": _mixer(layer, cfg),
            "norm2": norm() if ff else None, "norm2b": norm() if ff else None, "feed_forward": ff, "entry": entry,
            "side": side, "names": _BLOCK_NAMES})))
    if cfg.loop is None:
        ignorable.append(LOOP_STEP_TENSOR)
    order = [LayerCall(layer=i, cache=run, repeat=t) for run, (i, t, _) in enumerate(cfg.run_order())]
    embedding = {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "suffix": ""}
    if cfg.side_dim is not None:
        embedding.update(side_table=SIDE_TABLE, side_width=len(cfg.layers) * cfg.side_dim)
    return ModelSpec(
        embedding=("embed", PartSpec("token_embedding", embedding)),
        layers=layers, order=order,
        final_norm=("final.norm", norm()),
        head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "suffix": ""})),
        vocab_size=cfg.vocab,
        max_positions=1 << 30,  # nothing in the design depends on a longest position
        ignorable_weights=tuple(ignorable),
        eos_token_id=cfg.eos_token_id,
    )
