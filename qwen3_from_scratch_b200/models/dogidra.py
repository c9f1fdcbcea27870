"""Dogidra as a model specification: pre-norm blocks with layer norms and a short causal convolution in front of
every sub-layer; a mixer that runs, side by side on the same input, softmax attention over a sliding window with
pooled blocks before it and a gated recurrence; a feed-forward of routed experts with a shared one, or none.  The
embedding is scaled and tied to the head.  A span of layers may run several times; every pass is entered through
one projection of [stream | embedding output].

Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1`` / ``.norm1.b``, ``l<i>.norm2`` / ``.norm2.b``, ``l<i>.canon1``,
``l<i>.canon2``, ``l<i>.mix.left.{q,k,v,q.norm,k.norm,o}``, ``l<i>.mix.right.{z,z.b,x,x.b,g,o}``,
``l<i>.mlp.{router,correction,e<n>.up,e<n>.down,shared.up,shared.down}``, ``final.norm`` / ``final.norm.b``.  A looped
span becomes further entries of the run order on the same layers, each with a cache id (pages, state slots) of its own.
"""

from __future__ import annotations

from ..config.dogidra_config import ARCHITECTURE, DogidraConfig, DogidraLayer
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..registry import register_architecture

# constants of the design (what config.json cannot change)
YARN_MAGNITUDE = (0.1, 1.0)  # sines and cosines are multiplied by 0.1 * ln(factor) + 1
EXPERT_ACTIVATION = "relu_sq"  # the square of relu, in routed and shared experts alike
REENTRY_TENSOR = "loop.in"
_BLOCK_NAMES = {"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feed_forward": "mlp", "conv1": "canon1",
                "conv2": "canon2"}


def _mixer(layer: DogidraLayer, cfg: DogidraConfig) -> PartSpec:
    a = layer.left
    scaling = None
    if a.rot_scaling is not None:
        s = a.rot_scaling
        scaling = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow, "magnitude": YARN_MAGNITUDE}
    left = PartSpec("pooled_window_attention", {
        "hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
        "scale": a.scale, "softcap": a.softcap, "window": a.window, "pool": a.pool, "norm_eps": cfg.norm_eps,
        "position": PartSpec("rotary_stretched", {"dims": a.rot_dims, "base": a.rot_base, "scaling": scaling})})
    right = PartSpec("mingru", {"hidden_size": cfg.width, "width": layer.right_width})
    return PartSpec("parallel", {"hidden_size": cfg.width, "branches": [
        {"label": "left", "mixer": left, "scale": layer.left_scale},
        {"label": "right", "mixer": right, "scale": layer.right_scale}]})


def _feed_forward(layer: DogidraLayer, cfg: DogidraConfig):
    e = layer.mlp
    if e is None:
        return None
    shared = None
    if e.shared_ff is not None:
        shared = PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": e.shared_ff,
                                        "activation": EXPERT_ACTIVATION, "names": {"up": "up", "down": "down"}})
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "experts": e.experts, "top": e.top,
                                       "expert_ff": e.expert_ff, "router_scale": e.router_scale,
                                       "activation": EXPERT_ACTIVATION, "shared": shared})


@register_architecture(ARCHITECTURE, DogidraConfig)
def dogidra_spec(cfg: DogidraConfig) -> ModelSpec:
    norm = PartSpec("layer_norm", {"dim": cfg.width, "eps": cfg.norm_eps, "suffix": "", "bias_suffix": ".b"})
    layers, ignorable = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _feed_forward(layer, cfg)
        if ff is None:  # a folder may still carry what a feed-forward's norm and convolution would need
            ignorable += [f"l{i}.norm2", f"l{i}.norm2.b", f"l{i}.canon2"]
        layers.append((f"l{i}", PartSpec("pre_norm", {
            "norm1": norm, "mixer": _mixer(layer, cfg), "norm2": norm if ff else None, "feed_forward": ff,
            "names": _BLOCK_NAMES, "conv_taps": cfg.taps, "width": cfg.width,
            "reentry": REENTRY_TENSOR if cfg.loop is not None and i == cfg.loop[0] else None})))
    if cfg.loop is None:
        ignorable.append(REENTRY_TENSOR)
    order = [LayerCall(layer=i, cache=run) for run, i in enumerate(cfg.run_order())]
    return ModelSpec(
        embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "suffix": "",
                                                         "scale": cfg.embedding_scale})),
        layers=layers, order=order,
        final_norm=("final.norm", norm),
        head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed"})),
        vocab_size=cfg.vocab,
        max_positions=1 << 30,  # nothing in the design depends on a longest position
        ignorable_weights=tuple(ignorable),
        eos_token_id=cfg.eos_token_id,
    )
