"""Surinex as data: its configuration turned into a ModelSpec of registered parts.

Every layer is a ``parallel_conv`` block (one RMS norm; the mixer and a dense SwiGLU feed-forward read it side by
side, each through its own short causal convolution over time). The mixer is ``gla`` (gated linear attention),
``latent_attention`` (query latent, shared rotated key part, softmax) or a ``mixer_pair`` of ``attention`` with
sigmoid weights and rotated values beside ``gated_delta`` with one decay per head. A range of layers may run
several times with the same weights: every run is a schedule entry with a cache slot of its own, and the run
that opens a pass has the ``pass_offset`` interlude in front of it.
Checkpoint names: ``embed``, ``head``, ``final.norm``, ``loop.step``, ``l<i>.norm1``, ``l<i>.canon1|canon2``,
``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``.
"""
from __future__ import annotations

from typing import Optional

from ..config.surinex import SurinexConfig
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _scaling(rot):
    if rot is None or rot.scaling is None:
        return None
    factor, low, high, original = rot.scaling
    return {"factor": factor, "low_freq_factor": low, "high_freq_factor": high,
            "original_max_position_embeddings": original}


def _mixer(cfg: SurinexConfig, layer) -> PartSpec:
    m, w, eps = layer.mixer, cfg.width, cfg.eps
    if layer.kind == "gla":
        return PartSpec("gla", {"name": "mix", "hidden_size": w, "heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                "tau": m.tau, "decay_rank": m.decay_rank or 16, "eps": eps})
    if layer.kind == "latent_attention":
        return PartSpec("latent_attention", {
            "name": "mix", "hidden_size": w, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
            "q_rank": m.q_rank, "rot_dim": m.rot_dim, "rot_base": m.rot.base, "rot_scaling": _scaling(m.rot),
            "scale": m.scale, "eps": eps, "gate": False})
    left, right = m
    position = PartSpec("rope", {"head_dim": left.dim, "rot_dim": left.rot.dims, "theta": left.rot.base,
                                 "scaling": _scaling(left.rot), "interleaved": True, "exact": True})
    return PartSpec("mixer_pair", {
        "name": "mix", "hidden_size": w, "eps": eps,
        "left": {"kind": "attention", "params": {
            "hidden_size": w, "num_heads": left.heads, "num_kv_heads": left.kv_heads, "head_dim": left.dim,
            "value_dim": left.vdim, "position": position, "qk_norm_weighted": True, "qk_norm_eps": eps,
            "scale": left.scale, "names": "short", "weights": "sigmoid",
            "value_rotation": {"base": left.rot.base, "interleaved": True}}},
        "right": {"kind": "gated_delta", "params": {
            "hidden_size": w, "heads": right.heads, "kv_heads": right.kv_heads, "dim": right.dim, "vdim": right.vdim,
            "conv": right.conv, "decay_per": "head", "gate": "silu", "eps": eps}}})


def build_surinex_spec(cfg: SurinexConfig) -> ModelSpec:
    w = cfg.width
    layers = []
    for i, l in enumerate(cfg.layers):
        ffn = None if l.ff is None else PartSpec("dense_swiglu", {"name": "mlp", "hidden_size": w,
                                                                 "intermediate_size": l.ff, "names": "short"})
        norm = PartSpec("rmsnorm", {"name": "norm1", "size": w, "eps": cfg.eps, "tensor": "bare"})
        layers.append(LayerSpec(prefix=f"l{i}", mixer=_mixer(cfg, l), feed_forward=ffn, norm_mixer=norm,
                                norm_feed_forward=None,
                                arrangement=PartSpec("parallel_conv", {"hidden_size": w, "taps": cfg.taps,
                                                                       "feed_forward": ffn is not None})))
    n = len(layers)
    order = [(i, None) for i in range(n)]
    interludes = ()
    if cfg.loop is not None:
        lo, hi, times = cfg.loop.start, cfg.loop.stop, cfg.loop.times
        order = [(i, None) for i in range(lo)]
        for t in range(times):
            order += [(i, t if i == lo else None) for i in range(lo, hi)]
        order += [(i, None) for i in range(hi, n)]
        interludes = (PartSpec("pass_offset", {"name": "loop.step", "hidden_size": w, "times": times,
                                               "add_embedding": True}),)
    schedule = tuple(ScheduleEntry(layer=i, cache=run, interlude=None if opens is None else 0,
                                   interlude_arg=opens or 0) for run, (i, opens) in enumerate(order))
    return ModelSpec(
        hidden_size=w, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": cfg.vocab, "hidden_size": w}),
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"name": "final.norm", "size": w, "eps": cfg.eps, "tensor": "bare"}),
        head=PartSpec("linear_head", {"name": "head", "vocab_size": cfg.vocab, "hidden_size": w, "tensor": "head"}),
        eos_token_ids=cfg.eos_token_ids, max_position_embeddings=None, interludes=interludes)


def normalize_surinex_tensor_name(name: str) -> Optional[str]:
    """The parts ask for the checkpoint's own names, but for the embedding table (``embed`` is the
    token-embedding part's ``embed.weight``)."""
    return "embed.weight" if name == "embed" else name
