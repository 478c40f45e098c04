"""Bezasun as data: its configuration turned into a ModelSpec of registered parts.

Every layer is a ``hyper_connections`` block: a pre-norm block over a residual stream of several copies, whose norms
store their weight around zero. The mixer is ``latent_attention`` (query latent, shared rotated key part with ramped
frequencies, interleaved pairs, sliding window), ``mamba2`` or ``attention`` (weighted q/k norm, no rotation, a query
temperature, capped scores, a distance bias per head, a learned sink). The feed-forward is ``routed_experts`` with
softmax scores over all experts that scale the experts' outputs, and a shared expert of its own size.
Checkpoint names: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.{in,out,mix}``,
``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}``.
"""
from __future__ import annotations

from typing import Optional

from ..config.bezasun import BezasunConfig
from .spec import LayerSpec, ModelSpec, PartSpec

DISTANCE_BIAS_EXPONENT = 8.0      # slope of head h: 2^(-8 (h + 1) / heads)


def _mixer(cfg: BezasunConfig, layer) -> PartSpec:
    m, w, eps = layer.mixer, cfg.width, cfg.eps
    if layer.kind == "latent_attention":
        scaling = None
        if m.rot.scaling is not None:
            scaling = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
        return PartSpec("latent_attention", {
            "name": "mix", "hidden_size": w, "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
            "q_rank": m.q_rank, "rot_dim": m.rot_dim, "rot_base": m.rot.base, "rot_scaling": scaling, "rot_kind": "yarn",
            "rot_interleaved": True, "scale": m.scale, "eps": eps, "gate": False,
            "window": ("sliding", m.window) if m.window else None})
    if layer.kind == "mamba2":
        return PartSpec("mamba2", {"name": "mix", "hidden_size": w, "heads": m.heads, "vdim": m.vdim, "state": m.state,
                                   "groups": m.groups, "conv": m.conv, "norm_groups": m.norm_groups, "eps": eps})
    return PartSpec("attention", {
        "name": "mix", "hidden_size": w, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
        "value_dim": m.vdim, "qk_norm_weighted": True, "qk_norm_eps": eps, "scale": m.scale, "names": "short",
        "temperature": (m.q_temp[1], m.q_temp[0]) if m.q_temp else None, "softcap": m.softcap,
        "distance_bias": DISTANCE_BIAS_EXPONENT, "sink": "learned"})


def build_bezasun_spec(cfg: BezasunConfig) -> ModelSpec:
    w = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"name": name, "size": w, "eps": cfg.eps, "tensor": "bare", "one_plus": True})

    layers = []
    for i, l in enumerate(cfg.layers):
        ffn = None
        if l.mlp is not None:
            ffn = PartSpec("routed_experts", {
                "name": "mlp", "hidden_size": w, "num_experts": l.mlp.experts, "top_k": l.mlp.top,
                "intermediate_size": l.mlp.ff, "shared_expert": l.mlp.shared_ff is not None,
                "shared_intermediate_size": l.mlp.shared_ff, "score": "softmax", "renormalize": False, "scale": "output",
                "names": "per_expert"})
        block = PartSpec("hyper_connections", {"hidden_size": w, "streams": cfg.streams or 1, "mult": cfg.residual_mult,
                                               "learned": cfg.streams is not None, "feed_forward": ffn is not None})
        layers.append(LayerSpec(prefix=f"l{i}", mixer=_mixer(cfg, l), feed_forward=ffn, norm_mixer=norm("norm1"),
                                norm_feed_forward=norm("norm2") if ffn is not None else None, arrangement=block))
    return ModelSpec(
        hidden_size=w, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": cfg.vocab, "hidden_size": w,
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=ModelSpec.sequential(len(layers)), final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"name": "head", "vocab_size": cfg.vocab, "hidden_size": w, "tensor": "head",
                                      "scale": cfg.logit_scale}),
        eos_token_ids=cfg.eos_token_ids, max_position_embeddings=None)


def normalize_bezasun_tensor_name(name: str) -> Optional[str]:
    """The parts ask for the checkpoint's own names, but for the embedding table (``embed`` is the
    token-embedding part's ``embed.weight``)."""
    return "embed.weight" if name == "embed" else name
