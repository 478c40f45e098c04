"""Typed configuration of the Bezasun decoder: pre-norm layers over a residual stream kept as several copies
(hyper-connections), three kinds of mixer, and a mixture of experts with a shared expert as feed-forward.

config.json keys: ``architecture`` ("Bezasun"), ``vocab``, ``width``, ``norm.eps``, optionally ``embedding.scale``
(default 1), ``logit_scale`` (default 1), ``residual_mult`` (default 1), ``streams`` (copies of the residual stream;
absent: one plain stream without learned coefficients), and ``layers``: a list of
``{"type": "latent_attention" | "mamba2" | "attention", "mixer": {...}, "mlp": {...} | null}``.

Mixer keys.
  latent_attention  ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale``; ``rot`` = ``{base, dims, scaling?}`` with
                    ``scaling`` = ``{factor, original, fast, slow}`` (``rot.dims`` = ``rot_dim``); ``mask.size``
                    (optional: a query reads itself and the ``size - 1`` tokens before it)
  mamba2            ``heads, vdim, state, groups, conv, norm_groups``
  attention         ``heads, kv_heads, dim, vdim, scale``; optional ``softcap``, ``q_temp`` = ``{coef, every}``
mlp keys: ``kind`` ("moe"), ``router.experts``, ``router.top``, ``expert.ff``, optional ``shared.ff``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, get_key, token_ids

MIXERS = ("latent_attention", "mamba2", "attention")


@dataclass(frozen=True)
class BezasunRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow


@dataclass(frozen=True)
class BezasunLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: BezasunRotation
    window: Optional[int] = None


@dataclass(frozen=True)
class BezasunMamba:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class BezasunAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float] = None
    q_temp: Optional[Tuple[float, float]] = None                     # coef, every


@dataclass(frozen=True)
class BezasunMoe:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int] = None


@dataclass(frozen=True)
class BezasunLayer:
    kind: str
    mixer: Any                        # BezasunLatent | BezasunMamba | BezasunAttention
    mlp: Optional[BezasunMoe]


@dataclass(frozen=True)
class BezasunConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[BezasunLayer, ...]
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    residual_mult: float = 1.0
    streams: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = ("Bezasun",)

    @staticmethod
    def from_json(raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "BezasunConfig":
        def obj(parent, key, where, required=True):
            value = parent.get(key)
            if value is None and not required:
                return None
            if not isinstance(value, dict):
                raise ConfigError(f"config.json: required key '{where}' is missing or not an object")
            return value

        def need(parent, key, typ, where):
            try:
                return get_key(parent, key, typ, required=True)
            except ConfigError as e:
                raise ConfigError(str(e).replace("key '", f"key '{where}.")) from None

        def sizes(parent, keys, where):
            values = [need(parent, k, int, where) for k in keys]
            if min(values) <= 0:
                raise ConfigError(f"config.json: {where}: {', '.join(keys)} must be positive")
            return values

        def number(parent, key, where, default):
            value = get_key(parent, key, float) if parent is not None else None
            return default if value is None else value

        vocab = get_key(raw, "vocab", int, required=True)
        width = get_key(raw, "width", int, required=True)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = need(obj(raw, "norm", "norm"), "eps", float, "norm")
        streams = get_key(raw, "streams", int)
        if streams is not None and not 1 <= streams <= 16:
            raise ConfigError("config.json: 'streams' must be between 1 and 16")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json: {where} needs 'type' and a 'mixer' object")
            kind, m, mw = entry.get("type"), entry["mixer"], f"{where}.mixer"
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type is {kind!r}; known mixers: {MIXERS}")
            if kind == "latent_attention":
                heads, dim, rot_dim, vdim, kv_rank, q_rank = sizes(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), mw)
                r = obj(m, "rot", f"{mw}.rot")
                base, dims = need(r, "base", float, f"{mw}.rot"), need(r, "dims", int, f"{mw}.rot")
                if dims != rot_dim or dims % 2 or not base > 1.0:
                    raise ConfigError(f"config.json: {mw}.rot.dims must be even and equal rot_dim, base above 1")
                sc, scaling = obj(r, "scaling", f"{mw}.rot.scaling", required=False), None
                if sc:
                    scaling = tuple(need(sc, k, float, f"{mw}.rot.scaling") for k in ("factor", "original", "fast", "slow"))
                    if min(scaling) <= 0:
                        raise ConfigError(f"config.json: {mw}.rot.scaling values must be positive")
                mask, window = obj(m, "mask", f"{mw}.mask", required=False), None
                if mask:
                    (window,) = sizes(mask, ("size",), f"{mw}.mask")
                scale = get_key(m, "scale", float)
                mixer = BezasunLatent(heads, dim, rot_dim, vdim, kv_rank, q_rank,
                                      (dim + rot_dim) ** -0.5 if scale is None else scale,
                                      BezasunRotation(base, dims, scaling), window)
            elif kind == "mamba2":
                heads, vdim, state, groups, conv, parts = sizes(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), mw)
                if heads % groups or (heads * vdim) % parts:
                    raise ConfigError(f"config.json: {mw}: heads must be a multiple of groups, heads * vdim of norm_groups")
                mixer = BezasunMamba(heads, vdim, state, groups, conv, parts)
            else:
                heads, kv_heads, dim, vdim = sizes(m, ("heads", "kv_heads", "dim", "vdim"), mw)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {mw}: heads must be a multiple of kv_heads")
                scale, softcap = get_key(m, "scale", float), get_key(m, "softcap", float)
                if softcap is not None and not softcap > 0:
                    raise ConfigError(f"config.json: {mw}.softcap must be positive")
                qt, q_temp = obj(m, "q_temp", f"{mw}.q_temp", required=False), None
                if qt:
                    q_temp = (need(qt, "coef", float, f"{mw}.q_temp"), need(qt, "every", float, f"{mw}.q_temp"))
                    if not q_temp[1] > 0:
                        raise ConfigError(f"config.json: {mw}.q_temp.every must be positive")
                mixer = BezasunAttention(heads, kv_heads, dim, vdim, dim ** -0.5 if scale is None else scale, softcap, q_temp)
            mlp_raw, mlp = entry.get("mlp"), None
            if mlp_raw is not None:
                lw = f"{where}.mlp"
                if not isinstance(mlp_raw, dict) or mlp_raw.get("kind", "moe") != "moe":
                    raise ConfigError(f"config.json: {lw}.kind must be 'moe' (or mlp null)")
                experts, top = sizes(obj(mlp_raw, "router", f"{lw}.router"), ("experts", "top"), f"{lw}.router")
                (ff,) = sizes(obj(mlp_raw, "expert", f"{lw}.expert"), ("ff",), f"{lw}.expert")
                if top > experts:
                    raise ConfigError(f"config.json: {lw}.router.top is larger than the number of experts")
                shared_raw, shared_ff = obj(mlp_raw, "shared", f"{lw}.shared", required=False), None
                if shared_raw:
                    (shared_ff,) = sizes(shared_raw, ("ff",), f"{lw}.shared")
                mlp = BezasunMoe(experts, top, ff, shared_ff)
            layers.append(BezasunLayer(kind, mixer, mlp))
        eos = token_ids(raw, "eos_token_id") or (token_ids(generation, "eos_token_id") if generation else [])
        return BezasunConfig(vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                             embedding_scale=number(obj(raw, "embedding", "embedding", required=False), "scale", "embedding", 1.0),
                             logit_scale=number(raw, "logit_scale", "", 1.0),
                             residual_mult=number(raw, "residual_mult", "", 1.0), streams=streams,
                             eos_token_ids=tuple(eos))
