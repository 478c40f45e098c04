"""Typed configuration of the Surinex decoder: layers whose mixer and feed-forward sit side by side on one
norm's output (each behind its own short causal convolution of it), three kinds of mixer, and a range of
layers that runs several times with the same weights.

config.json keys: ``architecture`` ("Surinex"), ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (taps of
the convolutions in front of the sub-layers), optionally ``loop`` = ``{start, stop, times}`` (layers
start .. stop-1 run ``times`` times in a row), and ``layers``: a list of
``{"type": "gla" | "latent_attention" | "parallel", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}``.

Mixer keys.
  gla               ``heads, dim, vdim, tau``; the inner size of the decay's low-rank map is not in config.json:
                    the checkpoint's ``l<i>.mix.a1`` [rank, width] gives it (:func:`sizes_from_tensors`); a
                    configuration without a checkpoint may name it ``decay_rank`` and otherwise gets 16.
  latent_attention  ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot.base`` (``rot.dims`` = ``rot_dim``)
  parallel          ``left``: ``heads, kv_heads, dim, vdim, scale, rot`` = ``{base, dims, scaling?}`` with
                    ``scaling`` = ``{factor, low, high, original}``; ``right``: ``heads, kv_heads, dim, vdim, conv``
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, get_key, token_ids

MIXERS = ("gla", "latent_attention", "parallel")


@dataclass(frozen=True)
class SurinexRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original


@dataclass(frozen=True)
class SurinexGla:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: Optional[int] = None


@dataclass(frozen=True)
class SurinexLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: SurinexRotation


@dataclass(frozen=True)
class SurinexLeft:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: SurinexRotation


@dataclass(frozen=True)
class SurinexRight:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class SurinexLayer:
    kind: str
    mixer: Any                        # SurinexGla | SurinexLatent | (SurinexLeft, SurinexRight)
    ff: Optional[int]                 # None: the layer has no feed-forward


@dataclass(frozen=True)
class SurinexLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class SurinexConfig:
    vocab: int
    width: int
    eps: float
    taps: int
    layers: Tuple[SurinexLayer, ...]
    loop: Optional[SurinexLoop] = None
    eos_token_ids: Tuple[int, ...] = ()
    architectures: Tuple[str, ...] = ("Surinex",)

    @staticmethod
    def from_json(raw: Dict[str, Any], generation: Optional[Dict[str, Any]] = None) -> "SurinexConfig":
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

        def rotation(parent, where, head_dim, required=True):
            r = obj(parent, "rot", f"{where}.rot", required=required)
            if r is None:
                return None
            rw = f"{where}.rot"
            base, dims = need(r, "base", float, rw), need(r, "dims", int, rw)
            if dims <= 0 or dims % 2 or dims > head_dim or not base > 1.0:
                raise ConfigError(f"config.json: {rw}.dims must be even and at most the head's size, base above 1")
            sc, scaling = obj(r, "scaling", f"{rw}.scaling", required=False), None
            if sc:
                scaling = tuple(need(sc, k, float, f"{rw}.scaling") for k in ("factor", "low", "high", "original"))
                if min(scaling) <= 0 or scaling[2] == scaling[1]:
                    raise ConfigError(f"config.json: {rw}.scaling values must be positive, high other than low")
            return SurinexRotation(base=base, dims=dims, scaling=scaling)

        vocab = get_key(raw, "vocab", int, required=True)
        width = get_key(raw, "width", int, required=True)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        eps = need(obj(raw, "norm", "norm"), "eps", float, "norm")
        taps = need(obj(raw, "canon", "canon"), "taps", int, "canon")
        if taps < 1:
            raise ConfigError("config.json: 'canon.taps' must be at least 1")
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
            mlp, ff = entry.get("mlp"), None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null)")
                (ff,) = sizes(mlp, ("ff",), f"{where}.mlp")
            if kind == "gla":
                heads, dim, vdim = sizes(m, ("heads", "dim", "vdim"), mw)
                tau = need(m, "tau", float, mw)
                if not tau > 0:
                    raise ConfigError(f"config.json: {mw}.tau must be positive")
                mixer = SurinexGla(heads, dim, vdim, tau, decay_rank=get_key(m, "decay_rank", int))
            elif kind == "latent_attention":
                heads, dim, rot_dim, vdim, kv_rank, q_rank = sizes(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), mw)
                rot = rotation(m, mw, rot_dim)
                if rot.dims != rot_dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims must equal rot_dim (the whole rotated part turns)")
                scale = get_key(m, "scale", float)
                mixer = SurinexLatent(heads, dim, rot_dim, vdim, kv_rank, q_rank,
                                      (dim + rot_dim) ** -0.5 if scale is None else scale, rot)
            else:
                left, right = obj(m, "left", f"{mw}.left"), obj(m, "right", f"{mw}.right")
                lh, lg, ld, lv = sizes(left, ("heads", "kv_heads", "dim", "vdim"), f"{mw}.left")
                rh, rg, rd, rv, conv = sizes(right, ("heads", "kv_heads", "dim", "vdim", "conv"), f"{mw}.right")
                if lh % lg or rh % rg:
                    raise ConfigError(f"config.json: {mw}: heads must be a multiple of kv_heads")
                if lv % 2:
                    raise ConfigError(f"config.json: {mw}.left.vdim must be even (its values rotate in pairs)")
                scale = get_key(left, "scale", float)
                mixer = (SurinexLeft(lh, lg, ld, lv, ld ** -0.5 if scale is None else scale,
                                     rotation(left, f"{mw}.left", ld)),
                         SurinexRight(rh, rg, rd, rv, conv))
            layers.append(SurinexLayer(kind, mixer, ff))
        loop_raw, loop = obj(raw, "loop", "loop", required=False), None
        if loop_raw:
            start, stop, times = (need(loop_raw, k, int, "loop") for k in ("start", "stop", "times"))
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise ConfigError(f"config.json: loop needs 0 <= start <= stop <= {len(layers)} layers and times >= 1")
            if start < stop:
                loop = SurinexLoop(start, stop, times)
        eos = token_ids(raw, "eos_token_id") or (token_ids(generation, "eos_token_id") if generation else [])
        return SurinexConfig(vocab=vocab, width=width, eps=eps, taps=taps, layers=tuple(layers), loop=loop,
                             eos_token_ids=tuple(eos))


def sizes_from_tensors(cfg: SurinexConfig, shapes: Dict[str, tuple]) -> SurinexConfig:
    """The size that only the checkpoint gives: the inner size of each gla mixer's low-rank decay map, read off
    ``l<i>.mix.a1`` ([rank, width])."""
    layers = list(cfg.layers)
    for i, layer in enumerate(layers):
        a1 = shapes.get(f"l{i}.mix.a1")
        if layer.kind == "gla" and a1:
            layers[i] = replace(layer, mixer=replace(layer.mixer, decay_rank=int(a1[0])))
    return replace(cfg, layers=tuple(layers))
