"""Norm, position encoding, embedding, output head and the block arrangement."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np
import torch

from ..kernels import ops
from .context import GatedPending, HyperPending, Pending
from .linear import linear
from .registry import BuildEnv, build, register
from .spec import PartSpec, TensorSpec


class Part:
    """Common shape of a part: parameters in, tensors by name, nothing model-specific.

    ``graph_safe``: the part's forward only enqueues work whose shape depends on the number of
    tokens and reads the step's device tensors, never its host-side lists; a decode step made of
    such parts may be captured in a CUDA graph. A part that does not say so is never captured."""

    graph_safe = False

    def __init__(self, params: dict, prefix: str, env: BuildEnv):
        self.params, self.prefix, self.env = params, prefix, env

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, fetch) -> None:
        """``fetch(name)`` returns the named tensor on the device (or None if optional and absent)."""

    def cache_spec(self):
        return None

    def state_size(self) -> int:
        """Block arrangements: float32 numbers the block keeps per request and cache slot (0: none)."""
        return 0


# --------------------------------------------------------------------------- norms
@register("norm", "rmsnorm")
class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * w, statistics in float32
    (crates/hi-mlx/src/models.rs:1977-1979; crates/hi-cuda/src/kernels.cu:61-77).
    params: ``size``, ``eps``, ``name`` (tensor ``<prefix>.weight``; with ``tensor`` = "bare" the tensor
    is ``<prefix>`` itself), ``one_plus`` (the tensor is stored around zero and acts as 1 + w; the sum is
    taken in float32 and kept so).

    Where the block keeps its residual stream as several copies (:class:`~hi_b200.parts.context.HyperPending`)
    the norm reads the plain sum of the copies."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.one_plus = bool(params.get("one_plus", False))
        self.weight: Optional[torch.Tensor] = None
        self.tensor_name = prefix if params.get("tensor") == "bare" else f"{prefix}.weight"

    def tensor_specs(self):
        return [TensorSpec(self.tensor_name, (self.size,), init="zeros" if self.one_plus else "ones")]

    def load(self, fetch):
        w = fetch(self.tensor_name)
        self.weight = (w.to(torch.float32) + 1.0).contiguous() if self.one_plus else w.contiguous()

    def forward(self, residual: torch.Tensor, delta, row_map: Optional[torch.Tensor] = None, also_f32: bool = False,
                out_dtype: Optional[torch.dtype] = None):
        """``delta``: None, a tensor, or a :class:`~hi_b200.parts.context.Pending`. ``out_dtype``: the engine's
        dtype, or float32 for a consumer that goes on in 32-bit."""
        out_dtype = out_dtype or self.env.dtype
        if isinstance(delta, HyperPending):
            return resolve_hyper(residual, delta, self.weight, self.eps, out_dtype, None, row_map, also_f32)
        if isinstance(delta, Pending):
            if delta.top_k > 8:
                delta = delta.materialize(residual.shape[0])
            else:
                return ops.add_rmsnorm(residual, delta.dense, self.weight, self.eps, out_dtype, row_map, also_f32,
                                       delta.routed, delta.slot_of_entry, delta.top_k, delta.entry_weights,
                                       delta2=delta.dense2)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype, row_map, also_f32)


@register("norm", "dynamic_tanh")
class DynamicTanh(Part):
    """y = tanh(alpha x) * w + b: a norm that takes no mean or variance; alpha is one learned number.
    params: ``size``, ``name``; tensors ``<prefix>`` (w), ``<prefix>.b``, ``<prefix>.alpha`` (a scalar).
    alpha and the arithmetic are float32.

    ``forward`` takes what the other norms take as ``delta`` (None, a tensor or a ``Pending``: added
    into the stream in place) and also a :class:`~hi_b200.parts.context.GatedPending`, whose sum and
    average give a NEW stream tensor; that form returns ``(stream, y)`` from :meth:`resolve`."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix, (self.size,), init="ones"),
                TensorSpec(f"{self.prefix}.b", (self.size,), init="normal"),
                TensorSpec(f"{self.prefix}.alpha", (), init="ones")]

    def load(self, fetch):
        self.weight = fetch(self.prefix).contiguous()
        self.bias = fetch(f"{self.prefix}.b").to(self.weight.dtype).contiguous()
        self.alpha = fetch(f"{self.prefix}.alpha").to(torch.float32).reshape(1).contiguous()

    def triple(self):
        return (self.alpha, self.weight, self.bias)

    @staticmethod
    def resolve(residual, pending, norms, out_dtype, row_map=None, want_stream=True):
        """The stream after ``pending`` and the outputs of up to two norms of it, in one kernel:
        ``(stream | None, [y])``. Without a ``GatedPending`` the stream is ``residual`` itself."""
        triples = [n.triple() for n in norms]
        if isinstance(pending, GatedPending):
            z, ys = ops.gated_depth_dyt(residual, pending.terms, pending.history, pending.filled, pending.mix,
                                        triples, out_dtype, row_map, want_z=want_stream)
            return z, ys
        if isinstance(pending, Pending):
            pending = pending.materialize(residual.shape[0])
        terms = [] if pending is None else [(pending, None)]
        # a plain sum goes into the stream in place, as with the other norms
        z, ys = ops.gated_depth_dyt(residual, terms, None, 0, None, triples, out_dtype, row_map,
                                    want_z=bool(terms) and row_map is None)
        if z is not None:
            residual.copy_(z)
        return residual, ys

    @staticmethod
    def open_history(residual, history, norms, out_dtype):
        """The norms of the stream that enters the first layer, which the same kernel stores as
        result 0 of ``history``."""
        _z, ys = ops.gated_depth_dyt(residual, [], history, 0, None, [n.triple() for n in norms], out_dtype,
                                     want_z=False)
        return ys

    def forward(self, residual: torch.Tensor, delta, row_map: Optional[torch.Tensor] = None, also_f32: bool = False):
        _stream, ys = self.resolve(residual, delta, [self], self.env.dtype, row_map, want_stream=False)
        if also_f32:
            return ys[0], ys[0].to(torch.float32)
        return ys[0]


# --------------------------------------------------------------------------- positions
def llama3_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> np.ndarray:
    """inv_freq[j] = theta^(-2j/hd), rescaled by parts when ``scaling`` is given
    (crates/hi-mlx/src/models.rs:5897-5926, 6166-6175), all in float32 as there. Where the
    reference would divide 0 by 0 (high == low and the wavelength exactly on the boundary)
    the low-frequency value is taken."""
    f32 = np.float32
    out = np.empty(head_dim // 2, dtype=f32)
    for j in range(head_dim // 2):
        th = np.power(f32(theta), f32((2 * j) / head_dim), dtype=f32)
        inv = f32(1.0) / th
        if scaling:
            factor, low = f32(scaling["factor"]), f32(scaling["low_freq_factor"])
            high, orig = f32(scaling["high_freq_factor"]), f32(scaling["original_max_position_embeddings"])
            wavelen = f32(2.0) * f32(math.pi) / inv
            if wavelen > orig / low:
                inv = inv / factor
            elif wavelen < orig / high:
                pass
            else:
                smooth = f32(0.0) if high == low else (orig / wavelen - low) / (high - low)
                inv = (f32(1.0) - smooth) * inv / factor + smooth * inv
        out[j] = inv
    return out


def exact_inverse_frequencies(dims: int, theta: float, scaling: Optional[dict]) -> np.ndarray:
    """The table of :func:`llama3_inverse_frequencies` (same keys of ``scaling``) worked out in float64 and
    rounded to float32 once."""
    out = np.empty(dims // 2, dtype=np.float64)
    for j in range(dims // 2):
        inv = float(theta) ** (-2.0 * j / dims)
        if scaling:
            factor, low = float(scaling["factor"]), float(scaling["low_freq_factor"])
            high, orig = float(scaling["high_freq_factor"]), float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / inv
            if wavelen > orig / low:
                inv = inv / factor
            elif wavelen >= orig / high:
                smooth = 0.0 if high == low else (orig / wavelen - low) / (high - low)
                inv = (1.0 - smooth) * inv / factor + smooth * inv
        out[j] = inv
    return out.astype(np.float32)


@register("position", "rope")
class RotaryPosition(Part):
    """Rotary encoding of q and k: all head_dim dims, or with ``rot_dim`` the first rot_dim of them
    (an even number; the rest pass through; whole lanes of 16 dims take the faster encoding kernel).
    params: ``head_dim``, ``theta``, ``scaling`` (dict or None), ``interleaved`` (pairs (2j, 2j+1)
    instead of (j, j + rot_dim/2)), ``rot_dim`` (default head_dim; the frequencies are
    theta^(-2j/rot_dim)), ``exact`` (the table is worked out in float64 and rounded once, instead of in
    float32 step by step as the reference does)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.interleaved = bool(params.get("interleaved", False))
        self.rot_dim = int(params.get("rot_dim") or params["head_dim"])
        if self.rot_dim % 2 or not 0 < self.rot_dim <= int(params["head_dim"]):
            raise ValueError(f"{prefix}: rot_dim {self.rot_dim} must be even, at most head_dim")
        if params.get("exact"):
            self._table_host = exact_inverse_frequencies(self.rot_dim, float(params["theta"]), params.get("scaling"))
        else:
            self._table_host = llama3_inverse_frequencies(self.rot_dim, float(params["theta"]), params.get("scaling"))
        self._table: Optional[torch.Tensor] = None

    def rotary_table(self):
        if self._table is None:
            self._table = torch.from_numpy(self._table_host).to(self.env.device)
        return self._table, self.interleaved


def yarn_inverse_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency of each of the dims / 2 pairs as float32, factor on cos and sin).

    Pair i turns by base^(-2i/dims) per position. With ``scaling`` = {factor, original, fast, slow} the
    pairs that turn fewer than ``slow`` times over ``original`` positions are slowed by ``factor``, those
    that turn more than ``fast`` times stay, and a linear ramp over the pair index lies between:
    with i(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(i(fast)), 0),
    hi = min(ceil(i(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the
    frequency is f_i / factor * ramp_i + f_i (1 - ramp_i); cos and sin grow by 0.1 ln(factor) + 1.
    Worked out in float64, handed on in float32."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return f.astype(np.float32), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32), 0.1 * math.log(factor) + 1.0


@register("position", "rope_yarn")
class YarnRotaryPosition(Part):
    """Rotary encoding of the first ``dims`` dims of a head (any even number; the rest pass through),
    pairs (i, i + dims/2), with the ramped frequency scaling of :func:`yarn_inverse_frequencies` and its
    factor on cos and sin (``magnitude``, which the encoding kernel takes as a multiplier).
    params: ``head_dim``, ``dims``, ``base``, ``scaling`` ({factor, original, fast, slow} or None)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.dims = int(params["dims"])
        if self.dims % 2 or not 0 < self.dims <= int(params["head_dim"]):
            raise ValueError(f"{prefix}: {self.dims} rotating dims must be even and at most head_dim")
        self._table_host, self.magnitude = yarn_inverse_frequencies(self.dims, float(params["base"]), params.get("scaling"))
        self._table: Optional[torch.Tensor] = None

    def rotary_table(self):
        if self._table is None:
            self._table = torch.from_numpy(self._table_host).to(self.env.device)
        return self._table, False


@register("position", "none")
class NoPosition(Part):
    """NoPE: q and k are used as projected."""

    graph_safe = True

    def rotary_table(self):
        return None


# --------------------------------------------------------------------------- embedding and head
@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """x[t] = table[token[t]] * scale; no multiplier by default (crates/hi-mlx/src/models.rs:6206, 1915-1917).
    params: ``vocab_size``, ``hidden_size``, ``scale`` (default 1); tensor ``<prefix>.weight``."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.table: Optional[torch.Tensor] = None
        self.scale = float(params.get("scale", 1.0))

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.weight", (int(self.params["vocab_size"]), int(self.params["hidden_size"])))]

    def load(self, fetch):
        self.table = fetch(f"{self.prefix}.weight").contiguous()

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return ops.embed_gather(self.table, tokens, scale=self.scale)


@register("head", "linear_head")
class LinearHead(Part):
    """logits = z W^T in float32. The separate head is used when its tensor exists, else the
    embedding table (decided by presence, crates/hi-mlx/src/models.rs:6186-6193, 6211-6214).
    params: ``vocab_size``, ``hidden_size``, ``tie`` (random weights: write no head tensor),
    ``softcap`` (None, or c: logits <- c tanh(logits / c)), ``scale`` (a factor on the logits, default 1),
    ``tensor`` (the head tensor's whole name; default ``<prefix>.weight``)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.weight: Optional[torch.Tensor] = None
        self.tied = False
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        self.scale = float(params.get("scale", 1.0))
        self.tensor_name = params.get("tensor") or f"{prefix}.weight"

    def tensor_specs(self):
        # "absent": the random-weights writer leaves a tied head out of the folder
        return [TensorSpec(self.tensor_name, (int(self.params["vocab_size"]), int(self.params["hidden_size"])),
                           init="absent" if self.params.get("tie", False) else "normal", optional=True)]

    def load(self, fetch):
        w = fetch(self.tensor_name)
        self.tied = w is None
        self.weight = None if w is None else w.contiguous()

    def forward(self, normed_rows: torch.Tensor, embedding: TokenEmbedding) -> torch.Tensor:
        w = embedding.table if self.weight is None else self.weight
        logits = linear(normed_rows, w, out_dtype=torch.float32)
        if self.scale != 1.0:
            logits.mul_(self.scale)
        return logits if self.softcap is None else ops.softcap_(logits.contiguous(), self.softcap)


# --------------------------------------------------------------------------- block arrangement
@register("arrangement", "prenorm")
class PreNormBlock(Part):
    """h = x + mixer(norm(x)); y = h + ffn(norm(h))  (crates/hi-mlx/src/models.rs:6143-6149).

    The residual stream is float32. A sub-layer's output is carried as ``pending`` and added
    inside the next norm kernel, so each residual sum is one fused read-modify-write.
    """

    graph_safe = True

    def forward(self, layer, residual, pending, ctx, cache_view):
        h = layer.norm_mixer.forward(residual, pending)
        pending = layer.mixer.forward(h, ctx, cache_view)
        if getattr(layer.feed_forward, "wants_f32_input", False):
            h, h32 = layer.norm_feed_forward.forward(residual, pending, also_f32=True)
            pending = layer.feed_forward.forward(h, ctx, normed_f32=h32)
        else:
            h = layer.norm_feed_forward.forward(residual, pending)
            pending = layer.feed_forward.forward(h, ctx)
        return residual, pending


@register("arrangement", "postnorm")
class PostNormBlock(Part):
    """The norm comes after the sum: x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)).

    The sub-layers read the stream itself (its rounding to the engine's dtype, which the norm kernel
    writes beside the float32 stream). Each boundary is one kernel: the scaled stream, the sub-layer's
    output and the routed experts' rows are summed in float32, normalised, and written back as the
    stream. The first layer's mixer reads the embedding output, which no norm has touched: it is
    rounded here. A layer without feed-forward has the first half only.

    params: ``alpha`` (default 1)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.alpha = float(params.get("alpha", 1.0))

    def _boundary(self, norm, residual, delta):
        """stream <- norm(alpha * stream + delta); returns the stream in the engine's dtype."""
        if isinstance(delta, Pending):
            if delta.routed is None:
                delta = delta.dense
            elif delta.top_k > 8:
                delta = delta.materialize(residual.shape[0])
        if isinstance(delta, Pending):
            return ops.add_rmsnorm(residual, delta.dense, norm.weight, norm.eps, self.env.dtype, None, False,
                                   delta.routed, delta.slot_of_entry, delta.top_k, delta.entry_weights,
                                   x_scale=self.alpha, post=True)
        return ops.add_rmsnorm(residual, delta, norm.weight, norm.eps, self.env.dtype, x_scale=self.alpha, post=True)

    def forward(self, layer, residual, pending, ctx, cache_view):
        if not isinstance(layer.norm_mixer, RMSNorm):
            raise TypeError(f"{self.prefix}: the post-norm block works with rmsnorm norms")
        if pending is not None:
            raise TypeError(f"{self.prefix}: a post-norm block cannot follow a block that leaves a sum open")
        # the stream in the engine's dtype, as the block before this one left it
        owner, h = ctx.scratch.get("postnorm_stream", (None, None))
        if owner is not residual:
            h = residual if residual.dtype == self.env.dtype else ops.convert(residual, self.env.dtype)
        y = layer.mixer.forward(h, ctx, cache_view)
        h = self._boundary(layer.norm_mixer, residual, y)
        if layer.feed_forward is not None:
            if getattr(layer.feed_forward, "wants_f32_input", False):
                y = layer.feed_forward.forward(h, ctx, normed_f32=residual)
            else:
                y = layer.feed_forward.forward(h, ctx)
            h = self._boundary(layer.norm_feed_forward, residual, y)
        ctx.scratch["postnorm_stream"] = (residual, h)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.stream_out", residual)
        return residual, None


_side_streams: Dict[torch.device, "torch.cuda.Stream"] = {}


def _side_stream(device) -> "torch.cuda.Stream":
    """One second stream per device for branches that run beside the main one."""
    device = torch.device(device)
    if device not in _side_streams:
        _side_streams[device] = torch.cuda.Stream(device=device)
    return _side_streams[device]


@register("arrangement", "parallel_gated")
class ParallelGatedBlock(Part):
    """Mixer and feed-forward side by side on the same input, each result gated element by element,
    and optionally a weighted average over depth:

        h1 = norm1(x), h2 = norm2(x)
        X_next = x + sigmoid(W1 h1 + c1) * mixer(h1) + sigmoid(W2 h2 + c2) * ff(h2)
        x <- sum_j mix[j] X_j          (X_0 the embedding output, X_j the result of layer j - 1)

    The sums, the average and both norms of the NEXT layer run in one kernel at the layer boundary
    (``ops.gated_depth_dyt``): the block returns its results as a
    :class:`~hi_b200.parts.context.GatedPending`, as the pre-norm block returns its ``Pending``.

    params: ``hidden_size``; ``gated`` (default True); ``depth_average`` (default False): with it the
    layer has ``<prefix>.dwa`` with one weight per result so far, this layer's included.
    tensors: ``<prefix>.rg1`` [W, W], ``<prefix>.rg1.b`` [W] (and ``rg2`` when the layer has a
    feed-forward); ``<prefix>.dwa``. The norms must be ``dynamic_tanh``."""

    graph_safe = True
    OVERLAP_BRANCHES = True      # steps of few tokens: the feed-forward branch on a second stream beside the mixer
    OVERLAP_MAX_TOKENS = 128

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.width = int(params["hidden_size"])
        self.gated = bool(params.get("gated", True))
        self.depth = bool(params.get("depth_average", False))
        self.results_before = int(params.get("results_before", 0))     # entries of the history when the layer starts
        self.total_results = int(params.get("total_results", 0))
        self.has_ff = bool(params.get("feed_forward", True))
        self.w_g = [None, None]
        self.b_g = [None, None]
        self.mix: Optional[torch.Tensor] = None

    def _gates(self):
        return ("rg1", "rg2") if self.has_ff else ("rg1",)

    def tensor_specs(self):
        specs = []
        if self.gated:
            for g in self._gates():
                specs += [TensorSpec(f"{self.prefix}.{g}", (self.width, self.width)),
                          TensorSpec(f"{self.prefix}.{g}.b", (self.width,))]
        if self.depth:
            specs.append(TensorSpec(f"{self.prefix}.dwa", (self.results_before + 1,)))
        return specs

    def load(self, fetch):
        if self.gated:
            for i, g in enumerate(self._gates()):
                self.w_g[i] = fetch(f"{self.prefix}.{g}").contiguous()
                self.b_g[i] = fetch(f"{self.prefix}.{g}.b").to(self.w_g[i].dtype).contiguous()
        if self.depth:
            self.mix = fetch(f"{self.prefix}.dwa").to(torch.float32).contiguous()

    def _feed_forward_term(self, layer, h2, ctx):
        f = layer.feed_forward.forward(h2, ctx)
        if isinstance(f, Pending):
            f = f.materialize(h2.shape[0])
        return (f, linear(h2, self.w_g[1], bias=self.b_g[1]) if self.gated else None)

    def forward(self, layer, residual, pending, ctx, cache_view):
        norms = [layer.norm_mixer] + ([layer.norm_feed_forward] if self.has_ff else [])
        if not all(isinstance(n, DynamicTanh) for n in norms):
            raise TypeError(f"{self.prefix}: the parallel gated block works with dynamic_tanh norms")
        history = ctx.scratch.get("depth_history") if self.depth else None
        if self.depth and history is None:
            # the stream that enters the first layer (the embedding output) is result 0
            if self.results_before != 1:
                raise RuntimeError(f"{self.prefix}: the depth average has no results of earlier layers to read")
            history = torch.empty((self.total_results, *residual.shape), dtype=torch.float32, device=residual.device)
            ctx.scratch["depth_history"] = history
            if pending is not None:
                residual, _ = DynamicTanh.resolve(residual, pending, [], self.env.dtype)
            x, ys = residual, DynamicTanh.open_history(residual, history, norms, self.env.dtype)
        else:
            x, ys = DynamicTanh.resolve(residual, pending, norms, self.env.dtype)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.stream_in", x)        # debug: the stream as this layer reads it
        h1 = ys[0]
        second, gate1, side = None, None, None
        if self.has_ff and self.OVERLAP_BRANCHES and h1.shape[0] <= self.OVERLAP_MAX_TOKENS:
            # The two branches share nothing but their input. In a step of few tokens neither fills the GPU
            # and the step is a chain of short kernels: the feed-forward branch and the mixer's gate run on a
            # second stream beside the mixer (in a captured step: a parallel branch of the graph) and join
            # before the boundary kernel.
            cur, side = torch.cuda.current_stream(), _side_stream(h1.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                second = self._feed_forward_term(layer, ys[1], ctx)
                gate1 = linear(h1, self.w_g[0], bias=self.b_g[0]) if self.gated else None
            for t in ys:
                t.record_stream(side)
            for t in (*second, gate1):
                if t is not None:
                    t.record_stream(cur)
        elif self.gated:
            gate1 = linear(h1, self.w_g[0], bias=self.b_g[0])
        terms = [(layer.mixer.forward(h1, ctx, cache_view), gate1)]
        if self.has_ff:
            terms.append(second if second is not None else self._feed_forward_term(layer, ys[1], ctx))
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return x, GatedPending(terms=terms, history=history, filled=self.results_before, mix=self.mix)


@register("arrangement", "parallel_conv")
class ParallelConvBlock(Part):
    """One norm; the mixer and the feed-forward both read its output, each through its own short causal
    convolution over time, and their sum joins the stream:

        h = norm1(x)
        h_a = h + conv_a(h),  h_b = h + conv_b(h)      conv(h)[t] = sum_j taps[:, j] * h[t - (K-1) + j]
        x <- x + mixer(h_a) + ff(h_b)

    h stays float32 between the norm and the convolutions (one kernel for both, ``ops.canon_conv``); the two
    results are carried as a ``Pending`` with two dense parts and summed into the stream by the next norm.
    Per request and cache slot the block keeps the last K-1 rows of h (float32), zero at a sequence's start:
    ``state_size``. A layer without feed-forward has the first branch only.

    params: ``hidden_size``, ``taps`` (K >= 1), ``feed_forward`` (default True).
    tensors: ``<prefix>.canon1`` [W, K] (mixer), ``<prefix>.canon2`` [W, K] (feed-forward). The norm must be ``rmsnorm``."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.width, self.taps = int(params["hidden_size"]), int(params["taps"])
        if self.taps < 1:
            raise ValueError(f"{prefix}: a convolution has at least one tap, not {self.taps}")
        self.has_ff = bool(params.get("feed_forward", True))
        self.taps_a = self.taps_b = self._no_state = None

    def state_size(self) -> int:
        return (self.taps - 1) * self.width

    def tensor_specs(self):
        names = ("canon1", "canon2") if self.has_ff else ("canon1",)
        return [TensorSpec(f"{self.prefix}.{n}", (self.width, self.taps)) for n in names]

    def load(self, fetch):
        self.taps_a = fetch(f"{self.prefix}.canon1").to(torch.float32).contiguous()
        if self.has_ff:
            self.taps_b = fetch(f"{self.prefix}.canon2").to(torch.float32).contiguous()
        self._no_state = torch.zeros((1, 1), dtype=torch.float32, device=self.taps_a.device)

    def forward(self, layer, residual, pending, ctx, cache_view):
        norm = layer.norm_mixer
        if not isinstance(norm, RMSNorm):
            raise TypeError(f"{self.prefix}: the block works with an rmsnorm norm")
        h = norm.forward(residual, pending, out_dtype=torch.float32)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.stream_in", residual)        # debug: the stream as this layer reads it
        state = cache_view.block_state if self.taps > 1 else self._no_state
        if state is None:
            raise RuntimeError(f"{self.prefix}: the block has no state rows for its convolutions")
        h_a, h_b = ops.canon_conv(h, self.taps_a, self.taps_b, state, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots,
                                  self.env.dtype, single_tokens=ctx.max_new == 1)
        delta = layer.mixer.forward(h_a, ctx, cache_view)
        if not self.has_ff:
            return residual, Pending(dense=delta)
        second = layer.feed_forward.forward(h_b, ctx)
        if isinstance(second, Pending):
            second = second.materialize(h_b.shape[0])
        return residual, Pending(dense=delta, dense2=second)


def resolve_hyper(streams, pending, weight, eps, out_dtype, in_coef, row_map=None, also_f32=False):
    """One boundary of a residual stream of several copies (``ops.hyper_step``): what ``pending`` (a
    :class:`~hi_b200.parts.context.HyperPending` or None) holds enters the copies, and the weighted sum of the copies
    (``in_coef``; None: the plain sum) is normed with ``weight``."""
    if pending is None:
        return ops.hyper_step(streams, weight, eps, out_dtype, in_coef=in_coef, row_map=row_map, also_f32=also_f32)
    d = pending.delta
    if isinstance(d, Pending):
        return ops.hyper_step(streams, weight, eps, out_dtype, delta=d.dense, delta2=d.dense2, routed=d.routed,
                              slot_of_entry=d.slot_of_entry, top_k=d.top_k, routed_weight=d.entry_weights,
                              mix=pending.mix, out_coef=pending.out_coef, mult=pending.mult, in_coef=in_coef,
                              row_map=row_map, also_f32=also_f32)
    return ops.hyper_step(streams, weight, eps, out_dtype, delta=d, mix=pending.mix, out_coef=pending.out_coef,
                          mult=pending.mult, in_coef=in_coef, row_map=row_map, also_f32=also_f32)


@register("arrangement", "hyper_connections")
class HyperConnectionBlock(Part):
    """A pre-norm block whose residual stream is S copies x_1 .. x_S per token (all equal to the embedding output
    before the first layer). Sub-layer q (1: mixer, 2: feed-forward) reads one weighted sum of the copies and its
    result goes back into every copy while the copies are mixed among themselves:

        u = sum_s in_q[s] x_s;   y = sublayer_q(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + mult * out_q[t] * y

    for all t at once, from the old copies. Whoever reads the stream after the last layer takes the plain sum of
    the copies. The copies are float32 [N, S, W]; every boundary between two sub-layers is one kernel
    (``ops.hyper_step``): the update with the result the sub-layer before left, the next sub-layer's weighted sum and
    its norm. The block hands the copies on as the stream with its last result as a
    :class:`~hi_b200.parts.context.HyperPending`, as the pre-norm block hands on a ``Pending``.

    params: ``hidden_size``, ``streams`` (S >= 1), ``mult`` (default 1), ``feed_forward`` (default True),
    ``learned`` (default True; False: one copy, in = out = mix = 1: x <- x + mult * y, no tensors).
    tensors: ``<prefix>.hc<q>.in`` [S], ``<prefix>.hc<q>.out`` [S], ``<prefix>.hc<q>.mix`` [S, S] ([from, to]).
    The norms must be ``rmsnorm``."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.width, self.copies = int(params["hidden_size"]), int(params.get("streams", 1))
        self.mult = float(params.get("mult", 1.0))
        self.has_ff = bool(params.get("feed_forward", True))
        self.learned = bool(params.get("learned", True))
        if self.copies < 1 or self.copies > 16 or (not self.learned and self.copies != 1):
            raise ValueError(f"{prefix}: {self.copies} copies of the stream are not supported (1 to 16; without "
                             f"learned coefficients one)")
        self.coef = {}

    def _sublayers(self):
        return (1, 2) if self.has_ff else (1,)

    def tensor_specs(self):
        if not self.learned:
            return []
        s, specs = self.copies, []
        for q in self._sublayers():
            specs += [TensorSpec(f"{self.prefix}.hc{q}.in", (s,), init="ones"),
                      TensorSpec(f"{self.prefix}.hc{q}.out", (s,), init="ones"),
                      TensorSpec(f"{self.prefix}.hc{q}.mix", (s, s))]
        return specs

    def load(self, fetch):
        f32 = torch.float32
        for q in self._sublayers():
            if self.learned:
                self.coef[q] = tuple(fetch(f"{self.prefix}.hc{q}.{n}").to(f32).contiguous() for n in ("in", "out", "mix"))
            else:
                one = torch.ones(1, dtype=f32, device=self.env.device)
                self.coef[q] = (one, one, one.view(1, 1))

    def forward(self, layer, residual, pending, ctx, cache_view):
        norm1, norm2 = layer.norm_mixer, layer.norm_feed_forward
        if not isinstance(norm1, RMSNorm) or (self.has_ff and not isinstance(norm2, RMSNorm)):
            raise TypeError(f"{self.prefix}: the block works with rmsnorm norms")
        in1, out1, mix1 = self.coef[1]
        if residual.dim() == 2:
            # the first layer: the copies do not exist yet; all of them are the stream as it comes
            if pending is not None:
                raise TypeError(f"{self.prefix}: the first block of copies cannot follow a block that leaves a sum open")
            streams = torch.empty((residual.shape[0], self.copies, self.width), dtype=torch.float32, device=residual.device)
            h = ops.hyper_step(streams, norm1.weight, norm1.eps, self.env.dtype, x_in=residual, in_coef=in1)
        else:
            if pending is not None and not isinstance(pending, HyperPending):
                raise TypeError(f"{self.prefix}: the block before this one left a sum that is not for copies of the stream")
            streams = residual
            h = resolve_hyper(streams, pending, norm1.weight, norm1.eps, self.env.dtype, in1)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.stream_in", streams)        # debug: the copies as this layer reads them
        y = layer.mixer.forward(h, ctx, cache_view)
        pending = HyperPending(delta=y, mix=mix1, out_coef=out1, mult=self.mult)
        if self.has_ff:
            in2, out2, mix2 = self.coef[2]
            if getattr(layer.feed_forward, "wants_f32_input", False):
                h, h32 = resolve_hyper(streams, pending, norm2.weight, norm2.eps, self.env.dtype, in2, also_f32=True)
                y = layer.feed_forward.forward(h, ctx, normed_f32=h32)
            else:
                h = resolve_hyper(streams, pending, norm2.weight, norm2.eps, self.env.dtype, in2)
                y = layer.feed_forward.forward(h, ctx)
            pending = HyperPending(delta=y, mix=mix2, out_coef=out2, mult=self.mult)
        return streams, pending


# --------------------------------------------------------------------------- between passes
@register("interlude", "pass_offset")
class PassOffset(Part):
    """What a model adds to the stream right before a pass over a range of its layers that runs several times:
    a learned vector per pass, and (``add_embedding``) before every pass but the first the embedding output
    again. Whatever the layer before left open is summed into the stream by the same kernel.

    params: ``hidden_size``, ``times``, ``add_embedding`` (default True); tensor ``<prefix>`` [times, W]."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.width, self.times = int(params["hidden_size"]), int(params["times"])
        self.needs_embedding_output = bool(params.get("add_embedding", True)) and self.times > 1
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix, (self.times, self.width))]

    def load(self, fetch):
        self.table = fetch(self.prefix).to(torch.float32).contiguous()

    def forward(self, residual, pending, ctx, arg: int):
        d1 = d2 = None
        if isinstance(pending, Pending):
            if pending.routed is not None:
                d1 = pending.materialize(residual.shape[0])
            else:
                d1, d2 = pending.dense, pending.dense2
        elif pending is not None:
            d1 = pending
        again = ctx.scratch["embedding_output"] if self.needs_embedding_output and arg > 0 else None
        ops.stream_add(residual, d1, d2, again, self.table[arg])
        return residual, None
