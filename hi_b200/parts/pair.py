"""Two mixers side by side on the same input, joined by a normed mean."""
from __future__ import annotations

from ..kernels import ops
from .basic import Part
from .registry import build, register
from .spec import CacheSpec, PartSpec, TensorSpec


@register("mixer", "mixer_pair")
class MixerPair(Part):
    """out = (rmsnorm(left(h)) * w_left + rmsnorm(right(h)) * w_right) / 2, both norms over the model width.

    The two mixers are registered mixers of any kind; their tensors live under ``<prefix>.left`` and
    ``<prefix>.right``. Their cache needs are joined into one cache slot: at most one of them keeps paged keys
    and values, at most one a fixed-size state, and each reads its own half of the slot's view.

    params: ``hidden_size``, ``eps``, ``left`` and ``right`` = {"kind": registered mixer, "params": {...}}.
    tensors: the two mixers', ``<prefix>.left.out`` [W], ``<prefix>.right.out`` [W]."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.width, self.eps = int(params["hidden_size"]), float(params["eps"])
        self.sides = [build("mixer", PartSpec(params[s]["kind"], dict(params[s]["params"])), env, f"{prefix}.{s}")
                      for s in ("left", "right")]
        self.graph_safe = all(getattr(m, "graph_safe", False) for m in self.sides)
        self.w = [None, None]
        specs = [m.cache_spec() for m in self.sides]
        paged = [s for s in specs if s is not None and s.paged]
        stateful = [s for s in specs if s is not None and s.state_shape]
        if len(paged) > 1 or len(stateful) > 1:
            raise ValueError(f"{prefix}: a pair holds at most one mixer with paged keys and one with a state")
        self._cache_spec = None
        if paged or stateful:
            p, s = (paged[0] if paged else CacheSpec()), (stateful[0] if stateful else CacheSpec())
            self._cache_spec = CacheSpec(kv_heads=p.kv_heads, head_dim=p.head_dim, window=p.window, values=p.values,
                                         state_shape=s.state_shape, state_dtype=s.state_dtype)

    def cache_spec(self):
        return self._cache_spec

    def tensor_specs(self):
        specs = [t for m in self.sides for t in m.tensor_specs()]
        return specs + [TensorSpec(f"{self.prefix}.{s}.out", (self.width,), init="ones") for s in ("left", "right")]

    def load(self, fetch):
        for m in self.sides:
            m.load(fetch)
        self.w = [fetch(f"{self.prefix}.{s}.out").contiguous() for s in ("left", "right")]

    def forward(self, normed, ctx, cache):
        a = self.sides[0].forward(normed, ctx, cache)
        b = self.sides[1].forward(normed, ctx, cache)
        return ops.rmsnorm_mean2(a, b, self.w[0], self.w[1], self.eps, normed.dtype)
