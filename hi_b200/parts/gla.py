"""Gated linear attention: a matrix memory per head with a learned decay per key channel, a fixed-size state
per request instead of a cache that grows."""
from __future__ import annotations

import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "gla")
class GatedLinearAttentionMixer(Part):
    """Per head a matrix S [dim, vdim], zero at a sequence's start:

        q = W_q h * dim^-1/2, k = W_k h [heads, dim];  v = W_v h [heads, vdim]
        alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)                      [heads, dim]
        S <- diag(alpha) S + k v^T;  o = S^T q
        y = o / rms_vdim(o) * w_norm * silu(W_g h);  out = W_o y

    The recurrence is the one of the delta rule without its correction term and runs in the same kernels
    (``ops.delta_recurrence(plain=True)``); the decay is worked out in float32 as exp(-softplus(-z) / tau) from the
    float32 result of the second low-rank product (``ops.gla_prep``). State per request: S of every head, one
    float32 row.

    params: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``tau``, ``decay_rank``, ``eps`` (of the output norm).
    tensors: ``<prefix>.{q,k}`` [heads*dim, H], ``<prefix>.{v,g}`` [heads*vdim, H], ``<prefix>.a1`` [r, H],
    ``<prefix>.a2`` [heads*dim, r], ``<prefix>.a2.b`` [heads*dim], ``<prefix>.norm`` [vdim], ``<prefix>.o`` [H, heads*vdim]."""

    graph_safe = True
    GENERAL_KERNEL = False       # tests: force the recurrence kernel that keeps S in shared memory

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim = int(p["heads"]), int(p["dim"]), int(p["vdim"])
        self.tau, self.rank, self.eps = float(p["tau"]), int(p["decay_rank"]), float(p["eps"])
        if min(self.heads, self.dim, self.vdim, self.rank) <= 0 or not self.tau > 0:
            raise ValueError(f"{prefix}: heads, sizes and tau must be positive")
        self.w_in = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def cache_spec(self):
        return CacheSpec(state_shape=(self.heads * self.dim * self.vdim,), state_dtype="float32")

    def tensor_specs(self):
        h, pre = self.hidden, self.prefix
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        return [TensorSpec(f"{pre}.q", (hd, h)), TensorSpec(f"{pre}.k", (hd, h)), TensorSpec(f"{pre}.v", (hv, h)),
                TensorSpec(f"{pre}.g", (hv, h)), TensorSpec(f"{pre}.o", (h, hv)),
                TensorSpec(f"{pre}.norm", (self.vdim,), init="ones"),
                TensorSpec(f"{pre}.a1", (self.rank, h)), TensorSpec(f"{pre}.a2", (hd, self.rank)),
                TensorSpec(f"{pre}.a2.b", (hd,))]

    def load(self, fetch):
        pre = self.prefix
        rows = [fetch(f"{pre}.{n}") for n in ("q", "k", "v", "g", "a1")]
        dt = rows[0].dtype
        self.w_in = torch.cat([t.to(dt) for t in rows], dim=0).contiguous()     # one product: [q | k | v | gate | decay's inner]
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        self.off_k, self.off_v, self.off_g, self.off_a = hd, 2 * hd, 2 * hd + hv, 2 * hd + 2 * hv
        self.w_a2 = fetch(f"{pre}.a2").to(dt).contiguous()
        self.b_a2 = fetch(f"{pre}.a2.b").to(torch.float32).contiguous()
        self.w_norm = fetch(f"{pre}.norm").to(dt).contiguous()
        self.w_o = fetch(f"{pre}.o").contiguous()

    def forward(self, normed, ctx, cache):
        if cache.state is None or not cache.writes:
            raise RuntimeError(f"{self.prefix}: the recurrent mixer needs a state slot of its own")
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        proj = linear(normed, self.w_in)
        z = linear(proj[:, self.off_a: self.off_a + self.rank], self.w_a2, out_dtype=torch.float32)
        q, k, v, decay = ops.gla_prep(proj, 0, self.off_k, self.off_v, z, self.b_a2, self.tau, self.dim ** -0.5, hd, hv)
        o = ops.delta_recurrence(q, k, v, None, decay, cache.state, ctx.cu_seqlens, ctx.slots, self.heads, self.heads,
                                 self.dim, self.vdim, general=self.GENERAL_KERNEL, single_tokens=ctx.max_new == 1,
                                 plain=True)
        y = ops.delta_out_norm(o, proj[:, self.off_g: self.off_g + hv], self.w_norm, self.eps, self.vdim, proj.dtype,
                               gate_silu=True)
        return linear(y, self.w_o)
