"""Mamba-2: a selective state-space mixer with a scalar decay per head, a fixed-size state per request."""
from __future__ import annotations

import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "mamba2")
class Mamba2Mixer(Part):
    """One projection of the input gives [z | x | B | C | dt] (inner = heads * vdim; z, x [inner]; B, C [groups * N];
    dt [heads]). x, B and C pass a causal convolution over time per channel (``conv`` taps, the last the token's own,
    plus a bias) and silu. Per head a (which reads B and C of group a // (heads / groups)) a matrix S [N, vdim]:

        dt = softplus(dt + dt_bias)                       (no clamp)
        S <- exp(-exp(A_log_a) dt) S + dt B x_a^T;   y_a = S^T C + D_a x_a
        y <- y * silu(z);  RMS norm of y in ``norm_groups`` equal runs, each by its own root mean square; * w;  out = W_o y

    State per request (float32, one flat row of the cache's state tensor): S of every head, then the last
    (taps - 1) inputs of the convolution. The recurrence is the delta rule's kernel without its correction term
    (``ops.delta_recurrence(plain=True)`` with k = B, q = C, v = dt x); everything between the projection and the
    normed output is float32 (``ops.mamba2_prep``, ``ops.mamba2_out``).

    params: ``hidden_size``, ``heads``, ``vdim``, ``state`` (N), ``groups``, ``conv`` (taps), ``norm_groups``, ``eps``.
    tensors: ``<prefix>.in`` [2*inner + 2*groups*N + heads, H], ``<prefix>.conv`` [inner + 2*groups*N, taps],
    ``<prefix>.conv.b``, ``<prefix>.dt_bias`` [heads], ``<prefix>.A_log`` [heads], ``<prefix>.D`` [heads],
    ``<prefix>.norm`` [inner], ``<prefix>.o`` [H, inner]."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.taps, self.parts = int(p["groups"]), int(p["conv"]), int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        if self.heads % self.groups:
            raise ValueError(f"{prefix}: {self.heads} heads are not a multiple of {self.groups} groups")
        if self.taps < 1 or self.parts < 1 or self.inner % self.parts:
            raise ValueError(f"{prefix}: the convolution needs a tap, and norm_groups must divide heads * vdim")
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.s_len = self.heads * self.n_state * self.vdim
        self.w_in = self.w_o = self.conv_taps = self.conv_bias = self.dt_bias = self.a_log = self.d_skip = self.w_norm = None

    def cache_spec(self):
        return CacheSpec(state_shape=(self.s_len + (self.taps - 1) * self.channels,), state_dtype="float32")

    def tensor_specs(self):
        h, pre = self.hidden, self.prefix
        return [TensorSpec(f"{pre}.in", (self.inner + self.channels + self.heads, h)),
                TensorSpec(f"{pre}.conv", (self.channels, self.taps)), TensorSpec(f"{pre}.conv.b", (self.channels,)),
                TensorSpec(f"{pre}.dt_bias", (self.heads,)), TensorSpec(f"{pre}.A_log", (self.heads,), init="zeros"),
                TensorSpec(f"{pre}.D", (self.heads,), init="ones"), TensorSpec(f"{pre}.norm", (self.inner,), init="ones"),
                TensorSpec(f"{pre}.o", (h, self.inner))]

    def load(self, fetch):
        pre, f32 = self.prefix, torch.float32
        self.w_in = fetch(f"{pre}.in").contiguous()
        self.w_o = fetch(f"{pre}.o").contiguous()
        self.conv_taps = fetch(f"{pre}.conv").to(f32).contiguous()
        self.conv_bias = fetch(f"{pre}.conv.b").to(f32).contiguous()
        self.dt_bias = fetch(f"{pre}.dt_bias").to(f32).contiguous()
        self.a_log = fetch(f"{pre}.A_log").to(f32).contiguous()
        self.d_skip = fetch(f"{pre}.D").to(f32).contiguous()
        self.w_norm = fetch(f"{pre}.norm").to(self.w_in.dtype).contiguous()

    def forward(self, normed, ctx, cache):
        if cache.state is None or not cache.writes:
            raise RuntimeError(f"{self.prefix}: the recurrent mixer needs a state slot of its own")
        proj = linear(normed, self.w_in)
        x, v, k, q, decay = ops.mamba2_prep(proj, self.inner, self.inner + self.channels, self.conv_taps, self.conv_bias,
                                            cache.state, self.s_len, self.dt_bias, self.a_log, ctx.cu_seqlens,
                                            ctx.seq_of_token, ctx.slots, self.heads, self.groups, self.n_state, self.vdim)
        ops.delta_conv_update(proj, self.inner, self.channels, self.taps, cache.state, self.s_len, ctx.cu_seqlens,
                              ctx.slots)
        o = ops.delta_recurrence(q, k, v, None, decay, cache.state, ctx.cu_seqlens, ctx.slots, self.heads, self.groups,
                                 self.n_state, self.vdim, single_tokens=ctx.max_new == 1, plain=True)
        y = ops.mamba2_out(o, x, proj[:, : self.inner], self.d_skip, self.w_norm, self.eps, self.heads, self.vdim,
                           self.parts, proj.dtype)
        return linear(y, self.w_o)
