"""The gated delta rule with a decay per head and key channel: a recurrent mixer with a fixed-size
state per request instead of a cache that grows."""
from __future__ import annotations

import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "gated_delta")
@register("mixer", "channel_delta")
class ChannelDeltaMixer(Part):
    """Per head a matrix S [dim, vdim] that every token decays row by row, corrects towards its value
    along its key, and reads with its query:

        q, k = W_q h, W_k h [kv_heads, dim],  v = W_v h [heads, vdim]; head a uses q/k head a // (heads / kv_heads)
        each through a causal convolution over time per channel (``conv`` taps, the last the token's own) and silu
        q, k <- unit length per head; q <- q * dim^-1/2
        beta = sigmoid(W_b h) [heads]
        g = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))  [heads, dim]
        S <- g * S (rows);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
        o <- o / rms_vdim(o) * w_norm * sigmoid(W_g2 (W_g1 h));  out = W_o o

    State per request (float32, one flat row of the cache's state tensor): S of every head, then the
    last (taps - 1) inputs of the convolutions. Everything between the projections and the output norm is
    float32 (``ops.delta_prep``, ``ops.delta_recurrence``, ``ops.delta_out_norm``).

    params: ``hidden_size``, ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps), ``decay_rank`` and
    ``gate_rank`` (inner sizes of the two low-rank maps), ``eps`` (of the output norm);
    ``decay_per`` "channel" (default, as above) | "head": one decay per head,
    g = exp(-exp(A_log) * softplus(W_a h + dt_bias)) with ``<prefix>.a`` [heads, H] and ``dt_bias`` [heads] (no a1 / a2);
    ``gate`` "low_rank_sigmoid" (default, as above) | "silu": the output is multiplied by silu(W_g h) with
    ``<prefix>.g`` [heads*vdim, H] (no g1 / g2).
    tensors: ``<prefix>.{q,k,v}`` and ``<prefix>.{q,k,v}.conv`` [channels, taps], ``<prefix>.b`` [heads, H],
    ``<prefix>.A_log`` [heads], ``<prefix>.a1`` [r, H], ``<prefix>.a2`` [heads*dim, r], ``<prefix>.dt_bias``
    [heads*dim], ``<prefix>.g1`` [r', H], ``<prefix>.g2`` [heads*vdim, r'], ``<prefix>.norm`` [vdim],
    ``<prefix>.o`` [H, heads*vdim]."""

    graph_safe = True
    GENERAL_KERNEL = False       # tests: force the recurrence kernel that keeps S in shared memory

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.kvh, self.dim, self.vdim = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
        self.taps = int(p["conv"])
        self.head_decay = p.get("decay_per", "channel") == "head"
        self.silu_gate = p.get("gate", "low_rank_sigmoid") == "silu"
        if p.get("decay_per", "channel") not in ("channel", "head") or p.get("gate", "low_rank_sigmoid") not in ("low_rank_sigmoid", "silu"):
            raise ValueError(f"{prefix}: decay_per is 'channel' or 'head', gate 'low_rank_sigmoid' or 'silu'")
        self.decay_rank = self.heads if self.head_decay else int(p["decay_rank"])       # columns of the decay's part of the product
        self.gate_rank = self.heads * self.vdim if self.silu_gate else int(p["gate_rank"])
        self.eps = float(p["eps"])
        if self.heads % self.kvh:
            raise ValueError(f"{prefix}: {self.heads} heads are not a multiple of {self.kvh} kv heads")
        if self.taps < 1:
            raise ValueError(f"{prefix}: the convolution needs at least one tap")
        self.qk = self.kvh * self.dim
        self.channels = 2 * self.qk + self.heads * self.vdim
        self.s_len = self.heads * self.dim * self.vdim
        self.w_in = self.w_a2 = self.w_g2 = self.w_o = None
        self.conv_taps = self.a_log = self.dt_bias = self.w_norm = None

    def cache_spec(self):
        return CacheSpec(state_shape=(self.s_len + (self.taps - 1) * self.channels,), state_dtype="float32")

    def tensor_specs(self):
        h, pre = self.hidden, self.prefix
        hv, hd = self.heads * self.vdim, self.heads * self.dim
        specs = [TensorSpec(f"{pre}.q", (self.qk, h)), TensorSpec(f"{pre}.q.conv", (self.qk, self.taps)),
                 TensorSpec(f"{pre}.k", (self.qk, h)), TensorSpec(f"{pre}.k.conv", (self.qk, self.taps)),
                 TensorSpec(f"{pre}.v", (hv, h)), TensorSpec(f"{pre}.v.conv", (hv, self.taps)),
                 TensorSpec(f"{pre}.b", (self.heads, h)), TensorSpec(f"{pre}.A_log", (self.heads,), init="zeros"),
                 TensorSpec(f"{pre}.norm", (self.vdim,), init="ones"), TensorSpec(f"{pre}.o", (h, hv))]
        if self.head_decay:
            specs += [TensorSpec(f"{pre}.a", (self.heads, h)), TensorSpec(f"{pre}.dt_bias", (self.heads,))]
        else:
            specs += [TensorSpec(f"{pre}.a1", (self.decay_rank, h)), TensorSpec(f"{pre}.a2", (hd, self.decay_rank)),
                      TensorSpec(f"{pre}.dt_bias", (hd,))]
        if self.silu_gate:
            specs.append(TensorSpec(f"{pre}.g", (hv, h)))
        else:
            specs += [TensorSpec(f"{pre}.g1", (self.gate_rank, h)), TensorSpec(f"{pre}.g2", (hv, self.gate_rank))]
        return specs

    def load(self, fetch):
        pre = self.prefix
        rows = [fetch(f"{pre}.{n}") for n in ("q", "k", "v", "b", "a" if self.head_decay else "a1",
                                              "g" if self.silu_gate else "g1")]
        dt = rows[0].dtype
        # one product for everything that reads h: [q | k | v | beta | decay's inner | gate's inner]
        self.w_in = torch.cat([t.to(dt) for t in rows], dim=0).contiguous()
        self.off_beta = self.channels
        self.off_a = self.off_beta + self.heads
        self.off_g = self.off_a + self.decay_rank
        self.w_a2 = None if self.head_decay else fetch(f"{pre}.a2").contiguous()
        self.w_g2 = None if self.silu_gate else fetch(f"{pre}.g2").contiguous()
        self.w_o = fetch(f"{pre}.o").contiguous()
        f32 = torch.float32
        self.conv_taps = torch.cat([fetch(f"{pre}.{n}.conv").to(f32) for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log = fetch(f"{pre}.A_log").to(f32).contiguous()
        self.dt_bias = fetch(f"{pre}.dt_bias").to(f32).contiguous()
        self.w_norm = fetch(f"{pre}.norm").to(dt).contiguous()

    def forward(self, normed, ctx, cache):
        if cache.state is None or not cache.writes:
            raise RuntimeError(f"{self.prefix}: the recurrent mixer needs a state slot of its own")
        proj = linear(normed, self.w_in)
        a_pre = proj[:, self.off_a: self.off_a + self.decay_rank]
        a_pre = a_pre.contiguous() if self.head_decay else linear(a_pre, self.w_a2, out_dtype=torch.float32)
        gate = proj[:, self.off_g: self.off_g + self.gate_rank]
        if not self.silu_gate:
            gate = linear(gate, self.w_g2)
        q, k, v, beta, decay = ops.delta_prep(proj, 0, self.off_beta, self.conv_taps, cache.state, self.s_len, a_pre,
                                              self.dt_bias, self.a_log, ctx.cu_seqlens, ctx.seq_of_token, ctx.slots,
                                              self.heads, self.kvh, self.dim, self.vdim, head_decay=self.head_decay)
        ops.delta_conv_update(proj, 0, self.channels, self.taps, cache.state, self.s_len, ctx.cu_seqlens, ctx.slots)
        o = ops.delta_recurrence(q, k, v, beta, decay, cache.state, ctx.cu_seqlens, ctx.slots, self.heads, self.kvh,
                                 self.dim, self.vdim, general=self.GENERAL_KERNEL, single_tokens=ctx.max_new == 1)
        y = ops.delta_out_norm(o, gate, self.w_norm, self.eps, self.vdim, proj.dtype, gate_silu=self.silu_gate)
        return linear(y, self.w_o)
