"""The attention mixer: grouped-query attention over a paged cache, global or windowed."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..kernels import ops
from .basic import Part
from .linear import linear
from .registry import build, register
from .spec import CacheSpec, PartSpec, TensorSpec


def _key_splits(ctx, nh: int, chunk: int, sliding: int, single: bool, device) -> int:
    """Portions far into long contexts on a layer that sees every key: all blocks of the
    tensor-core prefill kernel then have about the same many key tiles, and a partly filled
    last round of blocks is worth splitting the keys for (ops.prefill_key_splits)."""
    if chunk or sliding:
        return 1
    portions = [(s, n) for s, n in zip(ctx.start_pos, ctx.n_new) if n > 1 or not single]
    if not portions:
        return 1
    shortest, longest_new = min(s for s, _n in portions), max(n for _s, n in portions)
    if shortest < 2 * longest_new:
        return 1
    blocks = nh * sum(-(-n // ops.PREFILL_TC_MIN_TOKENS) for _s, n in portions)
    return ops.prefill_key_splits(blocks, shortest // 64, ops.sm_count(device))


def attend_over_pages(q, k_pages, v_pages, block_table, ctx, nh: int, nkv: int, hd: int, chunk: int, sliding: int,
                      scale: float, sink: bool = False, softcap: float = 0.0, slopes=None, sink_values=None):
    """softmax(q k^T scale + mask) v for the step's tokens over the paged keys and values that are in
    the cache already, by the kernel that fits the step: single decoded tokens, portions of prompts
    (with single tokens of other requests beside them), or the general kernel for what those refuse
    (float32, other head sizes). ``q`` [N, nh, hd] -> [N, nh, hd]. Every mixer whose scores are dot
    products over paged rows comes through here; ``k_pages`` and ``v_pages`` may be the same pool.
    ``sink``: the softmax's denominator has one more term of score 0 (it has no value); ``sink_values``
    (float32 [nh]): of the head's own score instead. ``softcap`` > 0: scores become softcap tanh(score / softcap);
    ``slopes`` (float32 [nh]): slopes[head] * (distance to the key) is taken off after the cap."""
    positions = ctx.positions
    # the decode kernel packs the query heads of one kv head into a 16-row tile; more heads on ONE shared kv
    # head go through it sixteen at a time
    per_call = nh if nkv > 1 or nh <= 16 else 16
    decode_ok = ops.decode_attention_supported(q.dtype, per_call, nkv, hd)

    def decode(rows_q, seq, pos, longest):
        if per_call == nh:
            return ops.decode_attention(rows_q, k_pages, v_pages, block_table, seq, pos, chunk, sliding, scale, longest,
                                        sink=sink, softcap=softcap, slopes=slopes, sink_values=sink_values)
        out = torch.empty_like(rows_q)
        for first in range(0, nh, per_call):
            part = rows_q[:, first: first + per_call].contiguous()
            own = [None if t is None else t[first: first + per_call].contiguous() for t in (slopes, sink_values)]
            out[:, first: first + per_call] = ops.decode_attention(part, k_pages, v_pages, block_table, seq, pos, chunk,
                                                                   sliding, scale, longest, sink=sink, softcap=softcap,
                                                                   slopes=own[0], sink_values=own[1])
        return out

    if ctx.max_new == 1 and decode_ok:
        # every token of the step is one request's decoded token: the tensor-core kernel
        return decode(q, ctx.seq_of_token, positions, ctx.max_context)
    # at least a tile of new tokens somewhere: the tcgen05 kernel; short portions: mma.sync
    tc = ctx.max_new >= ops.PREFILL_TC_MIN_TOKENS and ops.prefill_attention_tc_supported(q.dtype, nh, nkv, hd, ctx.page_size)
    if ctx.max_new > 1 and ops.prefill_attention_supported(q.dtype, nh, nkv, hd):
        # portions of prompts (single tokens of other requests ride along as one-row tiles)
        single = ctx.decode_rows is not None and decode_ok
        if tc:
            o = ops.prefill_attention_tc(q, k_pages, v_pages, block_table, ctx.cu_seqlens, positions,
                                         ctx.n_seqs, ctx.max_new, chunk, sliding, scale, skip_single=single,
                                         key_splits=_key_splits(ctx, nh, chunk, sliding, single, q.device), sink=sink,
                                         softcap=softcap, slopes=slopes, sink_values=sink_values)
        else:
            o = ops.prefill_attention(q, k_pages, v_pages, block_table, ctx.cu_seqlens, positions,
                                      ctx.n_seqs, ctx.max_new, chunk, sliding, scale, skip_single=single, sink=sink,
                                      softcap=softcap, slopes=slopes, sink_values=sink_values)
        if single:
            # single tokens beside portions: their long key ranges go through the split decode kernel
            rows = ctx.decode_rows
            od = decode(q.index_select(0, rows), ctx.seq_of_token.index_select(0, rows), positions.index_select(0, rows),
                        ctx.decode_max_context)
            o.index_copy_(0, rows, od)
        return o
    return ops.paged_attention(q, k_pages, v_pages, block_table, ctx.seq_of_token, positions,
                               chunk, sliding, scale, ctx.max_context, sink=sink, softcap=softcap, slopes=slopes,
                               sink_values=sink_values)


def sigmoid_attend_over_pages(q, k_pages, v_pages, block_table, ctx, nh: int, nkv: int, hd: int, chunk: int,
                              sliding: int, scale: float, head_bias, v_inv_freq, v_interleaved: bool):
    """sum_j sigmoid(q . k_j scale + head_bias) v_j over the keys each token may read, turned back by the token's
    position where the values are cached rotated, by the kernel that fits the step, as :func:`attend_over_pages`
    chooses for the softmax: the tensor-core decode kernel for single tokens, the tcgen05 kernel for portions of
    at least a tile of new tokens (single tokens beside them through the decode kernel), the general kernel for the
    rest (float32, other head sizes, short portions)."""
    positions = ctx.positions
    if ops.sigmoid_attention_tc_supported(q.dtype, nh, nkv, hd, ctx.page_size):
        if ctx.max_new == 1:
            return ops.sigmoid_decode_attention(q, k_pages, v_pages, block_table, ctx.seq_of_token, positions, chunk,
                                                sliding, scale, head_bias, ctx.max_context, v_inv_freq, v_interleaved)
        if ctx.max_new >= ops.PREFILL_TC_MIN_TOKENS:
            single = ctx.decode_rows is not None
            o = ops.sigmoid_prefill_attention_tc(q, k_pages, v_pages, block_table, ctx.cu_seqlens, positions, ctx.n_seqs,
                                                 ctx.max_new, chunk, sliding, scale, head_bias, skip_single=single,
                                                 v_inv_freq=v_inv_freq, v_interleaved=v_interleaved)
            if single:
                rows = ctx.decode_rows
                od = ops.sigmoid_decode_attention(q.index_select(0, rows), k_pages, v_pages, block_table,
                                                  ctx.seq_of_token.index_select(0, rows), positions.index_select(0, rows),
                                                  chunk, sliding, scale, head_bias, ctx.decode_max_context, v_inv_freq,
                                                  v_interleaved)
                o.index_copy_(0, rows, od)
            return o
    return ops.sigmoid_attention(q, k_pages, v_pages, block_table, ctx.seq_of_token, positions, chunk, sliding, scale,
                                 head_bias, ctx.max_context, v_inv_freq=v_inv_freq, v_interleaved=v_interleaved)


@register("mixer", "attention")
class AttentionMixer(Part):
    """q/k/v projections, position encoding or temperature, optional weightless q/k norm, cache
    append, softmax(q k^T scale + mask) v, output projection
    (Llama4Attention::forward, crates/hi-mlx/src/models.rs:5978-6052).

    params:
      ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``
      ``window``       None (every earlier key) | ("chunk", C) | ("sliding", W)
      ``position``     PartSpec of the position family
      ``qk_norm``, ``qk_norm_eps``   weightless L2 norm of q and k after the rotation
      ``temperature``  None | (floor_scale, attn_scale): q *= 1 + attn_scale*ln(1 + floor((pos+1)/floor_scale))
      ``scale``        softmax scale; default head_dim ** -0.5 (models.rs:5963)
      ``bias``         the random-weights writer makes the projections' biases too: True (all four) or a
                       string of the projections that have one ("qkv")
      ``value_dim``    size of a value head where it differs from ``head_dim`` (the query/key size). Keys,
                       values and queries are then kept in rows of one padded size (the larger of the two,
                       rounded up to 16): the projections get zero rows, the output projection zero columns
      ``qk_norm_weighted``  the norm of q and k is an RMS norm BEFORE the rotation with a weight per dim,
                       ``<prefix>.q.norm`` / ``<prefix>.k.norm`` [head_dim], shared by the heads
      ``sink``         the softmax's denominator has one more term of score 0: exp(s_j) / (1 + sum exp(s_j));
                       "learned": the term's score is a number per head, ``<prefix>.sink`` [heads], that is not
                       scaled, capped or biased: exp(s_j) / (exp(sink_h) + sum exp(s_j))
      ``softcap``      None | c: the scaled score becomes c tanh(score / c)
      ``distance_bias``  None | e: slope_h * (i - j) is taken off the (capped) score of query i and key j,
                       slope_h = 2^(-e (h + 1) / heads) for head h = 0 .. heads - 1
      ``names``        "proj" (default): ``<prefix>.{q,k,v,o}_proj.weight`` / ``.bias``;
                       "short": ``<prefix>.{q,k,v,o}`` and ``<prefix>.{q,k,v,o}.b``
      ``weights``      "softmax" (default) | "sigmoid": the weight of a visible key is sigmoid(score + pb[head]),
                       ``<prefix>.pb`` [heads], and the weights are not normalised over the keys
      ``value_rotation``  None | {"base": b, "interleaved": bool}: the value of position j is cached rotated by j
                       over all its dims (pair m by j * b^(-2m / value_dim)) and each head's sum at position i is
                       turned back by i, so a value's weight in the output also depends on i - j
    tensors: the four projections, and each projection's bias where the checkpoint has one (a bias is
    used iff its tensor exists: crates/hi-mlx/src/models.rs:1808, 1843-1845).
    """

    graph_safe = True
    FUSED_DECODE = True      # decode steps: one launch for encoding, cache append, attention and merge

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"{prefix}: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        self.dim, self.vdim = self.hd, int(p.get("value_dim") or self.hd)      # sizes as the checkpoint has them
        self.norm_weighted = bool(p.get("qk_norm_weighted", False))
        self.sink = bool(p.get("sink", False))
        self.learned_sink = p.get("sink") == "learned"
        self.softcap = float(p["softcap"]) if p.get("softcap") else 0.0
        self.distance_bias = float(p["distance_bias"]) if p.get("distance_bias") else None
        self.sink_values = self.slopes = None
        self.sigmoid = p.get("weights", "softmax") == "sigmoid"
        if p.get("weights", "softmax") not in ("softmax", "sigmoid") or (self.sigmoid and self.sink):
            raise ValueError(f"{prefix}: weights are 'softmax' or 'sigmoid' (which has no sink)")
        self.value_rotation = dict(p["value_rotation"]) if p.get("value_rotation") else None
        if self.value_rotation and not self.sigmoid:
            raise ValueError(f"{prefix}: rotated values are built for sigmoid weights only")
        if self.sigmoid and (self.softcap or self.distance_bias is not None):
            raise ValueError(f"{prefix}: a cap or a distance bias on the scores is built for softmax weights only")
        self.head_bias = self._v_table = None
        self.short_names = p.get("names", "proj") == "short"
        if self.dim != self.vdim or self.dim % 16:
            self.hd = -(-max(self.dim, self.vdim) // 16) * 16                  # rows of the cache and of q
        if self.hd > (1024 if self.hd != self.dim or self.norm_weighted else 256):
            raise ValueError(f"{prefix}: head size {self.hd} is not supported")
        self.window = tuple(p["window"]) if p.get("window") else None
        self.position = build("position", p.get("position") or PartSpec("none"), env, prefix)
        self.qk_norm = bool(p.get("qk_norm", False)) or self.norm_weighted
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.temperature = tuple(p["temperature"]) if p.get("temperature") else None
        self.scale = float(p.get("scale") or self.dim ** -0.5)
        self.bias = p.get("bias", False)
        self.w_qnorm = self.w_knorm = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    def cache_spec(self):
        return CacheSpec(kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    def _name(self, proj: str, bias: bool = False) -> str:
        if self.short_names:
            return f"{self.prefix}.{proj}.b" if bias else f"{self.prefix}.{proj}"
        return f"{self.prefix}.{proj}_proj.bias" if bias else f"{self.prefix}.{proj}_proj.weight"

    def tensor_specs(self):
        h, nh, nkv = self.hidden, self.nh, self.nkv
        have = "qkvo" if self.bias is True else (self.bias or "")
        rows = {"q": nh * self.dim, "k": nkv * self.dim, "v": nkv * self.vdim, "o": h}
        specs = [TensorSpec(self._name(n), (rows[n], h) if n != "o" else (h, nh * self.vdim)) for n in "qkvo"]
        # "absent": the random-weights writer leaves them out
        specs += [TensorSpec(self._name(n, bias=True), (rows[n],), init="normal" if n in have else "absent", optional=True)
                  for n in "qkvo"]
        if self.norm_weighted:
            specs += [TensorSpec(f"{self.prefix}.{n}.norm", (self.dim,), init="ones") for n in "qk"]
        if self.sigmoid:
            specs.append(TensorSpec(f"{self.prefix}.pb", (self.nh,)))
        if self.learned_sink:
            specs.append(TensorSpec(f"{self.prefix}.sink", (self.nh,)))
        return specs

    def _pad_heads(self, t, heads: int, size: int):
        """[heads * size, ...] -> [heads * hd, ...] with zero rows behind every head's own."""
        if t is None or size == self.hd:
            return t
        out = torch.zeros((heads, self.hd, *t.shape[1:]), dtype=t.dtype, device=t.device)
        out[:, :size] = t.view(heads, size, *t.shape[1:])
        return out.view(heads * self.hd, *t.shape[1:])

    def load(self, fetch):
        q, k, v = (fetch(self._name(n)) for n in "qkv")
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        sizes = ((self.nh, self.dim), (self.nkv, self.dim), (self.nkv, self.vdim))
        q, k, v = (self._pad_heads(t, *hs) for t, hs in zip((q, k, v), sizes))
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()     # one product for q, k and v
        w_o = fetch(self._name("o"))
        if self.vdim != self.hd:
            w_o = self._pad_heads(w_o.t().contiguous(), self.nh, self.vdim).t()
        self.w_o = w_o.contiguous()
        biases = [fetch(self._name(n, bias=True)) for n in "qkv"]
        if any(b is not None for b in biases):          # a projection without one adds zeros
            biases = [torch.zeros(hs[0] * self.hd, dtype=self.w_qkv.dtype, device=self.w_qkv.device) if b is None
                      else self._pad_heads(b, *hs) for b, hs in zip(biases, sizes)]
            self.b_qkv = torch.cat([b.to(self.w_qkv.dtype) for b in biases]).contiguous()
        b_o = fetch(self._name("o", bias=True))
        self.b_o = None if b_o is None else b_o.to(self.w_o.dtype).contiguous()
        if self.norm_weighted:
            def weight(n):
                w = torch.zeros(self.hd, dtype=torch.float32, device=self.w_qkv.device)
                w[: self.dim] = fetch(f"{self.prefix}.{n}.norm").to(torch.float32)
                return w
            self.w_qnorm, self.w_knorm = weight("q"), weight("k")
        if self.sigmoid:
            self.head_bias = fetch(f"{self.prefix}.pb").to(torch.float32).contiguous()
        if self.learned_sink:
            self.sink_values = fetch(f"{self.prefix}.sink").to(torch.float32).contiguous()
        if self.distance_bias is not None:
            slopes = [2.0 ** (-self.distance_bias * (h + 1) / self.nh) for h in range(self.nh)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(self.w_qkv.device)
        if self.value_rotation:
            if self.vdim % 2:
                raise ValueError(f"{self.prefix}: rotated values need an even value size")
            base = float(self.value_rotation["base"])
            table = np.array([base ** (-2.0 * m / self.vdim) for m in range(self.vdim // 2)], dtype=np.float64)
            self._v_table = torch.from_numpy(table.astype(np.float32)).to(self.w_qkv.device)

    def forward(self, normed, ctx, cache):
        qkv = linear(normed, self.w_qkv, bias=self.b_qkv)
        positions = ctx.positions
        table = self.position.rotary_table()
        if table is None and hasattr(self.position, "apply"):
            # a position part without a rotary table encodes q and k itself
            n = qkv.shape[0]
            q, k, v = qkv.split([self.nh * self.hd, self.nkv * self.hd, self.nkv * self.hd], dim=1)
            q, k = self.position.apply(q.reshape(n, self.nh, self.hd), k.reshape(n, self.nkv, self.hd), positions)
            qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v], dim=1).to(normed.dtype).contiguous()
        inv_freq, interleaved = table if table is not None else (None, False)
        block_table = ctx.block_tables[cache.group]
        chunk = self.window[1] if self.window and self.window[0] == "chunk" else 0
        sliding = self.window[1] if self.window and self.window[0] == "sliding" else 0
        rot_mul = float(getattr(self.position, "magnitude", 1.0))
        plain = not (self.norm_weighted or self.sink or self.hd != self.dim or rot_mul != 1.0)
        if self.sigmoid:
            v_inter = bool(self.value_rotation and self.value_rotation.get("interleaved", False))
            q = ops.qkv_post(qkv, self.nh, self.nkv, self.hd, positions, inv_freq, interleaved, self.qk_norm,
                             self.qk_norm_eps, self.temperature, ctx.seq_of_token, block_table, cache.k_pages,
                             cache.v_pages, ctx.page_size, cache.writes, q_norm_weight=self.w_qnorm,
                             k_norm_weight=self.w_knorm, norm_first=self.norm_weighted,
                             norm_dim=0 if plain else self.dim, rot_mul=rot_mul, v_inv_freq=self._v_table,
                             v_interleaved=v_inter)
            o = sigmoid_attend_over_pages(q, cache.k_pages, cache.v_pages, block_table, ctx, self.nh, self.nkv, self.hd,
                                          chunk, sliding, self.scale, self.head_bias, self._v_table, v_inter)
            return linear(o.view(o.shape[0], self.nh * self.hd), self.w_o, bias=self.b_o)
        extras = bool(self.softcap) or self.slopes is not None or self.sink_values is not None
        if self.hd == self.dim and ctx.max_new == 1 and cache.writes and self.FUSED_DECODE and qkv.dtype == torch.bfloat16 \
                and not extras:
            # a step of single decoded tokens: encoding, cache append, attention and the merge of its
            # splits in one launch, where the kernel takes the shapes
            o = ops.decode_attention_fused(qkv, self.nh, self.nkv, self.hd, positions, inv_freq, interleaved, self.qk_norm,
                                           self.qk_norm_eps, self.temperature, ctx.seq_of_token, block_table,
                                           cache.k_pages, cache.v_pages, chunk, sliding, self.scale, ctx.max_context,
                                           q_norm_weight=self.w_qnorm, k_norm_weight=self.w_knorm,
                                           norm_first=self.norm_weighted, rot_mul=rot_mul, sink=self.sink)
            if o is not None:
                return linear(o.view(o.shape[0], self.nh * self.hd), self.w_o, bias=self.b_o)
        q = ops.qkv_post(qkv, self.nh, self.nkv, self.hd, positions, inv_freq, interleaved, self.qk_norm,
                         self.qk_norm_eps, self.temperature, ctx.seq_of_token, block_table, cache.k_pages,
                         cache.v_pages, ctx.page_size, cache.writes, q_norm_weight=self.w_qnorm,
                         k_norm_weight=self.w_knorm, norm_first=self.norm_weighted,
                         norm_dim=0 if plain else self.dim, rot_mul=rot_mul)
        o = attend_over_pages(q, cache.k_pages, cache.v_pages, block_table, ctx, self.nh, self.nkv, self.hd, chunk,
                              sliding, self.scale, sink=self.sink, softcap=self.softcap, slopes=self.slopes,
                              sink_values=self.sink_values)
        return linear(o.view(o.shape[0], self.nh * self.hd), self.w_o, bias=self.b_o)
