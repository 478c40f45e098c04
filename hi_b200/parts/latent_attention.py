"""Latent attention: the cache holds one low-rank latent per token; every head's keys and values are
linear maps of it."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .attention import attend_over_pages
from .basic import Part, exact_inverse_frequencies, yarn_inverse_frequencies
from .linear import linear
from .registry import register
from .spec import CacheSpec, TensorSpec


@register("mixer", "latent_attention")
class LatentAttentionMixer(Part):
    """q = W_q h [heads, dim];  c = rmsnorm(W_dkv h) * w_c  [rank], the only thing cached;
    per head a: k_a = U_a c, v_a = V_a c;  o_a = softmax_j(q_a . k_a(j) * scale) v_a(j) over j <= i;
    o_a *= sigmoid(W_g h)_a;  out = W_o concat(o_a).  No position encoding.

    Computed on the latents: q_a . (U_a c) = (U_a^T q_a) . c and sum_j p_j V_a c_j = V_a (sum_j p_j c_j), so
    the step's queries are mapped into latent space (one batched product), attention runs over the paged
    latents with one shared "kv head" whose keys and values are the same rows (the paged attention kernels
    of the other mixers), and the result is mapped out by V_a (another batched product). The cached rows are
    padded with zeros to 64, 128 or 192 elements (longer ones to a multiple of 16), which changes no dot product.

    A mixer with ``kv_source`` makes no latents: its schedule entry reads the cache slot of the layer that
    does (``writes_cache=False``), with its own U, V, queries and everything else.

    With ``rot_dim`` > 0 every head's query has rot_dim more dims behind its ``dim`` plain ones, and the down
    projection rot_dim more rows behind the latent's: one key part per token that all heads share, not normed.
    Both are rotated by the token's position (pairs (i, i + rot_dim/2), pair i by position * base^(-2i/rot_dim))
    and the score is (q_plain . k_plain + q_rot . k_rot) * scale. The cached row is then [c | k_rot | zeros] and
    the query in latent space [U_a^T q_plain | q_rot]: one dot product over the row gives the whole score; the
    value map has zero rows for the key part. With ``q_rank`` the queries go through a latent of their own:
    q = W_uq rmsnorm(W_dq h) * w_dq.

    params: ``hidden_size``, ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``, ``eps`` (of the latents'
    norms), ``own_latents`` (False for a layer that reads another's), ``window`` (None | ("sliding", W) |
    ("chunk", C): which earlier latents a query reads; default all), ``gate`` (default True: the sigmoid gate
    per head), ``q_rank`` (default None: queries straight from h), ``rot_dim`` (default 0), ``rot_base``,
    ``rot_scaling`` (None | the keys of :func:`~hi_b200.parts.basic.exact_inverse_frequencies`),
    ``rot_kind`` ("llama3", the default | "yarn": ``rot_scaling`` = {factor, original, fast, slow}, the ramped
    frequencies of :func:`~hi_b200.parts.basic.yarn_inverse_frequencies` and their factor on cos and sin, which
    both the query's and the key's rotated part carry), ``rot_interleaved`` (pairs (2i, 2i + 1) instead of
    (i, i + rot_dim/2)).
    tensors: ``<prefix>.q`` [heads*dim, H] (or ``<prefix>.dq`` [q_rank, H], ``<prefix>.dq.norm`` [q_rank],
    ``<prefix>.uq`` [heads*(dim+rot_dim), q_rank]), ``<prefix>.dkv`` [rank+rot_dim, H] and ``<prefix>.dkv.norm``
    [rank] (own latents only), ``<prefix>.uk`` [heads*dim, rank], ``<prefix>.uv`` [heads*vdim, rank],
    ``<prefix>.g`` [heads, H] (with ``gate``), ``<prefix>.o`` [H, heads*vdim].
    """

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["kv_rank"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.dim ** -0.5
        self.eps = float(p["eps"])
        self.own = bool(p.get("own_latents", True))
        self.window = tuple(p["window"]) if p.get("window") else None
        self.gate = bool(p.get("gate", True))
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else 0
        self.rot = int(p.get("rot_dim") or 0)
        if self.rot % 2:
            raise ValueError(f"{prefix}: rot_dim {self.rot} must be even")
        self.qdim = self.dim + self.rot                          # a query head as the checkpoint has it
        # the cached row: padded with zeros to a length the tensor-core kernels take (64, 128, 192), else to 16s
        need = self.rank + self.rot
        self.row_len = next((n for n in ops.TC_ROW_LENGTHS if need <= n), -(-need // 16) * 16)
        if self.row_len > 1024:
            raise ValueError(f"{prefix}: kv_rank {self.rank} + rot_dim {self.rot} is not supported (up to 1024)")
        self._freq_host, self.rot_mul = None, 1.0
        self.rot_interleaved = bool(p.get("rot_interleaved", False))
        if p.get("rot_kind", "llama3") not in ("llama3", "yarn"):
            raise ValueError(f"{prefix}: rot_kind is 'llama3' or 'yarn'")
        if self.rot and p.get("rot_kind", "llama3") == "yarn":
            self._freq_host, self.rot_mul = yarn_inverse_frequencies(self.rot, float(p["rot_base"]), p.get("rot_scaling"))
        elif self.rot:
            self._freq_host = exact_inverse_frequencies(self.rot, float(p["rot_base"]), p.get("rot_scaling"))
        self._freq = None
        self.w_in = self.w_c = self.w_uk_t = self.w_uv_t = self.w_o = self.w_uq = self.w_qn = None

    def cache_spec(self):
        return CacheSpec(kv_heads=1, head_dim=self.row_len, window=self.window, values=False)

    def tensor_specs(self):
        h, hd, hv, r = self.hidden, self.heads * self.dim, self.heads * self.vdim, self.rank
        pre = self.prefix
        if self.q_rank:
            specs = [TensorSpec(f"{pre}.dq", (self.q_rank, h)), TensorSpec(f"{pre}.dq.norm", (self.q_rank,), init="ones"),
                     TensorSpec(f"{pre}.uq", (self.heads * self.qdim, self.q_rank))]
        else:
            specs = [TensorSpec(f"{pre}.q", (self.heads * self.qdim, h))]
        if self.own:
            specs += [TensorSpec(f"{pre}.dkv", (r + self.rot, h)), TensorSpec(f"{pre}.dkv.norm", (r,), init="ones")]
        specs += [TensorSpec(f"{pre}.uk", (hd, r)), TensorSpec(f"{pre}.uv", (hv, r))]
        if self.gate:
            specs.append(TensorSpec(f"{pre}.g", (self.heads, h)))
        return specs + [TensorSpec(f"{pre}.o", (h, hv))]

    def load(self, fetch):
        pre = self.prefix
        q = fetch(f"{pre}.dq" if self.q_rank else f"{pre}.q")
        parts = [q]
        self.n_q = q.shape[0]
        if self.gate:
            parts.append(fetch(f"{pre}.g"))
        if self.own:
            parts.append(fetch(f"{pre}.dkv"))
            self.w_c = fetch(f"{pre}.dkv.norm").to(q.dtype).contiguous()
        # one product for the queries (or their latent), the gates and (own latents) the down projection
        self.w_in = torch.cat([t.to(q.dtype) for t in parts], dim=0).contiguous()
        if self.q_rank:
            self.w_uq = fetch(f"{pre}.uq").to(q.dtype).contiguous()
            self.w_qn = fetch(f"{pre}.dq.norm").to(q.dtype).contiguous()
        pad = self.row_len - self.rank
        uk = fetch(f"{pre}.uk").view(self.heads, self.dim, self.rank)
        uv = fetch(f"{pre}.uv").view(self.heads, self.vdim, self.rank)
        if pad:
            uk = torch.nn.functional.pad(uk, (0, pad))
            uv = torch.nn.functional.pad(uv, (0, pad))
        self.w_uk = uk.contiguous()                              # [heads, dim, row_len]: q_a -> latent space
        self.w_uv_t = uv.transpose(1, 2).contiguous()            # [heads, row_len, vdim]: latent space -> o_a
        self.w_o = fetch(f"{pre}.o").contiguous()
        if self.rot:
            self._freq = torch.from_numpy(self._freq_host).to(self.w_in.device)

    def forward(self, normed, ctx, cache):
        n = normed.shape[0]
        proj = linear(normed, self.w_in)
        block_table = ctx.block_tables[cache.group]
        if self.own != cache.writes:
            raise RuntimeError(f"{self.prefix}: a layer with its own latents writes its cache slot, another reads one")
        off_g = self.n_q
        off_kv = off_g + (self.heads if self.gate else 0)
        if self.own:
            ops.latent_append(proj[:, off_kv:], self.w_c, self.eps, ctx.positions, ctx.seq_of_token, block_table,
                              cache.k_pages, inv_freq=self._freq, interleaved=self.rot_interleaved, rot_mul=self.rot_mul)
        if self.q_rank:
            q = linear(ops.rmsnorm_rows(proj[:, : self.q_rank], self.w_qn, self.eps), self.w_uq)
        else:
            q = proj[:, : self.n_q]
        q = q.view(n, self.heads, self.qdim) if q.is_contiguous() else q.reshape(n, self.heads, self.qdim)
        # queries into latent space, head by head: [heads, N, dim] x [heads, dim, row_len]
        q_lat = torch.empty((n, self.heads, self.row_len), dtype=proj.dtype, device=proj.device)
        torch.bmm(q[:, :, : self.dim].transpose(0, 1), self.w_uk, out=q_lat.transpose(0, 1))
        if self.rot:
            # the rotated part of every head's query, turned by the token's position, behind its latent part
            ops.rope_copy(q[:, :, self.dim:], q_lat[:, :, self.rank: self.rank + self.rot], ctx.positions, self._freq,
                          interleaved=self.rot_interleaved, rot_mul=self.rot_mul)
        chunk = self.window[1] if self.window and self.window[0] == "chunk" else 0
        sliding = self.window[1] if self.window and self.window[0] == "sliding" else 0
        o_lat = attend_over_pages(q_lat, cache.k_pages, cache.k_pages, block_table, ctx, self.heads, 1, self.row_len,
                                  chunk, sliding, self.scale)
        o = torch.empty((n, self.heads, self.vdim), dtype=proj.dtype, device=proj.device)
        torch.bmm(o_lat.transpose(0, 1), self.w_uv_t, out=o.transpose(0, 1))
        if self.gate:
            o = ops.head_gate(o, proj[:, off_g: off_g + self.heads])
        return linear(o.view(n, self.heads * self.vdim), self.w_o)
