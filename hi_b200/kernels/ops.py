"""Python faces of the CUDA kernels in ``hi_b200/csrc``.

Every function takes CUDA tensors, checks shapes and dtypes, and enqueues the kernel on
torch's current stream. There is no CPU path and no torch fallback: a tensor that is not
on a CUDA device, or a library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_uint64, c_void_p
from typing import Optional, Tuple

import torch

from . import build as _build

P, I, F = c_void_p, c_int, c_float

_SIGNATURES = {
    "hb_feed_tokens": [P, P, P, P, I, P],
    "hb_embed_gather": [P, I, P, P, I, I, I, F, P],
    "hb_add_rmsnorm": [P, P, I, P, I, P, P, P, I, P, I, P, I, P, P, I, I, F, F, I, P],
    "hb_swiglu": [P, P, I, I, I, P],
    "hb_relu2": [P, I, P, I, c_longlong, P],
    "hb_softcap": [P, F, c_longlong, P],
    "hb_convert": [P, I, P, I, c_longlong, P],
    "hb_moe_combine": [P, P, P, P, I, P, I, I, I, P],
    "hb_qkv_post": [P, I, P, I, I, I, F, I, F, F, P, P, I, I, F, P, I, I, P, P, P, I, P, P, P, I, I, I, I, I, I, P],
    "hb_paged_attention": [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, F, P, P, I, I, P, P, P],
    "hb_attention_merge": [P, P, P, I, I, I, I, I, I, P, P],
    "hb_attention_decode": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P, F, P, P, I, I, P, P, P],
    "hb_attention_decode_tma": [P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P, P, P],
    "hb_attention_decode_fused": [P, P, I, I, I, F, I, F, F, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, P, P, P, P, I, F, I, P],
    "hb_attention_prefill": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P],
    "hb_attention_prefill_reshaped": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, I, F, P, P, P],
    "hb_attention_prefill_tc": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P, I, P, P, P, P],
    "hb_attention_prefill_tc_reshaped": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, F, P, P, I, P, P, P,
                                         P],
    "hb_sigmoid_prefill_tc": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P, I, I, P, P],
    "hb_sigmoid_merge": [P, P, P, I, I, P, I, I, I, I, I, P],
    "hb_router_topk": [P, I, P, I, I, I, I, I, I, F, P, P, P, P],
    "hb_moe_plan": [P, I, I, P, P, P, P, P],
    "hb_router_plan": [P, I, P, I, I, I, I, I, I, F, P, P, P, P, P, P, P, P, P],
    "hb_moe_gate_up": [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, P],
    "hb_moe_down": [P, I, P, P, P, I, P, I, I, I, I, P],
    "hb_gather_rows": [P, P, I, P, I, I, P],
    "hb_moe_gate_up_tc": [P, P, P, P, P, I, P, P, I, I, I, P, P],
    "hb_moe_down_tc": [P, P, P, I, P, I, I, I, P, c_longlong, P, I, P, P],
    "hb_moe_up_relu2_tc": [P, P, P, I, P, I, I, I, P, P],
    "hb_argmax_rows": [P, I, I, I, P, P, P, P, P],
    "hb_ranked_rows": [P, I, I, P, P, P, P, P, P],
    "hb_sample_rows": [P, I, I, P, P, P, P],
    "hb_sample_rows_parts": [P, I, I, I, P, P, P, P, P, P, P, P, P],
    "hb_random_normal": [P, I, c_longlong, c_longlong, c_uint64, F, P],
    "hb_gated_depth_dyt": [P, P, I, P, I, P, I, P, I, P, c_longlong, I, P, P, P, P, P, P, P, P, P, P, I, I, P, I, I, P],
    "hb_xielu": [P, P, I, P, c_longlong, P],
    "hb_latent_append": [P, I, c_longlong, P, F, P, P, P, I, P, I, I, I, I, P, I, I, F, P],
    "hb_rmsnorm_rows": [P, I, c_longlong, P, F, P, I, I, P],
    "hb_rope_copy": [P, c_longlong, c_longlong, P, c_longlong, c_longlong, I, P, P, I, I, I, I, F, P],
    "hb_canon_conv": [P, P, P, P, c_longlong, P, P, P, P, P, I, I, I, I, I, I, P],
    "hb_stream_add": [P, P, I, P, I, P, P, c_longlong, I, P],
    "hb_rmsnorm_mean2": [P, P, I, P, P, I, F, P, I, I, I, P],
    "hb_sigmoid_attention": [P, I, P, P, P, I, P, P, P, P, I, I, P, I, I, I, I, I, I, I, F, I, I, P, P],
    "hb_gla_prep": [P, I, c_longlong, I, I, I, P, P, F, F, P, P, P, P, I, I, I, P],
    "hb_head_gate": [P, P, c_longlong, P, I, I, I, I, P],
    "hb_delta_prep": [P, I, c_longlong, I, I, P, P, c_longlong, c_longlong, P, I, P, P, P, P, P, P, P, P, P, P, I, I, I,
                      I, I, I, I, P],
    "hb_delta_conv_update": [P, I, c_longlong, I, P, c_longlong, c_longlong, P, P, I, I, I, P],
    "hb_delta_recurrence": [P, P, P, P, P, P, c_longlong, P, P, P, I, I, I, I, I, I, I, I, P],
    "hb_delta_out_norm": [P, P, I, P, F, P, I, c_longlong, I, I, c_longlong, I, P],
    "hb_hyper_step": [P, P, P, I, P, I, P, P, P, I, P, P, F, P, P, I, F, P, I, P, P, I, I, I, P],
    "hb_hyper_sum": [P, P, I, I, I, P],
    "hb_mamba2_prep": [P, I, c_longlong, I, I, P, P, P, c_longlong, c_longlong, P, P, P, P, P, P, P, P, P, P, I, I, I, I,
                       I, I, P],
    "hb_mamba2_out": [P, P, P, I, c_longlong, P, P, F, P, I, I, I, I, I, P],
    "hb_mlstm_gates": [P, P, P, F, P, c_longlong, c_longlong, P, P, P, P, P, I, I, P],
    "hb_mlstm_recurrence": [P, I, c_longlong, I, I, I, F, P, P, P, c_longlong, P, P, P, P, I, I, I, I, I, P],
    "hb_mlstm_out_norm": [P, P, P, P, I, c_longlong, I, P, I, F, P, I, c_longlong, I, I, P],
}

_UNSUPPORTED = 1002
_ERRORS = {1001: "bad argument (size, pointer or dtype)", 1002: "shape not supported by this kernel"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        handle = _build.library()
        for name, sig in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = sig
            fn.restype = c_int
        handle.hb_moe_down_tc_scratch_floats.argtypes = [I]
        handle.hb_moe_down_tc_scratch_floats.restype = c_longlong
        _lib = handle
    return _lib


LAUNCHES = [0]     # kernels of this library enqueued so far (benchmarks report the difference)
CALLS: dict = {}   # ... and by entry point: which kernel family took the work (tests look here)


def _check(code: int, name: str) -> None:
    LAUNCHES[0] += 1
    CALLS[name] = CALLS.get(name, 0) + 1
    if code != 0:
        what = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{name}: {what}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------------- elementwise
def feed_tokens(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, sampled: torch.Tensor) -> None:
    """tokens[dst[i]] = sampled[src[i]], all int32 on the device: a step takes tokens that the step
    before it sampled without the host having read them."""
    for t, nm in ((tokens, "tokens"), (dst, "dst"), (src, "src"), (sampled, "sampled")):
        _need(t, nm, torch.int32)
    if dst.numel() != src.numel():
        raise KernelError("dst and src need the same number of entries")
    _check(lib().hb_feed_tokens(_ptr(tokens), _ptr(dst), _ptr(src), _ptr(sampled), dst.numel(), _stream()), "feed_tokens")


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None,
                 scale: float = 1.0) -> torch.Tensor:
    """Rows of ``table`` [V, H] for int32 ``tokens`` [N], times ``scale`` -> float32 residual stream [N, H]
    (into ``out`` if given)."""
    _need(table, "table"); _need(tokens, "tokens", torch.int32)
    n, (vocab, hidden) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    else:
        _need(out, "out", torch.float32)
        if tuple(out.shape) != (n, hidden):
            raise KernelError(f"out has shape {tuple(out.shape)}, expected {(n, hidden)}")
    _check(lib().hb_embed_gather(_ptr(table), _dt(table), _ptr(tokens), _ptr(out), n, hidden, vocab, float(scale), _stream()),
           "embed_gather")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                out_dtype: torch.dtype, row_map: Optional[torch.Tensor] = None, also_f32: bool = False,
                routed: Optional[torch.Tensor] = None, slot_of_entry: Optional[torch.Tensor] = None,
                top_k: int = 0, routed_weight: Optional[torch.Tensor] = None, x_scale: float = 1.0,
                post: bool = False, delta2: Optional[torch.Tensor] = None):
    """``x = x_scale * x + delta (+ delta2)`` (float32, in place) then ``rmsnorm(x) * weight`` in ``out_dtype``.
    ``delta2``: a second sub-layer result of the same shape (two sub-layers side by side on one input).

    ``post``: the norm comes after the sum in the block, so the stream itself takes the normalised rows
    (unrounded float32) instead of the sum; the returned ``y`` is the same rows in ``out_dtype``.

    ``routed`` (float32 [N*k, H], rows in expert-sorted order) with ``slot_of_entry`` adds each
    token's k routed-expert rows into the same sum: the experts' combine, fused into the norm;
    ``routed_weight`` (float32 [N*k], by entry) multiplies each of them first (a router score that
    scales the experts' outputs).

    ``also_f32`` returns ``(y, y_float32)``: the same normalised rows unrounded, for a consumer
    that computes in 32-bit (the router).

    With ``row_map`` (int32 [R]) only those rows are normalised (output [R, H]) and ``x`` is
    left untouched: the rows whose logits are wanted.
    """
    _need(x, "x", torch.float32)
    rows_total, hidden = x.shape
    if delta is not None:
        _need(delta, "delta")
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} != residual shape {tuple(x.shape)}")
    if delta2 is not None:
        _need(delta2, "delta2")
        if delta2.shape != x.shape:
            raise KernelError(f"delta2 shape {tuple(delta2.shape)} != residual shape {tuple(x.shape)}")
    if weight is not None:
        _need(weight, "weight")
        if weight.numel() != hidden:
            raise KernelError(f"norm weight has {weight.numel()} elements for hidden size {hidden}")
    rows = rows_total
    if row_map is not None:
        if post:
            raise KernelError("a norm that writes the stream works on all rows (no row_map)")
        _need(row_map, "row_map", torch.int32)
        rows = row_map.numel()
    y = torch.empty((rows, hidden), dtype=out_dtype, device=x.device)
    y32 = None
    if also_f32 and out_dtype != torch.float32:
        y32 = torch.empty((rows, hidden), dtype=torch.float32, device=x.device)
    if routed is not None:
        _need(routed, "routed", torch.float32); _need(slot_of_entry, "slot_of_entry", torch.int32)
        if routed.shape[1] != hidden or not 1 <= top_k <= 8:
            raise KernelError("routed rows do not match the residual, or top_k is outside 1..8")
        if routed_weight is not None:
            _need(routed_weight, "routed_weight", torch.float32)
            if routed_weight.numel() != slot_of_entry.numel():
                raise KernelError("routed_weight needs one factor per routing entry")
    _check(lib().hb_add_rmsnorm(_ptr(x), _ptr(delta), _dt(delta) if delta is not None else 0,
                                _ptr(delta2), _dt(delta2) if delta2 is not None else 0, _ptr(routed),
                                _ptr(slot_of_entry), _ptr(routed_weight) if routed is not None else None, int(top_k),
                                _ptr(weight),
                                _dt(weight) if weight is not None else 0, _ptr(y), _dt(y), _ptr(y32), _ptr(row_map),
                                rows, hidden, float(eps), float(x_scale), 1 if post else 0, _stream()), "add_rmsnorm")
    if also_f32:
        return y, (y if y32 is None else y32)
    return y


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """[N, 2I] (gate columns first) -> silu(gate) * up, [N, I], same dtype, float32 math."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("swiglu input needs an even number of columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib().hb_swiglu(_ptr(gate_up), _ptr(out), _dt(gate_up), n, two_i // 2, _stream()), "swiglu")
    return out


def relu2(x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """max(x, 0)^2 in float32 math; the result in ``out_dtype`` (default: x's)."""
    _need(x, "x")
    out = torch.empty_like(x, dtype=out_dtype or x.dtype)
    _check(lib().hb_relu2(_ptr(x), _dt(x), _ptr(out), _dt(out), x.numel(), _stream()), "relu2")
    return out


def convert(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """A copy of ``x`` in ``out_dtype`` (float32 or bfloat16, rounded to nearest even)."""
    _need(x, "x")
    out = torch.empty_like(x, dtype=out_dtype)
    _check(lib().hb_convert(_ptr(x), _dt(x), _ptr(out), _dt(out), x.numel(), _stream()), "convert")
    return out


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), float32, in place."""
    _need(x, "x", torch.float32)
    _check(lib().hb_softcap(_ptr(x), float(cap), x.numel(), _stream()), "softcap")
    return x


# --------------------------------------------------------------------------- gated parallel block
def gated_depth_dyt(x: torch.Tensor, terms, history: Optional[torch.Tensor], n_prev: int,
                    mix: Optional[torch.Tensor], norms, out_dtype: torch.dtype,
                    row_map: Optional[torch.Tensor] = None, want_z: bool = True):
    """One pass over the rows of the float32 stream ``x`` [N, W]:

        s = x + sum_k sigmoid(gate_k) * delta_k      ``terms``: up to two (delta, gate | None), [N, W] each
        history[n_prev] = s                          ``history`` float32 [entries, N, W] (None: not kept)
        z = sum_{j <= n_prev} mix[j] * history[j]    ``mix`` float32 [n_prev + 1] (None: z = s)
        y_k = tanh(alpha_k z) w_k + b_k              ``norms``: up to two (alpha float32 [1], w [W], b [W])

    Returns ``(z | None, [y_k])``; ``y_k`` in ``out_dtype``. With ``row_map`` (int32 [R]) only those rows are
    worked out (outputs [R, W]) and the history is read but not extended."""
    _need(x, "x", torch.float32)
    n, width = x.shape
    terms = list(terms) + [(None, None)] * (2 - len(terms))
    norms = list(norms) + [None] * (2 - len(norms))
    if len(terms) > 2 or len(norms) > 2:
        raise KernelError("at most two gated terms and two norms")
    for d, g in terms:
        for t, nm in ((d, "delta"), (g, "gate")):
            if t is not None:
                _need(t, nm)
                if tuple(t.shape) != (n, width):
                    raise KernelError(f"{nm} has shape {tuple(t.shape)}, the stream {(n, width)}")
        if d is None and g is not None:
            raise KernelError("a gate without its term")
    if history is not None:
        _need(history, "history", torch.float32)
        if history.dim() != 3 or tuple(history.shape[1:]) != (n, width) or not 0 <= n_prev < history.shape[0]:
            raise KernelError(f"history {tuple(history.shape)} does not take entry {n_prev} of a {(n, width)} stream")
    if mix is not None:
        _need(mix, "mix", torch.float32)
        if history is None or mix.numel() != n_prev + 1:
            raise KernelError(f"mix has {mix.numel()} weights for {n_prev + 1} results")
    rows = n
    if row_map is not None:
        _need(row_map, "row_map", torch.int32)
        rows = row_map.numel()
    wb_dtype = None
    for nrm in norms:
        if nrm is None:
            continue
        alpha, w, b = nrm
        _need(alpha, "alpha", torch.float32); _need(w, "norm weight"); _need(b, "norm bias", w.dtype)
        if w.numel() != width or b.numel() != width or alpha.numel() != 1:
            raise KernelError("norm tensors do not match the stream's width")
        if wb_dtype is not None and w.dtype != wb_dtype:
            raise KernelError("the two norms need one dtype")
        wb_dtype = w.dtype
    z = torch.empty((rows, width), dtype=torch.float32, device=x.device) if want_z else None
    ys = [None if nrm is None else torch.empty((rows, width), dtype=out_dtype, device=x.device) for nrm in norms]
    dt = lambda t: 0 if t is None else _dt(t)
    (d0, g0), (d1, g1) = terms
    a = [(None, None, None) if nrm is None else nrm for nrm in norms]
    _check(lib().hb_gated_depth_dyt(
        _ptr(x), _ptr(d0), dt(d0), _ptr(g0), dt(g0), _ptr(d1), dt(d1), _ptr(g1), dt(g1),
        _ptr(history), n * width, int(n_prev), _ptr(mix), _ptr(z),
        _ptr(a[0][0]), _ptr(a[0][1]), _ptr(a[0][2]), _ptr(ys[0]), _ptr(a[1][0]), _ptr(a[1][1]), _ptr(a[1][2]), _ptr(ys[1]),
        0 if wb_dtype is None else (0 if wb_dtype == torch.float32 else 1), 0 if out_dtype == torch.float32 else 1,
        _ptr(row_map), rows, width, _stream()), "gated_depth_dyt")
    return z, [y for y in ys if y is not None]


def xielu(x: torch.Tensor, coef: torch.Tensor) -> torch.Tensor:
    """z > 0: a z^2 + z/2;  z <= 0: c (e^z - 1 - z) + z/2, with ``coef`` = (a, c) float32; same dtype out."""
    _need(x, "x"); _need(coef, "coef", torch.float32)
    if coef.numel() != 2:
        raise KernelError("xielu needs two coefficients")
    out = torch.empty_like(x)
    _check(lib().hb_xielu(_ptr(x), _ptr(out), _dt(x), _ptr(coef), x.numel(), _stream()), "xielu")
    return out


# --------------------------------------------------------------------------- latent attention
def _row_strided(t: torch.Tensor, name: str) -> int:
    """A 2-D view whose rows are contiguous runs (a column slice of a contiguous matrix); its row stride."""
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no CPU path")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be a matrix with contiguous rows")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def latent_append(x: torch.Tensor, weight: torch.Tensor, eps: float, positions: torch.Tensor,
                  seq_of_token: torch.Tensor, block_table: torch.Tensor, pages: torch.Tensor,
                  inv_freq: Optional[torch.Tensor] = None, interleaved: bool = False, rot_mul: float = 1.0) -> None:
    """pages[page of token, 0, place, :rank] = x / sqrt(mean(x^2) + eps) * weight for every token's row of
    ``x`` [N, rank] (rows may be a column slice of a wider matrix); ``pages`` [P, 1, page_size, row_len >= rank],
    the rest of a row is zero-filled. Statistics in float32.

    With ``inv_freq`` (float32 [pairs]) ``x`` is [N, rank + 2 * pairs]: the columns behind the latent are a key
    part that is not normed but rotated by the token's position (pairs (i, i + pairs), or (2i, 2i + 1) with
    ``interleaved``; cos and sin times ``rot_mul``) and written behind the latent in the page row."""
    stride = _row_strided(x, "x")
    _need(weight, "weight", x.dtype); _need(pages, "pages", x.dtype)
    for t, nm in ((positions, "positions"), (seq_of_token, "seq_of_token"), (block_table, "block_table")):
        _need(t, nm, torch.int32)
    pairs = 0
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        pairs = inv_freq.numel()
    n, rank = x.shape[0], x.shape[1] - 2 * pairs
    if rank <= 0 or pages.dim() != 4 or pages.shape[1] != 1 or pages.shape[3] < x.shape[1] or weight.numel() != rank:
        raise KernelError(f"pages {tuple(pages.shape)} / weight do not take latents of {rank} (+ {2 * pairs} rotated)")
    _check(lib().hb_latent_append(_ptr(x), _dt(x), stride, _ptr(weight), float(eps), _ptr(positions), _ptr(seq_of_token),
                                  _ptr(block_table), block_table.shape[1], _ptr(pages), pages.shape[2], rank,
                                  pages.shape[3], n, _ptr(inv_freq), pairs, int(interleaved), float(rot_mul), _stream()),
           "latent_append")


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight row by row (statistics in float32); ``x`` [N, W] may be a column slice
    of a wider matrix. The result is contiguous, of x's dtype."""
    stride = _row_strided(x, "x")
    _need(weight, "weight", x.dtype)
    n, width = x.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} elements for rows of {width}")
    out = torch.empty((n, width), dtype=x.dtype, device=x.device)
    _check(lib().hb_rmsnorm_rows(_ptr(x), _dt(x), stride, _ptr(weight), float(eps), _ptr(out), n, width, _stream()),
           "rmsnorm_rows")
    return out


def rope_copy(src: torch.Tensor, dst: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor,
              interleaved: bool = False, rot_mul: float = 1.0) -> None:
    """dst[t, h, :2p] = src[t, h, :2p] rotated by positions[t] (p = len(inv_freq) pairs; (i, i + p), or
    (2i, 2i + 1) with ``interleaved``; cos and sin times ``rot_mul``). ``src`` and ``dst`` are [N, heads, >= 2p] views whose last axis is
    contiguous (slices of wider tensors), of one dtype; they may be the same memory."""
    _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    pairs = inv_freq.numel()
    for t, nm in ((src, "src"), (dst, "dst")):
        if not t.is_cuda or t.dim() != 3 or t.shape[2] < 2 * pairs or (t.shape[2] > 1 and t.stride(2) != 1):
            raise KernelError(f"{nm} must be a CUDA view [N, heads, >= {2 * pairs}] with a contiguous last axis")
    if src.dtype != dst.dtype or src.shape[:2] != dst.shape[:2] or positions.numel() != src.shape[0]:
        raise KernelError("src and dst need one dtype and the same tokens and heads")
    _check(lib().hb_rope_copy(_ptr(src), src.stride(0), src.stride(1), _ptr(dst), dst.stride(0), dst.stride(1), _dt(src),
                              _ptr(positions), _ptr(inv_freq), src.shape[0], src.shape[1], pairs, int(interleaved),
                              float(rot_mul), _stream()), "rope_copy")


# --------------------------------------------------------------------------- convolved norm output, passes, two mixers
def canon_conv(h: torch.Tensor, taps_a: torch.Tensor, taps_b: Optional[torch.Tensor], state: torch.Tensor,
               cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, out_dtype: torch.dtype,
               update_state: bool = True, single_tokens: bool = False):
    """y[t] = h[t] + sum_j taps[:, j] * h[t - (K-1) + j] over time within each request, for ``taps_a`` and (if
    given) ``taps_b`` (float32 [W, K]); ``h`` float32 [N, W]. Rows before a portion's first token come from
    ``state[slot]`` (float32 [K-1, W] flat: the last K-1 rows of h the request has seen; zeros at its start),
    which then takes the portion's last rows (``single_tokens``: every request brings exactly one row, and the
    kernel moves the state itself instead of a second launch). Returns (y_a, y_b | None) in ``out_dtype``."""
    _need(h, "h", torch.float32); _need(taps_a, "taps_a", torch.float32); _need(state, "state", torch.float32)
    for t, nm in ((cu_seqlens, "cu_seqlens"), (seq_of_token, "seq_of_token"), (slots, "slots")):
        _need(t, nm, torch.int32)
    n, width = h.shape
    k = taps_a.shape[1]
    if tuple(taps_a.shape) != (width, k) or (taps_b is not None and taps_b.shape != taps_a.shape):
        raise KernelError("taps must be [width, K]")
    if taps_b is not None:
        _need(taps_b, "taps_b", torch.float32)
    if state.dim() != 2 or state.shape[1] < (k - 1) * width:
        raise KernelError("the state does not hold K-1 rows of the width")
    out_a = torch.empty((n, width), dtype=out_dtype, device=h.device)
    out_b = torch.empty_like(out_a) if taps_b is not None else None
    _check(lib().hb_canon_conv(_ptr(h), _ptr(taps_a), _ptr(taps_b), _ptr(state), state.shape[1], _ptr(cu_seqlens),
                               _ptr(seq_of_token), _ptr(slots), _ptr(out_a), _ptr(out_b), _dt(out_a), n, slots.numel(),
                               width, k, (2 if single_tokens and n < 1024 else 1) if update_state else 0, _stream()),
           "canon_conv")
    if update_state and k > 1 and not (single_tokens and n < 1024):
        LAUNCHES[0] += 1
    return out_a, out_b


def stream_add(x: torch.Tensor, d1: Optional[torch.Tensor] = None, d2: Optional[torch.Tensor] = None,
               rows_f32: Optional[torch.Tensor] = None, vector: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x += d1 + d2 + rows_f32 + vector (broadcast over rows), in place on the float32 stream [N, W]; any term
    may be absent. ``d1``/``d2`` [N, W] float32 or bfloat16, ``rows_f32`` float32 [N, W], ``vector`` float32 [W]."""
    _need(x, "x", torch.float32)
    n, width = x.shape
    for t, nm in ((d1, "d1"), (d2, "d2")):
        if t is not None:
            _need(t, nm)
            if t.shape != x.shape:
                raise KernelError(f"{nm} does not match the stream")
    if rows_f32 is not None:
        _need(rows_f32, "rows_f32", torch.float32)
        if rows_f32.shape != x.shape:
            raise KernelError("rows_f32 does not match the stream")
    if vector is not None:
        _need(vector, "vector", torch.float32)
        if vector.numel() != width:
            raise KernelError("vector needs one entry per column")
    _check(lib().hb_stream_add(_ptr(x), _ptr(d1), _dt(d1) if d1 is not None else 0, _ptr(d2),
                               _dt(d2) if d2 is not None else 0, _ptr(rows_f32), _ptr(vector), n, width, _stream()),
           "stream_add")
    return x


def rmsnorm_mean2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float,
                  out_dtype: torch.dtype) -> torch.Tensor:
    """(a / rms(a) * wa + b / rms(b) * wb) / 2 row by row, statistics in float32; a, b [N, W] of one dtype."""
    _need(a, "a"); _need(b, "b", a.dtype); _need(wa, "wa"); _need(wb, "wb", wa.dtype)
    n, width = a.shape
    if b.shape != a.shape or wa.numel() != width or wb.numel() != width:
        raise KernelError("the two inputs and their weights must match")
    out = torch.empty((n, width), dtype=out_dtype, device=a.device)
    _check(lib().hb_rmsnorm_mean2(_ptr(a), _ptr(b), _dt(a), _ptr(wa), _ptr(wb), _dt(wa), float(eps), _ptr(out), _dt(out),
                                  n, width, _stream()), "rmsnorm_mean2")
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x [N, heads, dim] * sigmoid(gate [N, heads]) per (token, head); ``gate`` may be a column slice."""
    _need(x, "x")
    stride = _row_strided(gate, "gate")
    n, heads, dim = x.shape
    if gate.dtype != x.dtype or tuple(gate.shape) != (n, heads):
        raise KernelError("gate must be [N, heads] of x's dtype")
    out = torch.empty_like(x)
    _check(lib().hb_head_gate(_ptr(x), _ptr(gate), stride, _ptr(out), _dt(x), n, heads, dim, _stream()), "head_gate")
    return out


# --------------------------------------------------------------------------- gated delta rule
def delta_prep(proj: torch.Tensor, chan_off: int, beta_off: int, taps: torch.Tensor, state: torch.Tensor,
               conv_off: int, a_pre: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor,
               cu_seqlens: torch.Tensor, seq_of_token: torch.Tensor, slots: torch.Tensor, heads: int, kvh: int,
               dim: int, vdim: int, head_decay: bool = False):
    """Per token: causal convolution over time (``taps`` float32 [C, K], last column = the token itself) and
    silu of the C = 2*kvh*dim + heads*vdim channels q | k | v that start at column ``chan_off`` of ``proj``
    [N, ld]; rows before a portion's first token come from ``state[slot, conv_off:]`` ([K-1, C] float32);
    q and k to unit length per head (q also * dim^-1/2); beta = sigmoid(proj[:, beta_off + h]);
    decay = exp(-exp(a_log[h]) * softplus(a_pre + dt_bias)). Returns float32 (q, k, v, beta, decay).
    ``head_decay``: one decay per head (``a_pre`` [N, heads], ``dt_bias`` [heads]), written out for every key
    channel of the head, so ``decay`` is [N, heads * dim] either way."""
    _need(proj, "proj"); _need(taps, "taps", torch.float32); _need(state, "state", torch.float32)
    _need(a_pre, "a_pre"); _need(dt_bias, "dt_bias", torch.float32); _need(a_log, "a_log", torch.float32)
    for t, nm in ((cu_seqlens, "cu_seqlens"), (seq_of_token, "seq_of_token"), (slots, "slots")):
        _need(t, nm, torch.int32)
    n, ld = proj.shape
    c = 2 * kvh * dim + heads * vdim
    k_taps = taps.shape[1]
    if tuple(taps.shape) != (c, k_taps) or chan_off + c > ld or beta_off + heads > ld:
        raise KernelError("taps / column offsets do not fit the projection")
    per = heads if head_decay else heads * dim
    if tuple(a_pre.shape) != (n, per) or dt_bias.numel() != per or a_log.numel() != heads:
        raise KernelError("decay inputs do not match heads (x dim)")
    if state.dim() != 2 or conv_off + (k_taps - 1) * c > state.shape[1]:
        raise KernelError("the state does not hold the convolution's inputs")
    dev, f32 = proj.device, torch.float32
    q = torch.empty((n, kvh * dim), dtype=f32, device=dev)
    k = torch.empty((n, kvh * dim), dtype=f32, device=dev)
    v = torch.empty((n, heads * vdim), dtype=f32, device=dev)
    beta = torch.empty((n, heads), dtype=f32, device=dev)
    decay = torch.empty((n, heads * dim), dtype=f32, device=dev)
    _check(lib().hb_delta_prep(_ptr(proj), _dt(proj), ld, int(chan_off), int(beta_off), _ptr(taps), _ptr(state),
                               state.shape[1], int(conv_off), _ptr(a_pre), _dt(a_pre), _ptr(dt_bias), _ptr(a_log),
                               _ptr(cu_seqlens), _ptr(seq_of_token), _ptr(slots), _ptr(q), _ptr(k), _ptr(v), _ptr(beta),
                               _ptr(decay), n, heads, kvh, dim, vdim, k_taps, int(head_decay), _stream()), "delta_prep")
    return q, k, v, beta, decay


def delta_conv_update(proj: torch.Tensor, chan_off: int, channels: int, taps_n: int, state: torch.Tensor,
                      conv_off: int, cu_seqlens: torch.Tensor, slots: torch.Tensor) -> None:
    """state[slot, conv_off:] <- the last K-1 convolution inputs of every request after this step's rows."""
    _need(proj, "proj"); _need(state, "state", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(slots, "slots", torch.int32)
    if chan_off + channels > proj.shape[1] or conv_off + (taps_n - 1) * channels > state.shape[1]:
        raise KernelError("channels do not fit the projection or the state")
    _check(lib().hb_delta_conv_update(_ptr(proj), _dt(proj), proj.shape[1], int(chan_off), _ptr(state), state.shape[1],
                                      int(conv_off), _ptr(cu_seqlens), _ptr(slots), slots.numel(), channels, taps_n,
                                      _stream()), "delta_conv_update")


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: Optional[torch.Tensor],
                     decay: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, heads: int,
                     kvh: int, dim: int, vdim: int, general: bool = False, rows: int = 0, single_tokens: bool = False,
                     plain: bool = False) -> torch.Tensor:
    """Token after token per request and head, on ``state[slot, :heads*dim*vdim]`` ([heads, dim, vdim] float32):
    S <- decay * S (per row); u = beta (v - S^T k); S <- S + k u^T; o = S^T q. Returns o float32 [N, heads*vdim].
    ``general`` forces the kernel that keeps S in shared memory (any dim) instead of registers (dim <= 256);
    ``rows`` (16, 32) forces how many rows of a column a lane holds, else ``single_tokens`` (every request
    brings one token) decides: the order of the sums differs between the forms, by rounding only.
    ``plain``: the rule without the correction, S <- decay * S + k v^T; o = S^T q (``beta`` is not read)."""
    for t, nm in ((q, "q"), (k, "k"), (v, "v"), (decay, "decay"), (state, "state")) + (() if plain else ((beta, "beta"),)):
        _need(t, nm, torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(slots, "slots", torch.int32)
    n = q.shape[0]
    if tuple(q.shape) != (n, kvh * dim) or tuple(k.shape) != (n, kvh * dim) or tuple(v.shape) != (n, heads * vdim) or \
            (not plain and tuple(beta.shape) != (n, heads)) or tuple(decay.shape) != (n, heads * dim):
        raise KernelError("q / k / v / beta / decay do not match the head sizes")
    if state.dim() != 2 or state.shape[1] < heads * dim * vdim or cu_seqlens.numel() != slots.numel() + 1:
        raise KernelError("the state or the request tables do not fit")
    out = torch.empty((n, heads * vdim), dtype=torch.float32, device=q.device)
    _check(lib().hb_delta_recurrence(_ptr(q), _ptr(k), _ptr(v), None if plain else _ptr(beta), _ptr(decay), _ptr(state),
                                     state.shape[1], _ptr(cu_seqlens), _ptr(slots), _ptr(out), slots.numel(), heads, kvh,
                                     dim, vdim, 1 if general else int(rows), int(single_tokens), int(plain), _stream()),
           "delta_recurrence")
    return out


def delta_out_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, vdim: int,
                   out_dtype: torch.dtype, gate_silu: bool = False) -> torch.Tensor:
    """o [N, heads*vdim] float32 -> o / sqrt(mean over each head's vdim (o^2) + eps) * weight[vdim] *
    sigmoid(gate) (``gate_silu``: * gate sigmoid(gate)), in ``out_dtype``. ``gate`` may be a column slice."""
    _need(o, "o", torch.float32); _need(weight, "weight", out_dtype)
    gate_stride = _row_strided(gate, "gate")
    if o.shape != gate.shape or o.shape[1] % vdim or weight.numel() != vdim:
        raise KernelError("gate / weight do not match the heads' value size")
    out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    _check(lib().hb_delta_out_norm(_ptr(o), _ptr(gate), _dt(gate), _ptr(weight), float(eps), _ptr(out), _dt(out),
                                   o.numel() // vdim, vdim, int(gate_silu), gate_stride, o.shape[1] // vdim, _stream()),
           "delta_out_norm")
    return out


def gla_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, z: torch.Tensor, bias: Optional[torch.Tensor],
             tau: float, q_scale: float, qk_cols: int, v_cols: int):
    """Inputs of the recurrence without correction from a projection's columns: q * q_scale, k [N, qk_cols] and
    v [N, v_cols] as float32, and decay = sigmoid(z + bias)^(1 / tau) [N, qk_cols] (``z`` float32)."""
    _need(proj, "proj"); _need(z, "z", torch.float32)
    n, ld = proj.shape
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != qk_cols:
            raise KernelError("one bias per key channel")
    if tuple(z.shape) != (n, qk_cols) or max(q_off, k_off) + qk_cols > ld or v_off + v_cols > ld:
        raise KernelError("columns do not fit the projection")
    dev, f32 = proj.device, torch.float32
    q = torch.empty((n, qk_cols), dtype=f32, device=dev)
    k = torch.empty((n, qk_cols), dtype=f32, device=dev)
    v = torch.empty((n, v_cols), dtype=f32, device=dev)
    decay = torch.empty((n, qk_cols), dtype=f32, device=dev)
    _check(lib().hb_gla_prep(_ptr(proj), _dt(proj), ld, int(q_off), int(k_off), int(v_off), _ptr(z), _ptr(bias),
                             float(tau), float(q_scale), _ptr(q), _ptr(k), _ptr(v), _ptr(decay), n, qk_cols, v_cols,
                             _stream()), "gla_prep")
    return q, k, v, decay


# --------------------------------------------------------------------------- a residual stream of several copies
def hyper_step(streams: torch.Tensor, weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
               x_in: Optional[torch.Tensor] = None, delta: Optional[torch.Tensor] = None,
               delta2: Optional[torch.Tensor] = None, routed: Optional[torch.Tensor] = None,
               slot_of_entry: Optional[torch.Tensor] = None, top_k: int = 0,
               routed_weight: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
               out_coef: Optional[torch.Tensor] = None, mult: float = 1.0, in_coef: Optional[torch.Tensor] = None,
               row_map: Optional[torch.Tensor] = None, also_f32: bool = False):
    """One sub-layer boundary of a residual stream kept as S copies per token (``streams`` float32 [N, S, W], in place).

    The result the sub-layer before left (``delta`` + ``delta2`` + the routed rows, as in :func:`add_rmsnorm`) enters
    every copy while the copies are mixed: x_t <- sum_s mix[s, t] x_s + mult * out_coef[t] * y (``mix`` None: the
    copies stay). Then u = sum_s in_coef[s] x_s (``in_coef`` None: the plain sum) and the result is
    u * rsqrt(mean(u^2) + eps) * weight in ``out_dtype`` (with ``also_f32`` a pair: rounded, unrounded).
    ``x_in`` (float32 [N, W]): the copies do not exist yet, every one of them is ``x_in``'s row, and they are written.
    ``row_map`` (int32 [R]): only those rows, output [R, W], nothing written back."""
    _need(streams, "streams", torch.float32)
    if streams.dim() != 3:
        raise KernelError("streams must be [tokens, copies, width]")
    n, s_n, width = streams.shape
    for t, nm in ((delta, "delta"), (delta2, "delta2")):
        if t is not None:
            _need(t, nm)
            if tuple(t.shape) != (n, width):
                raise KernelError(f"{nm} shape {tuple(t.shape)} does not match {n} tokens of width {width}")
    if x_in is not None:
        _need(x_in, "x_in", torch.float32)
        if tuple(x_in.shape) != (n, width):
            raise KernelError("x_in does not match the streams")
    if mix is not None:
        _need(mix, "mix", torch.float32); _need(out_coef, "out_coef", torch.float32)
        if tuple(mix.shape) != (s_n, s_n) or out_coef.numel() != s_n:
            raise KernelError("mix / out_coef do not match the number of copies")
    elif delta is not None or delta2 is not None or routed is not None:
        raise KernelError("a sub-layer result needs the coefficients it enters the copies with")
    if in_coef is not None:
        _need(in_coef, "in_coef", torch.float32)
        if in_coef.numel() != s_n:
            raise KernelError("in_coef does not match the number of copies")
    if weight is not None:
        _need(weight, "weight")
        if weight.numel() != width:
            raise KernelError(f"norm weight has {weight.numel()} elements for width {width}")
    if routed is not None:
        _need(routed, "routed", torch.float32); _need(slot_of_entry, "slot_of_entry", torch.int32)
        if routed.shape[1] != width or top_k < 1 or slot_of_entry.numel() != n * top_k:
            raise KernelError("routed rows do not match the streams")
        if routed_weight is not None:
            _need(routed_weight, "routed_weight", torch.float32)
            if routed_weight.numel() != slot_of_entry.numel():
                raise KernelError("routed_weight needs one factor per routing entry")
    rows = n
    if row_map is not None:
        _need(row_map, "row_map", torch.int32)
        rows = row_map.numel()
    y = torch.empty((rows, width), dtype=out_dtype, device=streams.device)
    y32 = torch.empty((rows, width), dtype=torch.float32, device=streams.device) \
        if also_f32 and out_dtype != torch.float32 else None
    _check(lib().hb_hyper_step(_ptr(streams), _ptr(x_in), _ptr(delta), _dt(delta) if delta is not None else 0,
                               _ptr(delta2), _dt(delta2) if delta2 is not None else 0, _ptr(routed),
                               _ptr(slot_of_entry) if routed is not None else None,
                               _ptr(routed_weight) if routed is not None else None, int(top_k), _ptr(mix),
                               _ptr(out_coef), float(mult), _ptr(in_coef), _ptr(weight),
                               _dt(weight) if weight is not None else 0, float(eps), _ptr(y), _dt(y), _ptr(y32),
                               _ptr(row_map), rows, s_n, width, _stream()), "hyper_step")
    if also_f32:
        return y, (y if y32 is None else y32)
    return y


def hyper_sum(streams: torch.Tensor) -> torch.Tensor:
    """The sum of the copies of a residual stream: float32 [N, S, W] -> [N, W]."""
    _need(streams, "streams", torch.float32)
    n, s_n, width = streams.shape
    out = torch.empty((n, width), dtype=torch.float32, device=streams.device)
    _check(lib().hb_hyper_sum(_ptr(streams), _ptr(out), n, s_n, width, _stream()), "hyper_sum")
    return out


# --------------------------------------------------------------------------- Mamba-2 around its recurrence
def mamba2_prep(proj: torch.Tensor, chan_off: int, dt_off: int, taps: torch.Tensor, conv_bias: Optional[torch.Tensor],
                state: torch.Tensor, conv_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor, cu_seqlens: torch.Tensor,
                seq_of_token: torch.Tensor, slots: torch.Tensor, heads: int, groups: int, n_state: int, vdim: int):
    """Per token, from a projection row laid out [... x | B | C ... dt ...] (``chan_off``: first column of the
    C = heads*vdim + 2*groups*n_state convolved channels; ``dt_off``: of the heads' step sizes): causal convolution
    over time (``taps`` float32 [C, K], last column the token's own; ``conv_bias`` [C]) and silu, rows before a
    portion's first token from ``state[slot, conv_off:]`` ([K-1, C] float32); dt = softplus(dt + dt_bias);
    decay = exp(-exp(a_log[h]) * dt) written out per state channel. Returns float32
    (x [N, heads*vdim], v = dt * x, k = B [N, groups*n_state], q = C, decay [N, heads*n_state])."""
    _need(proj, "proj"); _need(taps, "taps", torch.float32); _need(state, "state", torch.float32)
    _need(dt_bias, "dt_bias", torch.float32); _need(a_log, "a_log", torch.float32)
    for t, nm in ((cu_seqlens, "cu_seqlens"), (seq_of_token, "seq_of_token"), (slots, "slots")):
        _need(t, nm, torch.int32)
    n, ld = proj.shape
    inner, gn = heads * vdim, groups * n_state
    c = inner + 2 * gn
    k_taps = taps.shape[1]
    if tuple(taps.shape) != (c, k_taps) or chan_off + c > ld or dt_off + heads > ld:
        raise KernelError("taps / column offsets do not fit the projection")
    if conv_bias is not None:
        _need(conv_bias, "conv_bias", torch.float32)
        if conv_bias.numel() != c:
            raise KernelError("one convolution bias per channel")
    if dt_bias.numel() != heads or a_log.numel() != heads or heads % groups:
        raise KernelError("dt_bias / a_log / groups do not match the heads")
    if state.dim() != 2 or conv_off + (k_taps - 1) * c > state.shape[1]:
        raise KernelError("the state does not hold the convolution's inputs")
    dev, f32 = proj.device, torch.float32
    x = torch.empty((n, inner), dtype=f32, device=dev)
    v = torch.empty((n, inner), dtype=f32, device=dev)
    k = torch.empty((n, gn), dtype=f32, device=dev)
    q = torch.empty((n, gn), dtype=f32, device=dev)
    decay = torch.empty((n, heads * n_state), dtype=f32, device=dev)
    _check(lib().hb_mamba2_prep(_ptr(proj), _dt(proj), ld, int(chan_off), int(dt_off), _ptr(taps), _ptr(conv_bias),
                                _ptr(state), state.shape[1], int(conv_off), _ptr(dt_bias), _ptr(a_log), _ptr(cu_seqlens),
                                _ptr(seq_of_token), _ptr(slots), _ptr(x), _ptr(v), _ptr(k), _ptr(q), _ptr(decay), n, heads,
                                groups, n_state, vdim, k_taps, _stream()), "mamba2_prep")
    return x, v, k, q, decay


def mamba2_out(o: torch.Tensor, x: torch.Tensor, z: torch.Tensor, d_skip: torch.Tensor, weight: torch.Tensor, eps: float,
               heads: int, vdim: int, parts: int, out_dtype: torch.dtype) -> torch.Tensor:
    """y = (o + d_skip[head] * x) * silu(z), RMS-normed in ``parts`` equal runs of channels (each by its own root
    mean square), times ``weight`` [heads*vdim], in ``out_dtype``. ``o``, ``x`` float32 [N, heads*vdim]; ``z`` may be
    a column slice of a wider matrix."""
    _need(o, "o", torch.float32); _need(x, "x", torch.float32); _need(d_skip, "d_skip", torch.float32)
    _need(weight, "weight", out_dtype)
    z_stride = _row_strided(z, "z")
    inner = heads * vdim
    if o.shape != x.shape or o.shape[1] != inner or z.shape != o.shape or d_skip.numel() != heads or \
            weight.numel() != inner or inner % parts:
        raise KernelError("o / x / z / d_skip / weight do not match the heads, or the parts do not divide the channels")
    out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    _check(lib().hb_mamba2_out(_ptr(o), _ptr(x), _ptr(z), _dt(z), z_stride, _ptr(d_skip), _ptr(weight), float(eps),
                               _ptr(out), _dt(out), o.shape[0], heads, vdim, int(parts), _stream()), "mamba2_out")
    return out


# --------------------------------------------------------------------------- mLSTM matrix memory
def mlstm_state_floats(heads: int, dim: int, vdim: int) -> int:
    """Floats of a request's state row: S column by column with n as one more column, then m per head."""
    return heads * (vdim + 1) * dim + heads


def mlstm_gates(z: torch.Tensor, bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor], cap: float,
                state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor, heads: int, dim: int, vdim: int):
    """From the gates' pre-activations ``z`` float32 [N, 2 * heads] (input gates, then forget gates):
    i = cap tanh((z_i + b_i) / cap), f = logsigmoid(cap tanh((z_f + b_f) / cap)), the running maximum
    m' = max(f + m, i) token after token from the request's state (which takes the last m), and per
    (token, head) ``keep`` = e^(f + m - m'), ``take`` = e^(i - m'), ``floor`` = e^(-m'), float32 [N, heads]."""
    _need(z, "z", torch.float32); _need(state, "state", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(slots, "slots", torch.int32)
    n = z.shape[0]
    if z.shape[1] != 2 * heads or state.dim() != 2 or state.shape[1] < mlstm_state_floats(heads, dim, vdim):
        raise KernelError("gate pre-activations or the state row do not match the heads and sizes")
    for b in (bias_i, bias_f):
        if b is not None:
            _need(b, "gate bias", torch.float32)
            if b.numel() != heads:
                raise KernelError("a gate bias has one number per head")
    keep, take, floor = (torch.empty((n, heads), dtype=torch.float32, device=z.device) for _ in range(3))
    _check(lib().hb_mlstm_gates(_ptr(z), _ptr(bias_i), _ptr(bias_f), float(cap), _ptr(state), state.stride(0),
                                heads * (vdim + 1) * dim, _ptr(cu_seqlens), _ptr(slots), _ptr(keep), _ptr(take),
                                _ptr(floor), slots.numel(), heads, _stream()), "mlstm_gates")
    return keep, take, floor


def mlstm_recurrence(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, q_scale: float, keep: torch.Tensor,
                     take: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, slots: torch.Tensor,
                     heads: int, dim: int, vdim: int, rows_per_lane: int = 0):
    """S <- keep S + take k v^T and n <- keep n + take k token after token, from and into the requests' state
    rows; q, k [heads, dim] and v [heads, vdim] of a token are column runs of ``proj`` [N, ld] at the given
    offsets, q times ``q_scale``. Returns S^T q float32 [N, heads, vdim] and n . q float32 [N, heads]."""
    _need(proj, "proj"); _need(keep, "keep", torch.float32); _need(take, "take", torch.float32)
    _need(state, "state", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(slots, "slots", torch.int32)
    n, ld = proj.shape
    if max(q_off + heads * dim, k_off + heads * dim, v_off + heads * vdim) > ld or tuple(keep.shape) != (n, heads):
        raise KernelError("the projection's columns or the gates do not match the heads and sizes")
    if state.dim() != 2 or state.shape[1] < mlstm_state_floats(heads, dim, vdim):
        raise KernelError("the state row is too short for this memory")
    o = torch.empty((n, heads, vdim), dtype=torch.float32, device=proj.device)
    nq = torch.empty((n, heads), dtype=torch.float32, device=proj.device)
    _check(lib().hb_mlstm_recurrence(_ptr(proj), _dt(proj), ld, q_off, k_off, v_off, float(q_scale), _ptr(keep),
                                     _ptr(take), _ptr(state), state.stride(0), _ptr(cu_seqlens), _ptr(slots), _ptr(o),
                                     _ptr(nq), slots.numel(), heads, dim, vdim, int(rows_per_lane), _stream()),
           "mlstm_recurrence")
    return o, nq


def mlstm_out_norm(o: torch.Tensor, nq: torch.Tensor, floor: torch.Tensor, proj: torch.Tensor, g_off: int,
                   weight: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """h = o / (max(|n . q|, floor) + 1e-6) per (token, head), h / sqrt(mean h^2 + eps) over the head's values,
    times ``weight`` [heads * vdim], times the sigmoid of the gate (columns ``g_off`` .. of ``proj``);
    [N, heads * vdim] in ``out_dtype``."""
    _need(o, "o", torch.float32); _need(nq, "nq", torch.float32); _need(floor, "floor", torch.float32)
    _need(proj, "proj"); _need(weight, "weight")
    n, heads, vdim = o.shape
    if weight.numel() != heads * vdim or g_off + heads * vdim > proj.shape[1] or proj.shape[0] != n:
        raise KernelError("the norm weight or the gate columns do not match the heads and sizes")
    out = torch.empty((n, heads * vdim), dtype=out_dtype, device=o.device)
    _check(lib().hb_mlstm_out_norm(_ptr(o), _ptr(nq), _ptr(floor), _ptr(proj), _dt(proj), proj.shape[1], g_off,
                                   _ptr(weight), _dt(weight), float(eps), _ptr(out), _dt(out), n, heads, vdim,
                                   _stream()), "mlstm_out_norm")
    return out


def moe_combine(y: torch.Tensor, slot_of_entry: torch.Tensor, shared: Optional[torch.Tensor], n: int,
                top_k: int, routed_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = shared[t] + sum_j w[t*k + j] * y[slot_of_entry[t*k + j]]  -> float32 [n, H] (w = 1 without
    ``routed_weight``)."""
    _need(y, "y", torch.float32); _need(slot_of_entry, "slot_of_entry", torch.int32)
    hidden = y.shape[1]
    if shared is not None:
        _need(shared, "shared")
        if tuple(shared.shape) != (n, hidden):
            raise KernelError("shared expert output has the wrong shape")
    out = torch.empty((n, hidden), dtype=torch.float32, device=y.device)
    if routed_weight is not None:
        _need(routed_weight, "routed_weight", torch.float32)
    _check(lib().hb_moe_combine(_ptr(y), _ptr(slot_of_entry), _ptr(routed_weight), _ptr(shared),
                                _dt(shared) if shared is not None else 0,
                                _ptr(out), n, hidden, top_k, _stream()), "moe_combine")
    return out


def random_normal(out: torch.Tensor, key: int, scale: float, first: int = 0) -> torch.Tensor:
    """Fill ``out`` (float32 or bfloat16, contiguous) with the seeded values of elements
    ``first ..`` of the tensor with ``key``; ``scale`` = std / (sigma * 2**24) as float32
    (``hi_b200/weights/random_values.py`` computes the same bits on the host)."""
    _need(out, "out")
    _check(lib().hb_random_normal(_ptr(out), _dt(out), out.numel(), int(first), int(key), float(scale), _stream()),
           "random_normal")
    return out


# --------------------------------------------------------------------------- attention
def qkv_post(qkv: torch.Tensor, nh: int, nkv: int, hd: int, positions: torch.Tensor,
             inv_freq: Optional[torch.Tensor], interleaved: bool, qk_norm: bool, qk_eps: float,
             temperature: Optional[Tuple[float, float]], seq_of_token: Optional[torch.Tensor],
             block_table: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
             v_pages: Optional[torch.Tensor], page_size: int, write_kv: bool,
             q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
             norm_first: bool = False, norm_dim: int = 0, rot_mul: float = 1.0,
             v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False) -> torch.Tensor:
    """Rotary or temperature, optional L2 norm, and the cache append; returns q [N, nh, hd].

    By default the norm of q and k is weightless and comes after the rotation. ``norm_first``: it comes
    before, over the first ``norm_dim`` dims of a head (0: all; dims past them are padding), times
    ``q_norm_weight`` / ``k_norm_weight`` (float32 [hd], shared by the heads). ``rot_mul`` multiplies
    cos and sin. Any even number of rotating dims is taken then (a general kernel runs these forms).
    ``v_inv_freq`` (float32 [pairs]): the values are cached rotated by their own position, pair m of their first
    2 * pairs dims by position * v_inv_freq[m] (pairs (m, m + pairs), or (2m, 2m + 1) with ``v_interleaved``).

    ``qkv`` is [N, (nh + 2*nkv) * hd]; ``k_pages``/``v_pages`` are [pages, nkv, page_size, hd];
    ``block_table`` [S, width] int32 maps (sequence row, position // page_size) to a page.
    """
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(nh + 2 * nkv) * hd}")
    general = v_inv_freq is not None or norm_first or q_norm_weight is not None or k_norm_weight is not None or rot_mul != 1.0 or \
        (norm_dim not in (0, hd)) or (inv_freq is not None and inv_freq.numel() % 8 != 0)
    if hd % 8 != 0 or hd > 1024 or (not general and (hd % 16 != 0 or hd > 256)):
        raise KernelError(f"head_dim {hd} is not supported (multiples of 16 up to 256; the general form: of 8 up to 1024)")
    v_pairs = 0
    if v_inv_freq is not None:
        _need(v_inv_freq, "v_inv_freq", torch.float32)
        v_pairs = v_inv_freq.numel()
        if 2 * v_pairs > hd:
            raise KernelError("more rotating value dims than a head has")
    if general:
        rot_pairs = 0 if inv_freq is None else inv_freq.numel()
        if inv_freq is not None:
            _need(inv_freq, "inv_freq", torch.float32)
        for wt, nm in ((q_norm_weight, "q_norm_weight"), (k_norm_weight, "k_norm_weight")):
            if wt is not None:
                _need(wt, nm, torch.float32)
                if wt.numel() != hd:
                    raise KernelError(f"{nm} needs one weight per dim of a head ({hd})")
    else:
        rot_pairs = _rot_pairs(inv_freq, hd)
    stride = 0
    if write_kv:
        for t, nm in ((seq_of_token, "seq_of_token"), (block_table, "block_table")):
            _need(t, nm, torch.int32)
        _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
        if tuple(k_pages.shape[1:]) != (nkv, page_size, hd) or k_pages.shape != v_pages.shape:
            raise KernelError(f"cache pages have shape {tuple(k_pages.shape)}, expected [*, {nkv}, {page_size}, {hd}]")
        stride = block_table.shape[1]
    q = torch.empty((n, nh, hd), dtype=qkv.dtype, device=qkv.device)
    fs, asc = temperature if temperature is not None else (1.0, 0.0)
    _check(lib().hb_qkv_post(_ptr(qkv), _dt(qkv), _ptr(inv_freq), rot_pairs, int(interleaved), int(qk_norm),
                             float(qk_eps), int(temperature is not None), float(fs), float(asc), _ptr(q_norm_weight),
                             _ptr(k_norm_weight), int(norm_first), int(norm_dim), float(rot_mul), _ptr(v_inv_freq),
                             v_pairs, int(v_interleaved), _ptr(positions),
                             _ptr(seq_of_token), _ptr(block_table), stride, _ptr(q), _ptr(k_pages), _ptr(v_pages),
                             page_size, int(write_kv), n, nh, nkv, hd, _stream()), "qkv_post")
    return q


def _rot_pairs(inv_freq: Optional[torch.Tensor], hd: int) -> int:
    """How many pairs of a head rotate: the table's length; whole lanes of 8 pairs, at most head_dim / 2."""
    if inv_freq is None:
        return 0
    _need(inv_freq, "inv_freq", torch.float32)
    pairs = inv_freq.numel()
    if pairs % 8 or not 0 < 2 * pairs <= hd:
        raise KernelError(f"inv_freq has {pairs} entries: the rotated dims must be a multiple of 16, at most head_dim ({hd})")
    return pairs


ATTENTION_SPLIT = 256      # keys per split of the general attention kernel
DECODE_RESIDENT_BLOCKS = 148 * 3   # blocks of the decode kernel resident at a time


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                    seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int,
                    scale: float, max_context: int = 0, sink: bool = False, softcap: float = 0.0,
                    slopes: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(q k^T * scale) v over the keys each token may read; q [N, nh, hd] -> [N, nh, hd].
    ``sink`` (here and in the other attention kernels): the softmax's denominator has one more term of
    score 0, p_j = e^{s_j} / (1 + sum_j e^{s_j}); the term has no value. ``sink_values`` (float32 [nh]): the
    term's score is the head's own number instead of 0. ``softcap`` > 0: the scaled score becomes
    softcap * tanh(score / softcap). ``slopes`` (float32 [nh]): slopes[h] * (query position - key position)
    is taken off the score (after the cap).

    ``max_context`` (an upper bound of position + 1 over the tokens) lets long ranges be cut into
    splits of ``ATTENTION_SPLIT`` keys that run in parallel and are merged; a token's splits depend
    on its own range only. 0 = one pass per (token, head)."""
    _need(q, "q"); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if nh % nkv:
        raise KernelError(f"{nh} query heads are not a multiple of {nkv} kv heads")
    if hd % 16 != 0 or hd > 1024:
        raise KernelError(f"head_dim {hd} is not supported (multiples of 16 up to 1024)")
    for t, nm in ((slopes, "slopes"), (sink_values, "sink_values")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != nh:
                raise KernelError(f"{nm} needs one number per query head")
    out = torch.empty_like(q)
    longest = max_context
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    splits = max(1, -(-longest // ATTENTION_SPLIT))
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=q.device)
    _check(lib().hb_paged_attention(_ptr(q), _dt(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                    block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv,
                                    hd, page_size, int(chunk), int(window), float(scale),
                                    int(sink or sink_values is not None), float(softcap), _ptr(slopes),
                                    _ptr(sink_values), ATTENTION_SPLIT, splits, _ptr(part_acc), _ptr(part_ml), _stream()),
           "paged_attention")
    return out


def sigmoid_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int, scale: float,
                      head_bias: Optional[torch.Tensor], max_context: int = 0,
                      v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False,
                      split_size: Optional[int] = None) -> torch.Tensor:
    """sum_j sigmoid(q . k_j * scale + head_bias[h]) v_j over the keys each token may read (no normalisation);
    q [N, nh, hd] -> [N, nh, hd]. With ``v_inv_freq`` the cached values are taken as rotated by their positions
    and every head's sum is turned back by the query's position (see :func:`qkv_post`). Long ranges are cut into
    splits of ``split_size`` keys (default ``ATTENTION_SPLIT``) as in :func:`paged_attention`; the splits add."""
    _need(q, "q"); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape or nh % nkv:
        raise KernelError("cache pages do not match the query's heads")
    if hd % 8 != 0 or hd > 512:
        raise KernelError(f"head_dim {hd} is not supported (multiples of 8 up to 512)")
    if head_bias is not None:
        _need(head_bias, "head_bias", torch.float32)
        if head_bias.numel() != nh:
            raise KernelError("one bias per query head")
    v_pairs = 0
    if v_inv_freq is not None:
        _need(v_inv_freq, "v_inv_freq", torch.float32)
        v_pairs = v_inv_freq.numel()
    out = torch.empty_like(q)
    longest = max_context
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size = int(split_size or ATTENTION_SPLIT)
    splits = max(1, -(-longest // split_size))
    part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device) if splits > 1 else None
    _check(lib().hb_sigmoid_attention(_ptr(q), _dt(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                      block_table.shape[1], _ptr(seq_of_token), _ptr(positions), _ptr(head_bias),
                                      _ptr(v_inv_freq), v_pairs, int(v_interleaved), _ptr(out), n, nh, nkv, hd,
                                      page_size, int(chunk), int(window), float(scale), split_size, splits,
                                      _ptr(part_acc), _stream()), "sigmoid_attention")
    return out


def sigmoid_merge(part_acc: torch.Tensor, positions: torch.Tensor, out_dtype: torch.dtype,
                  v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False) -> torch.Tensor:
    """part_acc float32 [N, nh, splits, hd] -> [N, nh, hd]: the splits of every (token, head) added in split order,
    then (``v_inv_freq``) the sum turned back by the token's position."""
    _need(part_acc, "part_acc", torch.float32); _need(positions, "positions", torch.int32)
    n, nh, splits, hd = part_acc.shape
    v_pairs = 0
    if v_inv_freq is not None:
        _need(v_inv_freq, "v_inv_freq", torch.float32)
        v_pairs = v_inv_freq.numel()
    out = torch.empty((n, nh, hd), dtype=out_dtype, device=part_acc.device)
    _check(lib().hb_sigmoid_merge(_ptr(part_acc), _ptr(positions), _ptr(v_inv_freq), v_pairs, int(v_interleaved), _ptr(out),
                                  _dt(out), n, nh, hd, splits, _stream()), "sigmoid_merge")
    return out


def sigmoid_attention_tc_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Shapes the tensor-core kernels take with sigmoid weights: those of the decode kernel and of the tcgen05
    prefill kernel at once."""
    return decode_attention_supported(q_dtype, nh, nkv, hd) and prefill_attention_tc_supported(q_dtype, nh, nkv, hd, page_size)


def sigmoid_decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                             seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int, scale: float,
                             head_bias: torch.Tensor, max_context: int, v_inv_freq: Optional[torch.Tensor] = None,
                             v_interleaved: bool = False) -> torch.Tensor:
    """:func:`sigmoid_attention` for a batch of single decoded tokens in bfloat16 on the tensor cores: the decode
    kernel of :func:`decode_attention` with sigmoid weights (the query heads of a kv head in one tile, the keys cut
    into splits as there); the splits' plain sums are added and turned back by :func:`sigmoid_merge`."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(head_bias, "head_bias", torch.float32)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape or head_bias.numel() != nh:
        raise KernelError("cache pages or head_bias do not match the query's heads")
    if not decode_attention_supported(q.dtype, nh, nkv, hd):
        raise KernelError(f"decode attention does not take nh={nh} nkv={nkv} head_dim={hd}")
    longest = max(int(max_context), 1)
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size, splits = _decode_splits(longest, n * nkv)
    part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device)
    _check(lib().hb_attention_decode(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                     _ptr(seq_of_token), _ptr(positions), _ptr(part_acc), n, nh, nkv, hd, page_size,
                                     int(chunk), int(window), float(scale), 2, _ptr(head_bias), 0.0, None, None, split_size,
                                     splits, _ptr(part_acc), None, _stream()), "attention_decode")
    return sigmoid_merge(part_acc, positions, q.dtype, v_inv_freq, v_interleaved)


def sigmoid_prefill_attention_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                                 cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, max_new: int, chunk: int,
                                 window: int, scale: float, head_bias: torch.Tensor, skip_single: bool = False,
                                 v_inv_freq: Optional[torch.Tensor] = None, v_interleaved: bool = False) -> torch.Tensor:
    """:func:`sigmoid_attention` for portions of prompts in bfloat16 on tcgen05: the kernel of
    :func:`prefill_attention_tc` with sigmoid weights, which turns its rows back by their positions in its epilogue
    (pairs in halves over a part of the row only: float32 sums out and :func:`sigmoid_merge`). Rows of requests
    that bring one token are zero with ``skip_single``."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    _need(head_bias, "head_bias", torch.float32)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    n_pages, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape or head_bias.numel() != nh:
        raise KernelError("cache pages or head_bias do not match the query's heads")
    if not prefill_attention_tc_supported(q.dtype, nh, nkv, hd, page_size):
        raise KernelError(f"tcgen05 prefill attention does not take nh={nh} nkv={nkv} head_dim={hd} page={page_size}")
    if cu_seqlens.numel() != n_seqs + 1 or block_table.shape[0] < n_seqs:
        raise KernelError("cu_seqlens / block_table do not match the number of requests")
    v_pairs = 0
    if v_inv_freq is not None:
        _need(v_inv_freq, "v_inv_freq", torch.float32)
        v_pairs = v_inv_freq.numel()
    if v_pairs == 0 or v_interleaved or 2 * v_pairs == hd:
        # the kernel turns its rows back itself and writes the result
        out = torch.zeros_like(q) if skip_single else torch.empty_like(q)
        _check(lib().hb_sigmoid_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                           _ptr(cu_seqlens), _ptr(positions), _ptr(out), n, n_pages, n_seqs, int(max_new), nh,
                                           nkv, hd, page_size, int(chunk), int(window), float(scale), int(skip_single),
                                           _ptr(head_bias), _ptr(v_inv_freq), v_pairs, int(v_interleaved),
                                           _ptr(_tc_status(q.device)), _stream()), "sigmoid_prefill_tc")
        TC_USED[0] = True
        return out
    part_acc = torch.zeros((n, nh, 1, hd), dtype=torch.float32, device=q.device)
    _check(lib().hb_attention_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                         block_table.shape[1], _ptr(cu_seqlens), _ptr(positions), _ptr(part_acc), n, n_pages,
                                         n_seqs, int(max_new), nh, nkv, hd, page_size, int(chunk), int(window),
                                         float(scale), int(skip_single), 2, _ptr(head_bias), 1, _ptr(part_acc), None,
                                         _ptr(_tc_status(q.device)), _stream()), "attention_prefill_tc")
    TC_USED[0] = True
    return sigmoid_merge(part_acc, positions, q.dtype, v_inv_freq, v_interleaved)


def _decode_splits(longest: int, groups: int) -> Tuple[int, int]:
    """How to cut ``longest`` keys for ``groups`` (token, kv head) pairs: the number of splits
    that minimises waves x (tiles per block + a block's fixed cost) + a cost per split (the
    merge) on 148 SMs x 3 resident blocks, none shorter than ATTENTION_SPLIT keys. Measured at
    8 requests x 8,192 keys: 6 splits (one wave of 384 blocks) 57 us, 13 splits (two waves) 63 us;
    one request x 32,768 keys: 32 splits 33 us, 47 splits 36 us.
    The cut moves results by rounding only."""
    best = (None, 1, longest)
    for s in range(1, max(1, -(-longest // ATTENTION_SPLIT)) + 1):
        size = -(-(-(-longest // s)) // 64) * 64
        real = -(-longest // size)
        waves = -(-(real * groups) // DECODE_RESIDENT_BLOCKS)
        cost = waves * (size // 64 + 1.5) + 0.2 * real + 0.3 * max(0, real - 32)   # past 32 the merge reads in turns
        if best[0] is None or cost < best[0]:
            best = (cost, real, size)
    return best[2], best[1]


# Row lengths (head dims) of the tensor-core attention kernels. 192 is a latent of 128 with a rotated key part of 64;
# only the cp.async decode kernel, the mma.sync prefill kernel and the tcgen05 prefill kernel take it (the TMA
# decode kernels answer "unsupported" and the callers fall back to those).
TC_ROW_LENGTHS = (64, 128, 192)


def decode_attention_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int) -> bool:
    """Shapes the tensor-core decode kernel takes; anything else goes to the general kernel."""
    return q_dtype == torch.bfloat16 and hd in TC_ROW_LENGTHS and nh % nkv == 0 and nh // nkv <= 16


def decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                     seq_of_token: torch.Tensor, positions: torch.Tensor, chunk: int, window: int, scale: float,
                     max_context: int, sink: bool = False, softcap: float = 0.0,
                     slopes: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention for a batch of single decoded tokens (every row of ``q`` is one request's
    token), bfloat16, split over runs of ``ATTENTION_SPLIT`` keys. Uses scratch memory for the
    partial results of the splits. ``softcap``, ``slopes``, ``sink_values``: as :func:`paged_attention`
    (the kernel that loads its tiles by cp.async takes them)."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not decode_attention_supported(q.dtype, nh, nkv, hd):
        raise KernelError(f"decode attention does not take nh={nh} nkv={nkv} head_dim={hd}")
    longest = max(int(max_context), 1)
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size, splits = _decode_splits(longest, n * nkv)
    out = torch.empty_like(q)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=q.device)
    reshaped = bool(softcap) or slopes is not None or sink_values is not None
    for t, nm in ((slopes, "slopes"), (sink_values, "sink_values")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != nh:
                raise KernelError(f"{nm} needs one number per query head")
    sink = bool(sink) or sink_values is not None
    # tile loads by TMA where the range and the pages allow it (the kernel says if not)
    code = _UNSUPPORTED if reshaped else lib().hb_attention_decode_tma(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(block_table), block_table.shape[1],
        _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv, hd, page_size, int(chunk), int(window), float(scale),
        int(sink), split_size, splits, _ptr(part_acc), _ptr(part_ml), _ptr(_tc_status(q.device)), _stream())
    if code == _UNSUPPORTED:
        code = lib().hb_attention_decode(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                                         _ptr(seq_of_token), _ptr(positions), _ptr(out), n, nh, nkv, hd, page_size,
                                         int(chunk), int(window), float(scale), int(sink), None, float(softcap),
                                         _ptr(slopes), _ptr(sink_values), split_size, splits,
                                         _ptr(part_acc), _ptr(part_ml), _stream())
        _check(code, "attention_decode")
    else:
        TC_USED[0] = True
        _check(code, "attention_decode_tma")
    if splits > 1:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, splits,
                                        int(sink), nh, _ptr(sink_values), _stream()), "attention_merge")
    return out


FUSED_COUNTERS = 1 << 18     # (token, kv head) pairs the fused decode kernel has counters for
# The fused kernel pays for what it saves in launches with work at the head and the tail of every
# block; once the blocks fill the machine several times over that shows. Measured at 8,192 keys, 8 kv
# heads: 2 / 8 / 16 requests 32.8 / 69.6 / 110.6 us against 38.9 / 76.7 / 117.8 us for the three
# kernels; 32 requests equal; 64 requests 364 against 352 us.
FUSED_MAX_GROUPS = 256       # (token, kv head) pairs up to which a decode step takes the fused kernel
_fused_counters: dict = {}   # device -> int32 zeros that the fused kernel leaves at zero


def _fused_counter_buffer(dev) -> torch.Tensor:
    key = (dev.type, dev.index)
    c = _fused_counters.get(key)
    if c is None:
        c = _fused_counters[key] = torch.zeros(FUSED_COUNTERS, dtype=torch.int32, device=dev)
    return c


def decode_attention_fused(qkv: torch.Tensor, nh: int, nkv: int, hd: int, positions: torch.Tensor,
                           inv_freq: Optional[torch.Tensor], interleaved: bool, qk_norm: bool, qk_eps: float,
                           temperature: Optional[Tuple[float, float]], seq_of_token: torch.Tensor,
                           block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, chunk: int,
                           window: int, scale: float, max_context: int, merge_inside: bool = True,
                           q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                           norm_first: bool = False, rot_mul: float = 1.0, sink: bool = False) -> Optional[torch.Tensor]:
    """:func:`qkv_post`, :func:`decode_attention` and the merge of its splits in ONE launch, for a step
    of single decoded tokens: ``qkv`` [N, (nh + 2 nkv) * hd] bfloat16 is the projection's output; the
    kernel encodes q, k and v, appends the token's key and value to its page, attends over the cache
    and combines the splits (the block that finishes last does it). Returns [N, nh, hd], or None
    where the kernel does not take the shapes (the caller then runs the three kernels). ``q_norm_weight``,
    ``k_norm_weight``, ``norm_first``, ``rot_mul`` and ``sink`` as in :func:`qkv_post` and :func:`paged_attention`
    (the norm then runs over the whole head)."""
    _need(qkv, "qkv", torch.bfloat16); _need(k_pages, "k_pages", qkv.dtype); _need(v_pages, "v_pages", qkv.dtype)
    for t, nm in ((block_table, "block_table"), (seq_of_token, "seq_of_token"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    n_pages, nkv2, page_size, hd2 = k_pages.shape
    if qkv.shape[1] != (nh + 2 * nkv) * hd or hd2 != hd or nkv2 != nkv or k_pages.shape != v_pages.shape:
        raise KernelError("qkv or the cache pages do not match the heads and head_dim")
    if not decode_attention_supported(qkv.dtype, nh, nkv, hd) or n * nkv > min(FUSED_COUNTERS, FUSED_MAX_GROUPS):
        return None
    if inv_freq is not None and (inv_freq.numel() % 8 or 2 * inv_freq.numel() > hd):
        return None                       # whole lanes of 8 pairs rotate in this kernel
    for wt in (q_norm_weight, k_norm_weight):
        if wt is not None:
            _need(wt, "norm weight", torch.float32)
            if wt.numel() != hd:
                raise KernelError(f"a q/k norm weight needs one number per dim of a head ({hd})")
    rot_pairs = _rot_pairs(inv_freq, hd)
    longest = max(int(max_context), 1)
    if chunk > 0:
        longest = min(longest, chunk)
    if window > 0:
        longest = min(longest, window)
    split_size, splits = _decode_splits(longest, n * nkv)
    out = torch.empty((n, nh, hd), dtype=qkv.dtype, device=qkv.device)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = torch.empty((n, nh, splits, hd), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((n, nh, splits, 2), dtype=torch.float32, device=qkv.device)
    fs, asc = temperature if temperature is not None else (1.0, 0.0)
    code = lib().hb_attention_decode_fused(
        _ptr(qkv), _ptr(inv_freq), rot_pairs, int(interleaved), int(qk_norm), float(qk_eps), int(temperature is not None), float(fs),
        float(asc), _ptr(k_pages), _ptr(v_pages), n_pages, _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
        _ptr(positions), _ptr(out), n, nh, nkv, hd, page_size, int(chunk), int(window), float(scale), split_size, splits,
        _ptr(part_acc), _ptr(part_ml), _ptr(_fused_counter_buffer(qkv.device)) if merge_inside else None,
        _ptr(_tc_status(qkv.device)), _ptr(q_norm_weight), _ptr(k_norm_weight), int(norm_first), float(rot_mul), int(sink),
        _stream())
    if code == _UNSUPPORTED:
        return None
    TC_USED[0] = True
    _check(code, "attention_decode_fused")
    if splits > 1 and not merge_inside:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, splits,
                                        int(sink), nh, None, _stream()), "attention_merge")
    return out


def prefill_attention_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int) -> bool:
    """Shapes the tensor-core prefill kernel takes; anything else goes to the general kernel."""
    return q_dtype == torch.bfloat16 and hd in TC_ROW_LENGTHS and nh % nkv == 0


def prefill_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, max_new: int, chunk: int,
                      window: int, scale: float, skip_single: bool = False,
                      out: Optional[torch.Tensor] = None, sink: bool = False, softcap: float = 0.0,
                      slopes: Optional[torch.Tensor] = None, sink_values: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention for portions of prompts: request ``s`` owns rows ``cu_seqlens[s]..cu_seqlens[s+1]``
    of ``q`` [N, nh, hd], at consecutive positions; bfloat16, flash attention on tensor cores.
    ``skip_single`` leaves the rows of requests that bring one token unwritten (the caller runs
    the decode kernel for them and passes the same ``out``). ``softcap``, ``slopes``, ``sink_values``: as
    :func:`paged_attention`."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    _, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not prefill_attention_supported(q.dtype, nh, nkv, hd):
        raise KernelError(f"prefill attention does not take nh={nh} nkv={nkv} head_dim={hd}")
    if cu_seqlens.numel() != n_seqs + 1 or block_table.shape[0] < n_seqs:
        raise KernelError("cu_seqlens / block_table do not match the number of requests")
    if out is None:
        out = torch.empty_like(q)
    for t, nm in ((slopes, "slopes"), (sink_values, "sink_values")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != nh:
                raise KernelError(f"{nm} needs one number per query head")
    _check(lib().hb_attention_prefill_reshaped(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                               block_table.shape[1], _ptr(cu_seqlens), _ptr(positions), _ptr(out), n_seqs,
                                               int(max_new), nh, nkv, hd, page_size, int(chunk), int(window), float(scale),
                                               int(skip_single), int(bool(sink) or sink_values is not None),
                                               float(softcap), _ptr(slopes), _ptr(sink_values), _stream()),
           "attention_prefill")
    return out


PREFILL_TC_MIN_TOKENS = 128     # a request needs at least a tile of new tokens for the tcgen05 kernel to pay


def prefill_attention_tc_supported(q_dtype: torch.dtype, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    """Shapes the tcgen05 prefill kernel takes: bfloat16, head_dim 64, 128 or 192, pages of 16, 32 or a
    multiple of 64 positions (a 64-key tile is loaded page by page with TMA)."""
    return q_dtype == torch.bfloat16 and hd in TC_ROW_LENGTHS and nh % nkv == 0 and page_size % 16 == 0 and \
        (64 % page_size == 0 or page_size % 64 == 0)


def prefill_attention_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, max_new: int, chunk: int,
                         window: int, scale: float, skip_single: bool = False,
                         out: Optional[torch.Tensor] = None, key_splits: int = 1, sink: bool = False,
                         softcap: float = 0.0, slopes: Optional[torch.Tensor] = None,
                         sink_values: Optional[torch.Tensor] = None) -> torch.Tensor:
    """As :func:`prefill_attention`, on tcgen05 (S, P V and O in tensor memory, TMA page loads).
    ``key_splits`` > 1: that many blocks share the key tiles of every (query tile, head) and a
    merge kernel combines their rows (see :func:`prefill_key_splits`). ``softcap``, ``slopes``, ``sink_values``:
    as :func:`paged_attention`."""
    _need(q, "q", torch.bfloat16); _need(k_pages, "k_pages", q.dtype); _need(v_pages, "v_pages", q.dtype)
    for t, nm in ((block_table, "block_table"), (cu_seqlens, "cu_seqlens"), (positions, "positions")):
        _need(t, nm, torch.int32)
    n, nh, hd = q.shape
    n_pages, nkv, page_size, hd2 = k_pages.shape
    if hd2 != hd or k_pages.shape != v_pages.shape:
        raise KernelError("cache pages do not match the query's head_dim")
    if not prefill_attention_tc_supported(q.dtype, nh, nkv, hd, page_size):
        raise KernelError(f"tcgen05 prefill attention does not take nh={nh} nkv={nkv} head_dim={hd} page={page_size}")
    if cu_seqlens.numel() != n_seqs + 1 or block_table.shape[0] < n_seqs:
        raise KernelError("cu_seqlens / block_table do not match the number of requests")
    if out is None:
        out = torch.empty_like(q)
    key_splits = int(key_splits)
    part_acc = part_ml = None
    if key_splits > 1:
        part_acc = torch.empty((n * nh, key_splits, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * nh, key_splits, 2), dtype=torch.float32, device=q.device)
    for t, nm in ((slopes, "slopes"), (sink_values, "sink_values")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != nh:
                raise KernelError(f"{nm} needs one number per query head")
    sink = bool(sink) or sink_values is not None
    if softcap or slopes is not None or sink_values is not None:
        _check(lib().hb_attention_prefill_tc_reshaped(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1], _ptr(cu_seqlens),
            _ptr(positions), _ptr(out), n, n_pages, n_seqs, int(max_new), nh, nkv, hd, page_size, int(chunk), int(window),
            float(scale), int(skip_single), int(sink), float(softcap), _ptr(slopes), _ptr(sink_values), key_splits,
            _ptr(part_acc), _ptr(part_ml), _ptr(_tc_status(q.device)), _stream()), "attention_prefill_tc")
    else:
        _check(lib().hb_attention_prefill_tc(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                             block_table.shape[1], _ptr(cu_seqlens), _ptr(positions), _ptr(out), n, n_pages,
                                             n_seqs, int(max_new), nh, nkv, hd, page_size, int(chunk), int(window),
                                             float(scale), int(skip_single), int(sink), None, key_splits,
                                             _ptr(part_acc) if part_acc is not None else None,
                                             _ptr(part_ml) if part_ml is not None else None, _ptr(_tc_status(q.device)),
                                             _stream()),
               "attention_prefill_tc")
    TC_USED[0] = True
    if key_splits > 1:
        _check(lib().hb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), _dt(out), n * nh, hd, key_splits,
                                        int(sink), nh, _ptr(sink_values), _stream()), "attention_merge")
    return out


_sm_counts: dict = {}


def sm_count(device) -> int:
    key = torch.device(device)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


PREFILL_RESIDENT_BLOCKS_PER_SM = 2     # of the tcgen05 prefill kernel (tensor memory: 256 of 512 columns each)
PREFILL_SPLIT_MIN_TILES = 512          # key tiles (of 64 keys) a block must have before its keys are shared out
PREFILL_SPLIT_MIN_SHARE = 128          # and the fewest a share may get


def prefill_key_splits(blocks: int, key_tiles: int, sms: int) -> int:
    """How many blocks should share the key tiles of each (query tile, head) of the tcgen05 prefill
    kernel, when the ``blocks`` of a launch all have about ``key_tiles`` key tiles (a short portion
    far into a long context). The kernel runs two blocks per SM; with fewer blocks than that, or a
    few more, most of the GPU waits for the last ones. Measured at 65,000 cached tokens, 40 heads:
    128 new tokens 933 -> 256 us in six shares, 256 tokens 935 -> 448 us in three, 512 tokens
    1,116 -> 795 us in five, 1,024 tokens 2,163 -> 1,521 us in four; nothing gained at 16,000
    cached tokens, and a loss from 2,048 new tokens on (4,096: 5.09 -> 5.88 ms in three: the
    unnormalised rows written out and merged cost more than the fuller last round gains).
    So: only launches of up to 1.25 rounds with at least 512 key tiles; the number of shares (up to
    8, at least 128 tiles each) that fills the rounds best, the fewest among those within 0.05."""
    places = PREFILL_RESIDENT_BLOCKS_PER_SM * max(int(sms), 1)
    if blocks <= 0 or blocks > 1.25 * places or key_tiles < PREFILL_SPLIT_MIN_TILES:
        return 1
    fill = {k: (blocks * k / places) / -(-blocks * k // places) for k in range(1, 9)
            if k == 1 or key_tiles // k >= PREFILL_SPLIT_MIN_SHARE}
    best = max(fill.values())
    choice = min(k for k, f in fill.items() if f >= best - 0.05)
    return choice if fill[choice] > fill[1] else 1


# --------------------------------------------------------------------------- experts
ROUTER_SOFTMAX, ROUTER_RENORMALIZE = 1, 2     # bits of a router's ``mode``


def router_groups(count: int, keep: int) -> int:
    """The bits of a router's ``mode`` that limit the choice to the ``keep`` best of ``count`` equal groups
    of neighbouring experts (a group counts as the sum of its two largest sigmoid scores)."""
    if not 0 < keep <= count <= 64:
        raise KernelError(f"{keep} of {count} expert groups: up to 64 groups, at least one kept")
    return (int(count) << 8) | (int(keep) << 16)


def router_topk(x: torch.Tensor, w: torch.Tensor, top_k: int, want_logits: bool = False, mode: int = 0,
                score_scale: float = 1.0):
    """Router logits (float32), the top-k expert ids (ties to the lower id) and their scores: the
    sigmoid of the chosen logit, or with ``ROUTER_SOFTMAX`` its softmax over all experts; with
    ``ROUTER_RENORMALIZE`` divided by the sum of the chosen scores."""
    _need(x, "x"); _need(w, "router weight")
    n, hidden = x.shape
    experts = w.shape[0]
    if w.shape[1] != hidden:
        raise KernelError("router weight does not match the hidden size")
    ids = torch.empty((n, top_k), dtype=torch.int32, device=x.device)
    scores = torch.empty((n, top_k), dtype=torch.float32, device=x.device)
    logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)   # the blocks' meeting place
    _check(lib().hb_router_topk(_ptr(x), _dt(x), _ptr(w), _dt(w), n, hidden, experts, top_k, int(mode), float(score_scale),
                                _ptr(logits), _ptr(ids), _ptr(scores), _stream()), "router_topk")
    return ids, scores, logits if want_logits else None


class MoePlan:
    """Rows grouped by expert: ``offsets`` [E+1], ``sorted_entry`` [n] (entry of each sorted slot),
    ``slot_of_entry`` [n], ``active`` [E+1] (count, then the ids of the experts that have rows)."""

    __slots__ = ("offsets", "sorted_entry", "slot_of_entry", "active")

    def __init__(self, offsets, sorted_entry, slot_of_entry, active):
        self.offsets, self.sorted_entry, self.slot_of_entry, self.active = offsets, sorted_entry, slot_of_entry, active

    def __iter__(self):       # (offsets, sorted_entry, slot_of_entry) for callers that unpack
        return iter((self.offsets, self.sorted_entry, self.slot_of_entry))


def _empty_plan(n: int, experts: int, dev) -> MoePlan:
    return MoePlan(torch.empty(experts + 1, dtype=torch.int32, device=dev),
                   torch.empty(max(n, 1), dtype=torch.int32, device=dev),
                   torch.empty(max(n, 1), dtype=torch.int32, device=dev),
                   torch.empty(experts + 1, dtype=torch.int32, device=dev))


_block_counters: dict = {}     # device -> one int32 that kernels leave at zero; launches that share it must
                               # follow one another (the engine runs its steps on one stream)


def _block_counter(dev) -> torch.Tensor:
    c = _block_counters.get(dev)
    if c is None:
        c = _block_counters[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return c


def router_plan(x: torch.Tensor, w: torch.Tensor, top_k: int, mode: int = 0, score_scale: float = 1.0):
    """:func:`router_topk` and :func:`moe_plan` in one call: with few tokens one kernel does both
    (the block that ends last groups the entries). Returns ids, scores and the plan."""
    _need(x, "x"); _need(w, "router weight")
    n, hidden = x.shape
    experts = w.shape[0]
    if w.shape[1] != hidden:
        raise KernelError("router weight does not match the hidden size")
    ids = torch.empty((n, top_k), dtype=torch.int32, device=x.device)
    scores = torch.empty((n, top_k), dtype=torch.float32, device=x.device)
    logits = torch.empty((n, experts), dtype=torch.float32, device=x.device)   # the blocks' meeting place
    plan = _empty_plan(n * top_k, experts, x.device)
    _check(lib().hb_router_plan(_ptr(x), _dt(x), _ptr(w), _dt(w), n, hidden, experts, top_k, int(mode), float(score_scale),
                                _ptr(logits), _ptr(ids), _ptr(scores), _ptr(plan.offsets), _ptr(plan.sorted_entry),
                                _ptr(plan.slot_of_entry), _ptr(plan.active), _ptr(_block_counter(x.device)),
                                _stream()), "router_plan")
    return ids, scores, plan


def moe_plan(ids: torch.Tensor, experts: int) -> MoePlan:
    """Group the routing entries by expert, on the device."""
    _need(ids, "ids", torch.int32)
    n = ids.numel()
    plan = _empty_plan(n, experts, ids.device)
    _check(lib().hb_moe_plan(_ptr(ids), n, experts, _ptr(plan.offsets), _ptr(plan.sorted_entry),
                             _ptr(plan.slot_of_entry), _ptr(plan.active), _stream()), "moe_plan")
    return plan


def moe_gate_up(x: torch.Tensor, plan: MoePlan, top_k: int, w_gate: Optional[torch.Tensor],
                w_up: torch.Tensor, scores: torch.Tensor, few_rows: bool, activation: str = "swiglu") -> torch.Tensor:
    """act[slot] = silu(s * x Wg[e]^T) * (s * x Wu[e]^T), [N*k, I] in the engine dtype; with
    ``activation="relu2"`` (experts without a gate branch; ``w_gate`` None) max(s * x Wu[e]^T, 0)^2."""
    _need(x, "x"); _need(w_up, "w_up", x.dtype)
    _need(scores, "scores", torch.float32)
    if activation not in ("swiglu", "relu2") or (w_gate is None) != (activation == "relu2"):
        raise KernelError("experts have a gate stack with swiglu and none with relu2")
    n, hidden = x.shape
    experts, inter, h2 = w_up.shape
    if w_gate is not None:
        _need(w_gate, "w_gate", x.dtype)
    if h2 != hidden or (w_gate is not None and w_up.shape != w_gate.shape):
        raise KernelError("expert gate/up weights do not match the hidden size")
    n_entries = n * top_k
    act = torch.empty((n_entries, inter), dtype=x.dtype, device=x.device)
    _check(lib().hb_moe_gate_up(_ptr(x), _dt(x), _ptr(plan.sorted_entry), top_k, _ptr(w_gate), _ptr(w_up),
                                _ptr(plan.offsets), _ptr(plan.active), experts, _ptr(scores), _ptr(act), n_entries,
                                inter, hidden, int(few_rows), 1 if activation == "relu2" else 0, _stream()),
           "moe_gate_up")
    return act


def moe_down(act: torch.Tensor, w_down: torch.Tensor, plan: MoePlan, few_rows: bool) -> torch.Tensor:
    """y[slot] = act[slot] Wd[e]^T, float32 [N*k, H]."""
    _need(act, "act"); _need(w_down, "w_down", act.dtype)
    n_entries, inter = act.shape
    experts, hidden, i2 = w_down.shape
    if i2 != inter:
        raise KernelError("expert down weights do not match the intermediate size")
    y = torch.empty((n_entries, hidden), dtype=torch.float32, device=act.device)
    _check(lib().hb_moe_down(_ptr(act), _dt(act), _ptr(w_down), _ptr(plan.offsets), _ptr(plan.active), experts,
                             _ptr(y), n_entries, hidden, inter, int(few_rows), _stream()), "moe_down")
    return y


# --------------------------------------------------------------------------- experts on tcgen05
_TC_STATUS = {}          # device -> int32[1]: nonzero after a tensor-core kernel gave up a bounded wait
TC_USED = [False]


def _tc_status(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def check_tc_status(device=None) -> None:
    """Raise if a kernel with bounded mbarrier waits (the tcgen05 products and attention, the TMA
    decode attention) timed out on one of its barriers since the last check
    (synchronises; skipped while a stream is being captured)."""
    TC_USED[0] = False
    if torch.cuda.is_current_stream_capturing():
        return
    for key, st in _TC_STATUS.items():
        code = int(st.item())
        if code != 0:
            st.zero_()
            for buffers in (_down_scratch_buffers.get(key),):       # a kernel that gave up may have left a count behind
                if buffers is not None:
                    buffers[1].zero_()
            where = {1: "grouped product: the TMA producer waiting for a free stage",
                     2: "grouped product: the MMA issuer waiting for a loaded stage",
                     3: "grouped product: the epilogue waiting for the accumulator",
                     4: "grouped product: the MMA issuer waiting for a free accumulator",
                     31: "decode attention: the warps waiting for a tile's TMA loads"}.get(
                code, f"prefill attention, wait {code}" if code >= 11 else f"code {code}")
            raise KernelError(f"a kernel gave up a bounded wait ({where}); its output is invalid")


class PendingStatus:
    """The status word copied to pinned memory behind the step's kernels; read it later."""

    def __init__(self, device: torch.device):
        self.host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.event = torch.cuda.Event()
        self.device = device
        self.pending = False
        self.claimed = False         # someone other than the engine has taken it and will resolve it

    def enqueue(self) -> None:
        self.host.copy_(_tc_status(self.device), non_blocking=True)
        self.event.record()
        self.pending = True

    def resolve(self, wait: bool = True) -> bool:
        """Read the copied word; raises if a kernel reported a failed wait. With ``wait=False`` it
        returns False, without blocking, while the copy has not run yet (the word on the device
        stays set until it is read, so a later look still sees it)."""
        if not self.pending:
            return True
        if not wait and not self.event.query():
            return False
        self.event.synchronize()
        self.pending = False
        if int(self.host[0]) != 0:
            check_tc_status()          # raises with the reason, and clears the word
        return True


def moe_tc_supported(x: torch.Tensor, w_gate: torch.Tensor) -> bool:
    """The tensor-core expert kernels take bfloat16 with hidden and intermediate sizes that are
    multiples of 8 (TMA needs 16-byte row strides)."""
    return x.dtype == torch.bfloat16 and w_gate.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and \
        w_gate.shape[1] % 8 == 0


def gather_rows(x: torch.Tensor, plan: MoePlan, top_k: int) -> torch.Tensor:
    """The tokens' rows in expert order: xs[slot] = x[sorted_entry[slot] // top_k], bfloat16."""
    _need(x, "x", torch.bfloat16)
    n, hidden = x.shape
    rows = n * top_k
    xs = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    _check(lib().hb_gather_rows(_ptr(x), _ptr(plan.sorted_entry), top_k, _ptr(xs), rows, hidden, _stream()),
           "gather_rows")
    return xs


def moe_gate_up_tc(x: torch.Tensor, plan: MoePlan, top_k: int, w_gate: torch.Tensor, w_up: torch.Tensor,
                   scores: torch.Tensor) -> torch.Tensor:
    """As :func:`moe_gate_up`, on tcgen05: gathers the rows into expert order, then one grouped
    product with the SwiGLU epilogue."""
    _need(x, "x", torch.bfloat16); _need(w_gate, "w_gate", torch.bfloat16); _need(w_up, "w_up", torch.bfloat16)
    _need(scores, "scores", torch.float32)
    n, hidden = x.shape
    experts, inter, h2 = w_gate.shape
    if h2 != hidden or w_up.shape != w_gate.shape:
        raise KernelError("expert gate/up weights do not match the hidden size")
    rows = n * top_k
    xs = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    _check(lib().hb_gather_rows(_ptr(x), _ptr(plan.sorted_entry), top_k, _ptr(xs), rows, hidden, _stream()),
           "gather_rows")
    act = torch.empty((rows, inter), dtype=x.dtype, device=x.device)
    _check(lib().hb_moe_gate_up_tc(_ptr(xs), _ptr(plan.sorted_entry), _ptr(w_gate), _ptr(w_up), _ptr(plan.offsets),
                                   experts, _ptr(scores), _ptr(act), rows, inter, hidden, _ptr(_tc_status(x.device)),
                                   _stream()), "moe_gate_up_tc")
    TC_USED[0] = True
    return act


def moe_up_relu2_tc(x: torch.Tensor, plan: MoePlan, top_k: int, w_up: torch.Tensor) -> torch.Tensor:
    """act[slot] = max(x W_up[e]^T, 0)^2 on tcgen05, bfloat16 [N*k, I]: experts without a gate branch (the rows are
    gathered into expert order first; the squared relu is the product's epilogue)."""
    _need(x, "x", torch.bfloat16); _need(w_up, "w_up", torch.bfloat16)
    experts, inter, h2 = w_up.shape
    if h2 != x.shape[1]:
        raise KernelError("expert up weights do not match the hidden size")
    xs = gather_rows(x, plan, top_k)
    act = torch.empty((xs.shape[0], inter), dtype=x.dtype, device=x.device)
    _check(lib().hb_moe_up_relu2_tc(_ptr(xs), _ptr(w_up), _ptr(plan.offsets), experts, _ptr(act), xs.shape[0], inter, h2,
                                    _ptr(_tc_status(x.device)), _stream()), "moe_up_relu2_tc")
    TC_USED[0] = True
    return act


_down_scratch_buffers: dict = {}   # device -> (partial tiles of a cut last round, their counters, left at zero)


def _down_scratch(dev):
    key = (dev.type, dev.index)
    b = _down_scratch_buffers.get(key)
    if b is None:
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        b = _down_scratch_buffers[key] = (
            torch.empty(int(lib().hb_moe_down_tc_scratch_floats(sms)), dtype=torch.float32, device=dev),
            torch.zeros(sms, dtype=torch.int32, device=dev))
    return b


def moe_down_tc(act: torch.Tensor, w_down: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """As :func:`moe_down`, on tcgen05."""
    _need(act, "act", torch.bfloat16); _need(w_down, "w_down", torch.bfloat16)
    rows, inter = act.shape
    experts, hidden, i2 = w_down.shape
    if i2 != inter:
        raise KernelError("expert down weights do not match the intermediate size")
    y = torch.empty((rows, hidden), dtype=torch.float32, device=act.device)
    scratch, counters = _down_scratch(act.device)
    _check(lib().hb_moe_down_tc(_ptr(act), _ptr(w_down), _ptr(plan.offsets), experts, _ptr(y), rows, hidden, inter,
                                _ptr(scratch), scratch.numel(), _ptr(counters), counters.numel(),
                                _ptr(_tc_status(act.device)), _stream()), "moe_down_tc")
    TC_USED[0] = True
    return y


# --------------------------------------------------------------------------- sampling
ARGMAX_PARTS = 16            # blocks per row of the all-greedy sampler
ARGMAX_MAX_ROWS = 1024
ARGMAX_MIN_VOCAB = 8192
SAMPLE_PARTS = 16            # blocks per row of the sampler with temperatures, for steps of few rows
SAMPLE_PARTS_MAX_BLOCKS = 2048   # beyond 128 rows a block per row keeps the GPU as busy
_argmax_scratch: dict = {}   # device -> (values, ids, counters); shared by launches that follow one another


def _argmax_buffers(dev):
    b = _argmax_scratch.get(dev)
    if b is None:
        b = _argmax_scratch[dev] = (torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.int32, device=dev),
                                    torch.zeros(ARGMAX_MAX_ROWS, dtype=torch.int32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev),
                                    torch.empty(ARGMAX_MAX_ROWS * ARGMAX_PARTS, dtype=torch.float32, device=dev))
    return b


def sample_rows(logits: torch.Tensor, temperatures: Optional[torch.Tensor],
                uniforms: Optional[torch.Tensor]) -> torch.Tensor:
    """One token per row of float32 logits: argmax where temperature <= 0, else inverse CDF.
    Without temperatures (every row greedy) a few rows of a large vocabulary are cut over
    ``ARGMAX_PARTS`` blocks each."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperatures is None and rows <= ARGMAX_MAX_ROWS and vocab >= ARGMAX_MIN_VOCAB:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        vals, ids, counters = _argmax_buffers(logits.device)[:3]
        _check(lib().hb_argmax_rows(_ptr(logits), rows, vocab, ARGMAX_PARTS, _ptr(vals), _ptr(ids), _ptr(counters),
                                    _ptr(out), _stream()), "argmax_rows")
        return out
    for t, nm in ((temperatures, "temperatures"), (uniforms, "uniforms")):
        if t is not None:
            _need(t, nm, torch.float32)
            if t.numel() != rows:
                raise KernelError(f"{nm} needs one entry per row")
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if rows * SAMPLE_PARTS <= SAMPLE_PARTS_MAX_BLOCKS and vocab >= ARGMAX_MIN_VOCAB:
        # a few rows of a large vocabulary: every row over SAMPLE_PARTS blocks, the last of them picks
        vals, ids, counters, maxima, sums = _argmax_buffers(logits.device)
        _check(lib().hb_sample_rows_parts(_ptr(logits), rows, vocab, SAMPLE_PARTS, _ptr(temperatures), _ptr(uniforms),
                                          _ptr(vals), _ptr(ids), _ptr(maxima), _ptr(sums), _ptr(counters), _ptr(out),
                                          _stream()), "sample_rows_parts")
        return out
    _check(lib().hb_sample_rows(_ptr(logits), rows, vocab, _ptr(temperatures), _ptr(uniforms), _ptr(out), _stream()),
           "sample_rows")
    return out


def ranked_rows(logits: torch.Tensor, temperatures: torch.Tensor, top_ps: torch.Tensor, top_ks: torch.Tensor,
                uniforms: torch.Tensor, out: torch.Tensor) -> None:
    """Top-k / top-p rows of float32 logits, sampled in place into ``out`` (int32 [R]) by the host
    sampler's rule; rows without a temperature, or with neither a top-k below the vocabulary nor a
    top-p inside (0, 1), are left as they are. ``out[r] == -1`` afterwards: the row has more than
    4,096 candidates or logits that are not finite, and has to be ranked on the host."""
    _need(logits, "logits", torch.float32)
    rows = logits.shape[0]
    for t, nm, dt in ((temperatures, "temperatures", torch.float32), (top_ps, "top_ps", torch.float32),
                      (top_ks, "top_ks", torch.int32), (uniforms, "uniforms", torch.float32), (out, "out", torch.int32)):
        _need(t, nm, dt)
        if t.numel() != rows:
            raise KernelError(f"{nm} needs one entry per row")
    _check(lib().hb_ranked_rows(_ptr(logits), rows, logits.shape[1], _ptr(temperatures), _ptr(top_ps), _ptr(top_ks),
                                _ptr(uniforms), _ptr(out), _stream()), "ranked_rows")
