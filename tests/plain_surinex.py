"""A plain, slow statement of the Surinex decoder: one function per mechanism, float64 on the CPU,
whole sequences, no cache and no batching. It shares no code with ``hi_b200``; the tests hold the
engine against it.

A model is ``(config, tensors)``: the dict that config.json holds and a dict name -> float64 tensor.
Notation: T tokens, W the model width; a linear map stored [out, in] acts as ``x @ M.T``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times ``weight``."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def time_convolution(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time, channel by channel: y[t] = sum_j taps[:, j] * x[t - (K-1) + j],
    x = 0 before the sequence starts. ``x`` [T, C], ``taps`` [C, K]; the last column weighs the token itself."""
    t_len, k = x.shape[0], taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(t_len):
        for j in range(k):
            src = t - (k - 1) + j
            if src >= 0:
                y[t] += taps[:, j] * x[src]
    return y


def pair_frequencies(base: float, dims: int, scaling: Optional[dict] = None) -> torch.Tensor:
    """Turn per position of each of the dims / 2 pairs: base^(-2i/dims). ``scaling`` = {factor, low, high,
    original} stretches the slow pairs: with wavelength L = 2 pi / f, f stays where L < original / high,
    becomes f / factor where L > original / low, and in between is blended by
    s = (original / L - low) / (high - low): (1 - s) f / factor + s f."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, layout: str, sign: float = 1.0) -> torch.Tensor:
    """Rotate the first 2 * len(freqs) dims of the last axis of ``x`` [T, heads, D] by position * freq per pair;
    ``layout`` "interleaved": pairs (2i, 2i+1); "halves": pairs (i, i + n) with n = len(freqs). The pair (u, v)
    becomes (u cos a - v sin a, v cos a + u sin a); ``sign`` -1 turns back."""
    n = freqs.numel()
    angle = sign * positions.to(F64)[:, None, None] * freqs[None, None, :]
    c, s = torch.cos(angle), torch.sin(angle)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * c - v * s
        out[..., 1:2 * n:2] = v * c + u * s
    elif layout == "halves":
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n] = u * c - v * s
        out[..., n:2 * n] = v * c + u * s
    else:
        raise ValueError(layout)
    return out


# ----------------------------------------------------------------------------- mixers
def sigmoid_attention(h, p: dict, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    """Grouped heads, weighted RMS norm of q and k before a partial interleaved rotation, values that are
    rotated by their own position over all their dims and whose sum is turned back by the query's, and a
    sigmoid of (score + a number per head) instead of a softmax: weights are not normalised."""
    t_len = h.shape[0]
    heads, groups, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    pos = torch.arange(t_len)
    q = (h @ w[pre + ".q"].T).view(t_len, heads, dim)
    k = (h @ w[pre + ".k"].T).view(t_len, groups, dim)
    v = (h @ w[pre + ".v"].T).view(t_len, groups, vdim)
    q = rms_norm(q, w[pre + ".q.norm"], eps)
    k = rms_norm(k, w[pre + ".k.norm"], eps)
    rot = p["rot"]
    f = pair_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
    q, k = rotate(q, pos, f, "interleaved"), rotate(k, pos, f, "interleaved")
    fv = pair_frequencies(rot["base"], vdim)
    v = rotate(v, pos, fv, "interleaved")
    out = torch.zeros(t_len, heads, vdim, dtype=F64)
    for a in range(heads):
        g = a // (heads // groups)
        score = (q[:, a] @ k[:, g].T) * p["scale"] + w[pre + ".pb"][a]
        weight = torch.sigmoid(score) * torch.tril(torch.ones(t_len, t_len, dtype=F64))
        out[:, a] = weight @ v[:, g]
    out = rotate(out, pos, fv, "interleaved", sign=-1.0)
    return out.reshape(t_len, heads * vdim) @ w[pre + ".o"].T


def gated_delta_rule(h, p: dict, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    """Per head a matrix S [dim, vdim]: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with one
    decay g per head and token; q, k, v first pass a short convolution over time and silu, q and k are made
    unit vectors."""
    t_len = h.shape[0]
    heads, groups, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]

    def branch(name, n, size):
        return silu(time_convolution(h @ w[f"{pre}.{name}"].T, w[f"{pre}.{name}.conv"])).view(t_len, n, size)

    q, k, v = branch("q", groups, dim), branch("k", groups, dim), branch("v", heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + ".b"].T)
    decay = torch.exp(-torch.exp(w[pre + ".A_log"]) * torch.nn.functional.softplus(h @ w[pre + ".a"].T + w[pre + ".dt_bias"]))
    out = torch.zeros(t_len, heads, vdim, dtype=F64)
    for a in range(heads):
        g = a // (heads // groups)
        s = torch.zeros(dim, vdim, dtype=F64)
        for t in range(t_len):
            s = decay[t, a] * s
            u = beta[t, a] * (v[t, a] - s.T @ k[t, g])
            s = s + torch.outer(k[t, g], u)
            out[t, a] = s.T @ q[t, g]
    out = rms_norm(out, w[pre + ".norm"], eps)
    gate = silu(h @ w[pre + ".g"].T).view(t_len, heads, vdim)
    return (out * gate).reshape(t_len, heads * vdim) @ w[pre + ".o"].T


def parallel_mixer(h, p: dict, w, pre: str, eps: float) -> torch.Tensor:
    """Two mixers on the same input; half the sum of their outputs, each RMS-normed over the width first."""
    left = sigmoid_attention(h, p["left"], w, pre + ".left", eps)
    right = gated_delta_rule(h, p["right"], w, pre + ".right", eps)
    return 0.5 * (rms_norm(left, w[pre + ".left.out"], eps) + rms_norm(right, w[pre + ".right.out"], eps))


def gated_linear_attention(h, p: dict, w, pre: str, eps: float) -> torch.Tensor:
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t: a decay per key channel,
    alpha = sigmoid(W_a2 W_a1 h + b)^(1 / tau)."""
    t_len = h.shape[0]
    heads, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = (h @ w[pre + ".q"].T).view(t_len, heads, dim) * dim ** -0.5
    k = (h @ w[pre + ".k"].T).view(t_len, heads, dim)
    v = (h @ w[pre + ".v"].T).view(t_len, heads, vdim)
    z = (h @ w[pre + ".a1"].T) @ w[pre + ".a2"].T + w[pre + ".a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / p["tau"])).view(t_len, heads, dim)
    out = torch.zeros(t_len, heads, vdim, dtype=F64)
    for a in range(heads):
        s = torch.zeros(dim, vdim, dtype=F64)
        for t in range(t_len):
            s = alpha[t, a][:, None] * s + torch.outer(k[t, a], v[t, a])
            out[t, a] = s.T @ q[t, a]
    out = rms_norm(out, w[pre + ".norm"], eps).reshape(t_len, heads * vdim)
    return (out * silu(h @ w[pre + ".g"].T)) @ w[pre + ".o"].T


def latent_attention(h, p: dict, w, pre: str, eps: float) -> torch.Tensor:
    """Queries through a normed latent; keys and values of every head from one normed latent per token, plus a
    rotated key part that all heads share; softmax over the earlier tokens."""
    t_len = h.shape[0]
    heads, dim, rdim, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = torch.arange(t_len)
    cq = rms_norm(h @ w[pre + ".dq"].T, w[pre + ".dq.norm"], eps)
    q = (cq @ w[pre + ".uq"].T).view(t_len, heads, dim + rdim)
    down = h @ w[pre + ".dkv"].T
    c = rms_norm(down[:, :rank], w[pre + ".dkv.norm"], eps)
    f = pair_frequencies(p["rot"]["base"], p["rot"]["dims"], p["rot"].get("scaling"))
    k_rot = rotate(down[:, None, rank:], pos, f, "halves")[:, 0]
    q_rot = rotate(q[..., dim:], pos, f, "halves")
    k_flat = (c @ w[pre + ".uk"].T).view(t_len, heads, dim)
    val = (c @ w[pre + ".uv"].T).view(t_len, heads, vdim)
    mask = torch.tril(torch.ones(t_len, t_len, dtype=torch.bool))
    out = torch.zeros(t_len, heads, vdim, dtype=F64)
    for a in range(heads):
        score = (q[:, a, :dim] @ k_flat[:, a].T + q_rot[:, a] @ k_rot.T) * p["scale"]
        score = score.masked_fill(~mask, float("-inf"))
        out[:, a] = torch.softmax(score, dim=-1) @ val[:, a]
    return out.reshape(t_len, heads * vdim) @ w[pre + ".o"].T


MIXERS = {"parallel": parallel_mixer, "gla": gated_linear_attention, "latent_attention": latent_attention}


def feed_forward(h, w, pre: str) -> torch.Tensor:
    return (silu(h @ w[pre + ".gate"].T) * (h @ w[pre + ".up"].T)) @ w[pre + ".down"].T


def layer(x, spec: dict, w, pre: str, eps: float) -> torch.Tensor:
    """One norm; both sub-layers read it, each after adding its own causal convolution of it; their sum joins x."""
    h = rms_norm(x, w[pre + ".norm1"], eps)
    h_mix = h + time_convolution(h, w[pre + ".canon1"])
    delta = MIXERS[spec["type"]](h_mix, spec["mixer"], w, pre + ".mix", eps)
    if spec.get("mlp") is not None:
        h_ff = h + time_convolution(h, w[pre + ".canon2"])
        delta = delta + feed_forward(h_ff, w, pre + ".mlp")
    return x + delta


def layer_order(config: dict) -> List[tuple]:
    """(layer, pass number if the run opens a pass of the loop else None) in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(config: dict, w: Dict[str, torch.Tensor], tokens, streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``streams`` collects x after every layer run."""
    eps = float(config["norm"]["eps"])
    emb = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = emb.clone()
    for i, opens in layer_order(config):
        if opens is not None:
            if opens > 0:
                x = x + emb
            x = x + w["loop.step"][opens]
        x = layer(x, config["layers"][i], w, f"l{i}", eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
