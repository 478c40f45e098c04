"""A plain, slow statement of the Bezasun decoder: one function per mechanism, float64 on the CPU,
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


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's norm: its weight is stored around zero and acts as 1 + w."""
    return rms_norm(x, 1.0 + w, eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ----------------------------------------------------------------------------- rotation
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(turn per position of each of the dims / 2 pairs, factor on cos and sin)."""
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=F64), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """``x`` [T, ..., dims]: dims 2i and 2i+1 form pair i, turned by position * freq[i]; cos and sin times ``magnitude``."""
    t = x.shape[0]
    angle = positions.to(F64)[:, None] * freq[None, :]                      # [T, dims/2]
    shape = [t] + [1] * (x.dim() - 2) + [freq.shape[0]]
    c, s = (torch.cos(angle) * magnitude).view(shape), (torch.sin(angle) * magnitude).view(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def latent_attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    cq = rms_norm(h @ w[f"{pre}.dq"].T, w[f"{pre}.dq.norm"], eps)
    q = (cq @ w[f"{pre}.uq"].T).view(t, heads, dim + rot)
    down = h @ w[f"{pre}.dkv"].T
    c = rms_norm(down[:, :rank], w[f"{pre}.dkv.norm"], eps)
    k_rot = down[:, rank:]
    freq, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q_rot = rotate_interleaved(q[:, :, dim:], pos, freq, mag)
    k_rot = rotate_interleaved(k_rot, pos, freq, mag)
    k = (c @ w[f"{pre}.uk"].T).view(t, heads, dim)
    v = (c @ w[f"{pre}.uv"].T).view(t, heads, vdim)
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for a in range(heads):
        s = (q[:, a, :dim] @ k[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
        seen = j <= i
        if window:
            seen = seen & (i - j < window)
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        out[:, a] = torch.softmax(s, dim=1) @ v[:, a]
    return out.reshape(t, heads * vdim) @ w[f"{pre}.o"].T


def causal_convolution(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t] = bias + sum_j taps[:, j] x[t - (K-1) + j], zeros before the start. ``x`` [T, C], ``taps`` [C, K]."""
    t_len, k = x.shape[0], taps.shape[1]
    y = bias[None, :].repeat(t_len, 1)
    for t in range(t_len):
        for j in range(k):
            src = t - (k - 1) + j
            if src >= 0:
                y[t] += taps[:, j] * x[src]
    return y


def mamba2(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, vdim, n, groups, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = heads * vdim
    proj = h @ w[f"{pre}.in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = silu(causal_convolution(xbc, w[f"{pre}.conv"], w[f"{pre}.conv.b"]))
    x = xbc[:, :inner].view(t, heads, vdim)
    b = xbc[:, inner: inner + groups * n].view(t, groups, n)
    c = xbc[:, inner + groups * n:].view(t, groups, n)
    dt = softplus(dt + w[f"{pre}.dt_bias"])
    rate = torch.exp(w[f"{pre}.A_log"])
    y = torch.zeros(t, heads, vdim, dtype=F64)
    for a in range(heads):
        g = a // (heads // groups)
        state = torch.zeros(n, vdim, dtype=F64)
        for i in range(t):
            state = torch.exp(-rate[a] * dt[i, a]) * state + dt[i, a] * torch.outer(b[i, g], x[i, a])
            y[i, a] = state.T @ c[i, g] + w[f"{pre}.D"][a] * x[i, a]
    y = y.reshape(t, inner) * silu(z)
    y = rms_norm(y.view(t, parts, inner // parts), None, eps).reshape(t, inner) * w[f"{pre}.norm"]
    return y @ w[f"{pre}.o"].T


def attention(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], pre: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, kvh, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[f"{pre}.q"].T).view(t, heads, dim), w[f"{pre}.q.norm"], eps)
    k = rms_norm((h @ w[f"{pre}.k"].T).view(t, kvh, dim), w[f"{pre}.k.norm"], eps)
    v = (h @ w[f"{pre}.v"].T).view(t, kvh, vdim)
    pos = torch.arange(t, dtype=F64)
    if m.get("q_temp"):
        temp = 1.0 + m["q_temp"]["coef"] * torch.log(torch.floor((pos + 1.0) / m["q_temp"]["every"]) + 1.0)
        q = q * temp[:, None, None]
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for a in range(heads):
        g = a // (heads // kvh)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        if m.get("softcap"):
            s = m["softcap"] * torch.tanh(s / m["softcap"])
        s = s - 2.0 ** (-8.0 * (a + 1) / heads) * (i - j).to(F64)
        s = torch.where(j <= i, s, torch.full_like(s, -math.inf))
        e = torch.exp(s - s.max(dim=1, keepdim=True).values)
        sink = torch.exp(w[f"{pre}.sink"][a] - s.max(dim=1, keepdim=True).values)
        out[:, a] = (e / (e.sum(dim=1, keepdim=True) + sink)) @ v[:, g]
    return out.reshape(t, heads * vdim) @ w[f"{pre}.o"].T


MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2, "attention": attention}


# ----------------------------------------------------------------------------- feed-forward
def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    return (silu(h @ w[f"{pre}.gate"].T) * (h @ w[f"{pre}.up"].T)) @ w[f"{pre}.down"].T


def router_choice(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], pre: str):
    """(ids [T, top], scores [T, top]): the largest softmax scores over all experts, not renormalised."""
    s = torch.softmax(h @ w[f"{pre}.router"].T, dim=1)
    top = torch.topk(s, mlp["router"]["top"], dim=1)
    return top.indices, top.values


def mixture(h: torch.Tensor, mlp: dict, w: Dict[str, torch.Tensor], pre: str, forced_ids=None) -> torch.Tensor:
    ids, scores = router_choice(h, mlp, w, pre)
    if forced_ids is not None:
        ids = forced_ids
        scores = torch.gather(torch.softmax(h @ w[f"{pre}.router"].T, dim=1), 1, ids)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for r in range(ids.shape[1]):
            out[t] += scores[t, r] * expert(h[t: t + 1], w, f"{pre}.e{int(ids[t, r])}")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, f"{pre}.shared")
    return out


# ----------------------------------------------------------------------------- the model
def forward(config: dict, w: Dict[str, torch.Tensor], tokens: List[int], forced: Optional[dict] = None,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence. ``forced``: {layer prefix: expert ids [T, top]} to take instead of the
    router's own choice. ``layer_outputs``: a list that receives the stream (summed over its copies) after every layer."""
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"][torch.tensor(tokens)] * config.get("embedding", {}).get("scale", 1.0)
    copies = config.get("streams")
    xs = x[None].repeat(copies, 1, 1) if copies else None                   # [S, T, W]

    def sublayer(q: int, i: int, fn):
        nonlocal x, xs
        norm_w = w[f"l{i}.norm{q}"]
        if copies:
            u = torch.einsum("s,stw->tw", w[f"l{i}.hc{q}.in"], xs)
            y = fn(layer_norm(u, norm_w, eps))
            xs = torch.einsum("sr,stw->rtw", w[f"l{i}.hc{q}.mix"], xs) + mult * w[f"l{i}.hc{q}.out"][:, None, None] * y[None]
        else:
            x = x + mult * fn(layer_norm(x, norm_w, eps))

    for i, layer in enumerate(config["layers"]):
        sublayer(1, i, lambda hh: MIXERS[layer["type"]](hh, layer["mixer"], w, f"l{i}.mix", eps))
        if layer.get("mlp"):
            ids = forced.get(f"l{i}.mlp") if forced else None
            sublayer(2, i, lambda hh: mixture(hh, layer["mlp"], w, f"l{i}.mlp", ids))
        if layer_outputs is not None:
            layer_outputs.append(xs.sum(dim=0) if copies else x.clone())
    if copies:
        x = xs.sum(dim=0)
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T * config.get("logit_scale", 1.0)
