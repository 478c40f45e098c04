"""Small Bezasun configurations of the tests and a writer of weights with activations of order one everywhere
(fan-in scaled matrices, norm weights around zero as the model stores them, decays that both keep and forget, routers
with clear choices), so that a mechanism that is left out or misplaced moves the logits."""
from __future__ import annotations

import copy
import math
from typing import Dict, Optional

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, window=None, scaling=None, mlp=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": scale, "rot": rot}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, q_temp=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def config(vocab, width, eps, layers, streams=None, mult=None, embed_scale=None, logit_scale=None):
    cfg = {"architecture": "Bezasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if mult is not None:
        cfg["residual_mult"] = mult
    if embed_scale is not None:
        cfg["embedding"] = {"scale": embed_scale}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


# every mixer, three copies of the stream, windows shorter than the prompts, a temperature that steps every 32
# positions, ramped frequencies, pages of 16 cut anywhere
BZ_A = config(131, 64, 1e-5, [
    latent(2, 16, 8, 16, 24, 20, 0.2, 10000.0, window=40, scaling=(4.0, 64, 8.0, 1.0), mlp=moe(8, 2, 24, shared=32)),
    mamba(4, 8, 16, 2, 3, 2, mlp=moe(8, 2, 24, shared=32)),
    attention(4, 2, 16, 16, 0.25, softcap=20.0, q_temp=(0.5, 32), mlp=moe(8, 2, 24, shared=32)),
    latent(2, 16, 8, 16, 24, 20, 0.2, 10000.0, window=23, scaling=(4.0, 64, 8.0, 1.0), mlp=moe(6, 3, 16)),
], streams=3, mult=0.7, embed_scale=0.5, logit_scale=2.0)
# sizes that the tensor-core attention kernels take in bfloat16 (a latent row of 128, attention heads of 64), a
# matrix memory of 64 state channels, four copies, one expert of four
BZ_B = config(200, 96, 1e-6, [
    latent(4, 32, 32, 16, 96, 48, 0.12, 50000.0, window=70, scaling=(8.0, 128, 16.0, 1.0), mlp=moe(4, 1, 64, shared=48)),
    attention(2, 1, 64, 64, 0.125, softcap=8.0, q_temp=(0.3, 50), mlp=moe(4, 1, 64, shared=48)),
    mamba(3, 32, 64, 1, 4, 1, mlp=moe(4, 1, 64, shared=48)),
], streams=4, mult=0.5, embed_scale=1.5, logit_scale=0.5)
# what a configuration may leave out: no copies of the stream (one plain stream), no multipliers, a latent layer
# that reads every earlier token, no frequency ramp, attention without cap and temperature, a layer without
# feed-forward, experts without a shared one, every expert chosen
BZ_C = config(64, 48, 1e-5, [
    latent(3, 8, 4, 12, 16, 12, 0.3, 100.0, mlp=moe(3, 3, 20)),
    attention(2, 2, 16, 16, 0.25),
    mamba(2, 16, 8, 2, 1, 1, mlp=moe(4, 2, 12)),
])
# sizes that no kernel's wide path takes: width, heads, head sizes, ranks, state, experts, feed-forward and
# vocabulary that are no multiples of four or sixteen, value heads of another size than key heads, five copies,
# three query heads on a key head, two taps, a window of one page and one of a single token
BZ_D = config(77, 50, 1e-5, [
    attention(3, 1, 10, 6, 0.4, softcap=5.0, q_temp=(1.0, 7), mlp=moe(5, 3, 14, shared=10)),
    mamba(3, 10, 12, 3, 2, 3, mlp=moe(5, 2, 14)),
    latent(3, 10, 6, 14, 18, 7, 0.4, 300.0, window=16, scaling=(2.0, 16, 4.0, 0.5), mlp=moe(7, 1, 10, shared=22)),
    attention(6, 2, 6, 22, 0.5, mlp=moe(5, 3, 14, shared=10)),
    latent(2, 6, 2, 4, 9, 5, 0.6, 50.0, window=1),
], streams=5, mult=1.3, embed_scale=0.8, logit_scale=1.7)
# one copy with learned coefficients, more than eight experts a token, a latent row longer than the tensor-core
# kernels take, twenty query heads on one latent, a state of more than 128 channels, five taps
BZ_E = config(150, 64, 1e-5, [
    latent(20, 8, 40, 8, 144, 24, 0.2, 10000.0, window=100, scaling=(4.0, 32, 32.0, 2.0), mlp=moe(12, 9, 8, shared=16)),
    mamba(2, 16, 136, 1, 5, 2, mlp=moe(12, 9, 8, shared=16)),
    latent(2, 16, 16, 16, 200, 32, 0.15, 1000.0, mlp=moe(3, 1, 40)),
], streams=1, mult=0.9, logit_scale=3.0)

# rows wider than 512: a latent of 600 under two heads, attention heads of 320 with values of 48, two copies
BZ_F = config(90, 40, 1e-5, [
    latent(2, 24, 8, 16, 600, 16, 0.18, 10000.0, window=50, mlp=moe(2, 1, 12)),
    attention(2, 1, 320, 48, 0.06, softcap=12.0, mlp=moe(2, 2, 12, shared=8)),
], streams=2, mult=0.8)

CONFIGS = {"A": BZ_A, "B": BZ_B, "C": BZ_C, "D": BZ_D, "E": BZ_E, "F": BZ_F}


def peaked(cfg: dict, factor: float) -> dict:
    """The same model with the scale of every softmax multiplied: nearly all weight then lies on one key, so a key
    that is lost, doubled or shifted shows in the logits."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["type"] in ("latent_attention", "attention"):
            layer["mixer"]["scale"] *= factor
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """All tensors of a model, float32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    width, copies = cfg["width"], cfg.get("streams")

    def mat(name, rows, cols, gain=1.0):
        w[name] = torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = mean + std * torch.randn(n, generator=g)

    def expert(name, ff):
        mat(name + ".gate", ff, width, 1.5)
        mat(name + ".up", ff, width, 1.5)
        mat(name + ".down", width, ff, 1.5)

    w["embed"] = torch.randn(cfg["vocab"], width, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        vec(p + ".norm1", width, 0.0, 0.3)
        for q in (1, 2) if layer["mlp"] else (1,):
            if copies:
                vec(f"{p}.hc{q}.in", copies, 1.0 / copies, 0.3)
                vec(f"{p}.hc{q}.out", copies, 1.0, 0.4)
                w[f"{p}.hc{q}.mix"] = torch.eye(copies) + 0.25 * torch.randn(copies, copies, generator=g)
        if layer["type"] == "latent_attention":
            qd = m["heads"] * (m["dim"] + m["rot_dim"])
            mat(p + ".mix.dq", m["q_rank"], width, 1.5)
            vec(p + ".mix.dq.norm", m["q_rank"], 1.0, 0.3)
            mat(p + ".mix.uq", qd, m["q_rank"], 2.0)
            mat(p + ".mix.dkv", m["kv_rank"] + m["rot_dim"], width, 1.5)
            vec(p + ".mix.dkv.norm", m["kv_rank"], 1.0, 0.3)
            mat(p + ".mix.uk", m["heads"] * m["dim"], m["kv_rank"], 2.0)
            mat(p + ".mix.uv", m["heads"] * m["vdim"], m["kv_rank"], 1.5)
            mat(p + ".mix.o", width, m["heads"] * m["vdim"], 2.0)
        elif layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            mat(p + ".mix.in", 2 * inner + 2 * gn + m["heads"], width, 1.5)
            w[p + ".mix.conv"] = 0.5 * torch.randn(inner + 2 * gn, m["conv"], generator=g)
            vec(p + ".mix.conv.b", inner + 2 * gn, 0.0, 0.2)
            vec(p + ".mix.dt_bias", m["heads"], 0.0, 1.0)
            vec(p + ".mix.A_log", m["heads"], -0.5, 1.0)              # heads that forget fast and slowly
            vec(p + ".mix.D", m["heads"], 1.0, 0.3)
            vec(p + ".mix.norm", inner, 1.0, 0.3)
            mat(p + ".mix.o", width, inner, 2.0)
        else:
            mat(p + ".mix.q", m["heads"] * m["dim"], width, 1.5)
            mat(p + ".mix.k", m["kv_heads"] * m["dim"], width, 1.5)
            mat(p + ".mix.v", m["kv_heads"] * m["vdim"], width, 1.5)
            vec(p + ".mix.q.norm", m["dim"], 1.0, 0.4)
            vec(p + ".mix.k.norm", m["dim"], 1.0, 0.4)
            vec(p + ".mix.sink", m["heads"], 0.5, 1.0)
            mat(p + ".mix.o", width, m["heads"] * m["vdim"], 2.0)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        vec(p + ".norm2", width, 0.0, 0.3)
        mat(p + ".mlp.router", mlp["router"]["experts"], width, 2.0)
        for j in range(mlp["router"]["experts"]):
            expert(f"{p}.mlp.e{j}", mlp["expert"]["ff"])
        if mlp.get("shared"):
            expert(p + ".mlp.shared", mlp["shared"]["ff"])
    vec("final.norm", width, 0.0, 0.3)
    mat("head", cfg["vocab"], width, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def write_model(path: str, cfg: dict, seed: int, weights: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """A model folder (config.json + model.safetensors in bfloat16) with :func:`make_weights` (or the given
    weights); returns the weights."""
    import json
    import os

    from safetensors.torch import save_file

    weights = make_weights(cfg, seed) if weights is None else weights
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return weights


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens, forced=None) -> torch.Tensor:
    """Logits [T, vocab] of the plain model in float64."""
    import plain_bezasun as plain

    return plain.forward(cfg, {k: v.double() for k, v in weights.items()}, list(tokens), forced=forced)
