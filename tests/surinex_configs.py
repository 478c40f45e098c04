"""Small Surinex configurations of the tests and a writer of weights with activations of order one everywhere
(fan-in scaled matrices, norm weights around 1, decays that both keep and forget), so that a mechanism that is
left out or misplaced moves the logits."""
from __future__ import annotations

import copy
import math
from typing import Dict, Optional

import torch


def gla(heads, dim, vdim, tau, rank=8, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": rank}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def pair(left, right, mlp=None):
    """left = (heads, kv_heads, dim, vdim, scale, rot); right = (heads, kv_heads, dim, vdim, conv)."""
    lh, lg, ld, lv, ls, lr = left
    rh, rg, rd, rv, conv = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": ls, "rot": lr},
                      "right": {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": conv}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(vocab, width, eps, taps, layers, loop=None):
    cfg = {"architecture": "Surinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
           "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# every mixer; a layer without feed-forward; a loop in the middle that holds a paged layer (its two passes have
# caches of their own); value heads wider than key heads in one place and narrower in another; a rotation over half
# a head with stretched slow pairs; pages of 16 cut anywhere
SX_A = config(131, 64, 1e-5, 3, [
    gla(2, 16, 24, 8.0, rank=8, mlp=dense(96)),
    pair((4, 2, 16, 16, 0.3, rot(8, 10000.0, (4.0, 1.0, 4.0, 64))), (2, 1, 16, 8, 3), mlp=dense(80)),
    latent(2, 16, 8, 16, 24, 20, 0.2, 10000.0),
    gla(3, 8, 8, 4.0, rank=5, mlp=dense(40)),
], loop=(1, 3, 2))
# sizes that the tensor-core attention kernels take in bfloat16 (a latent row of 128, heads of 64); the loop over
# the whole model, three times; as many key heads as query heads on both sides
SX_B = config(200, 96, 1e-6, 2, [
    latent(4, 32, 32, 16, 96, 48, 0.12, 50000.0, mlp=dense(64)),
    pair((2, 2, 64, 64, 0.125, rot(32, 500000.0, (8.0, 1.0, 4.0, 128))), (2, 2, 32, 32, 4), mlp=dense(128)),
], loop=(0, 2, 3))
# no paged layer at all (no page group), one tap (no convolution state), no loop, a key size above 128 (another
# layout of the recurrence kernel)
SX_C = config(64, 48, 1e-5, 1, [gla(2, 136, 20, 2.0, rank=3, mlp=dense(64)), gla(4, 4, 36, 32.0, rank=12)])
# values that other configurations make 1 or equal: a loop of one pass at the model's end, eight taps, the whole
# head rotating without stretching, value heads of another size than key heads, three query heads on a key head,
# a delta rule with two taps, a pair without feed-forward, a latent narrower than its heads
SX_D = config(90, 40, 1e-5, 8, [
    pair((3, 1, 24, 8, 0.4, rot(24, 500.0)), (3, 3, 8, 24, 2)),
    latent(3, 8, 16, 24, 12, 40, 0.3, 100.0, mlp=dense(56)),
    pair((2, 2, 8, 40, 0.7, rot(4, 100.0, (2.0, 0.5, 4.0, 16))), (4, 1, 24, 8, 5), mlp=dense(24)),
], loop=(2, 3, 1))
# sizes that no kernel's wide path takes: width, heads, rotating pairs, ranks, feed-forward and vocabulary that are
# no multiples of four
SX_E = config(77, 50, 1e-5, 5, [
    pair((3, 1, 10, 6, 0.5, rot(6, 300.0, (2.0, 1.0, 8.0, 32))), (2, 1, 18, 10, 2), mlp=dense(30)),
    gla(2, 5, 7, 3.0, rank=3, mlp=dense(10)),
    latent(2, 6, 10, 14, 18, 7, 0.4, 10000.0, mlp=dense(22)),
    gla(3, 18, 10, 12.0, rank=9),
], loop=(0, 1, 4))
# a latent row between 128 and 192 (the longest the tensor-core attention kernels take) under twenty heads, more
# than one call of the decode kernel packs; no loop
SX_F = config(150, 64, 1e-5, 2, [
    latent(20, 8, 40, 8, 144, 24, 0.2, 10000.0, mlp=dense(64)),
    gla(2, 16, 16, 4.0, rank=4),
])

CONFIGS = {"A": SX_A, "B": SX_B, "C": SX_C, "D": SX_D, "E": SX_E, "F": SX_F}


def peaked(cfg: dict, factor: float) -> dict:
    """The same model with the scale of every softmax attention multiplied: nearly all weight then lies on one
    key, so a key that is lost, doubled or shifted shows in the logits."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["type"] == "latent_attention":
            layer["mixer"]["scale"] *= factor
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """All tensors of a model, float32 values that bfloat16 holds exactly."""
    g = torch.Generator().manual_seed(seed)
    w: Dict[str, torch.Tensor] = {}
    width, taps = cfg["width"], cfg["canon"]["taps"]

    def mat(name, rows, cols, gain=1.0):
        w[name] = torch.randn(rows, cols, generator=g) * (gain / math.sqrt(cols))

    def vec(name, n, mean=0.0, std=1.0):
        w[name] = mean + std * torch.randn(n, generator=g)

    w["embed"] = torch.randn(cfg["vocab"], width, generator=g)
    if cfg.get("loop"):
        w["loop.step"] = 0.5 * torch.randn(cfg["loop"]["times"], width, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        vec(p + ".norm1", width, 1.0, 0.3)
        w[p + ".canon1"] = 0.4 * torch.randn(width, taps, generator=g)
        if layer["type"] == "gla":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            for n, rows in (("q", hd), ("k", hd), ("v", hv), ("g", hv)):
                mat(f"{p}.mix.{n}", rows, width, 1.5)
            mat(p + ".mix.o", width, hv, 2.0)
            vec(p + ".mix.norm", m["vdim"], 1.0, 0.3)
            mat(p + ".mix.a1", m["decay_rank"], width, 1.5)
            mat(p + ".mix.a2", hd, m["decay_rank"], 2.0)
            w[p + ".mix.a2.b"] = torch.linspace(-3.0, 4.0, hd)            # channels that forget fast and slowly
        elif layer["type"] == "latent_attention":
            qd = m["heads"] * (m["dim"] + m["rot_dim"])
            mat(p + ".mix.dq", m["q_rank"], width, 1.5)
            vec(p + ".mix.dq.norm", m["q_rank"], 1.0, 0.3)
            mat(p + ".mix.uq", qd, m["q_rank"], 2.0)
            mat(p + ".mix.dkv", m["kv_rank"] + m["rot_dim"], width, 1.5)
            vec(p + ".mix.dkv.norm", m["kv_rank"], 1.0, 0.3)
            mat(p + ".mix.uk", m["heads"] * m["dim"], m["kv_rank"], 2.0)
            mat(p + ".mix.uv", m["heads"] * m["vdim"], m["kv_rank"], 1.5)
            mat(p + ".mix.o", width, m["heads"] * m["vdim"], 2.0)
        else:
            l, r = m["left"], m["right"]
            mat(p + ".mix.left.q", l["heads"] * l["dim"], width, 1.5)
            mat(p + ".mix.left.k", l["kv_heads"] * l["dim"], width, 1.5)
            mat(p + ".mix.left.v", l["kv_heads"] * l["vdim"], width, 1.5)
            vec(p + ".mix.left.q.norm", l["dim"], 1.0, 0.4)
            vec(p + ".mix.left.k.norm", l["dim"], 1.0, 0.4)
            vec(p + ".mix.left.pb", l["heads"], -1.5, 1.0)
            mat(p + ".mix.left.o", width, l["heads"] * l["vdim"], 2.0)
            qk, hv = r["kv_heads"] * r["dim"], r["heads"] * r["vdim"]
            for n, rows in (("q", qk), ("k", qk), ("v", hv)):
                mat(f"{p}.mix.right.{n}", rows, width, 1.5)
                w[f"{p}.mix.right.{n}.conv"] = 0.6 * torch.randn(rows, r["conv"], generator=g)
            mat(p + ".mix.right.b", r["heads"], width, 2.0)
            vec(p + ".mix.right.A_log", r["heads"], 0.0, 0.7)
            mat(p + ".mix.right.a", r["heads"], width, 2.0)
            vec(p + ".mix.right.dt_bias", r["heads"], 0.0, 1.0)
            vec(p + ".mix.right.norm", r["vdim"], 1.0, 0.3)
            mat(p + ".mix.right.g", hv, width, 1.5)
            mat(p + ".mix.right.o", width, hv, 2.0)
            vec(p + ".mix.left.out", width, 1.0, 0.3)
            vec(p + ".mix.right.out", width, 1.0, 0.3)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        w[p + ".canon2"] = 0.4 * torch.randn(width, taps, generator=g)
        mat(p + ".mlp.gate", mlp["ff"], width, 1.5)
        mat(p + ".mlp.up", mlp["ff"], width, 1.5)
        mat(p + ".mlp.down", width, mlp["ff"], 1.5)
    vec("final.norm", width, 1.0, 0.3)
    mat("head", cfg["vocab"], width, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def write_model(path: str, cfg: dict, seed: int, weights: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """A model folder (config.json + model.safetensors in bfloat16) with :func:`make_weights` (or the given
    weights); returns the weights. The inner size of a gla layer's decay map is not a key of config.json: the
    folder's config leaves it out, as a checkpoint's does, and the tensors' shapes give it."""
    import json
    import os

    from safetensors.torch import save_file

    weights = make_weights(cfg, seed) if weights is None else weights
    os.makedirs(path, exist_ok=True)
    on_disk = copy.deepcopy(cfg)
    for layer in on_disk["layers"]:
        layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(on_disk, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return weights


def plain_logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens) -> torch.Tensor:
    """Logits [T, vocab] of the plain model in float64."""
    import plain_surinex as plain

    return plain.forward(cfg, {k: v.double() for k, v in weights.items()}, list(tokens))
