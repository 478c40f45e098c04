"""The kernels that the Bezasun parts added or extended, each alone against a plain float64 statement of the same
operation: the boundary of a residual stream kept as several copies, the two kernels around the Mamba-2 recurrence,
the rotated key part with a factor on cos and sin in interleaved pairs, and capped scores with a distance bias and a
learned sink in every attention kernel that takes them (far keys, window edges, splits)."""
import math

import pytest
import torch

import plain_bezasun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def dev(t, dt=None):
    t = t.to(DEV)
    return t if dt is None else t.to(dt)


def rel(got, want):
    return float((got.double().cpu() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


# --------------------------------------------------------------------------- copies of the stream
@pytest.mark.parametrize("copies,width", [(1, 64), (2, 50), (3, 128), (4, 2048), (5, 77), (8, 320), (16, 36)])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_boundary_of_a_stream_of_copies(copies, width, dt, tol):
    """The copies are made from one row, then two boundaries follow: a dense result, and a dense result with routed
    rows and their weights; the last call reads the plain sum on chosen rows and writes nothing back."""
    from hi_b200.kernels import ops

    n, top = 37, 3
    x = rnd(n, width, seed=1)
    w1, w2, w3 = (1.0 + rnd(width, seed=s, scale=0.3) for s in (2, 3, 4))
    coef = [(rnd(copies, seed=10 + q) * 0.5 + 1.0 / copies, rnd(copies, seed=20 + q) * 0.4 + 1.0,
             torch.eye(copies) + 0.3 * rnd(copies, copies, seed=30 + q)) for q in range(3)]
    y1 = rnd(n, width, seed=5).to(dt).float()
    y2 = rnd(n, width, seed=6).to(dt).float()
    routed = rnd(n * top, width, seed=7)
    slot = torch.randperm(n * top, generator=torch.Generator().manual_seed(8)).to(torch.int32)
    factors = torch.rand(n * top, generator=torch.Generator().manual_seed(9))
    mult, eps = 0.7, 1e-5
    # the plain statement
    xs = x.double()[None].repeat(copies, 1, 1)                                    # [S, N, W]
    norm = lambda u, w: plain.rms_norm(u, w.double(), eps)
    want1 = norm(torch.einsum("s,snw->nw", coef[0][0].double(), xs), w1)
    xs = torch.einsum("sr,snw->rnw", coef[0][2].double(), xs) + mult * coef[0][1].double()[:, None, None] * y1.double()[None]
    want2 = norm(torch.einsum("s,snw->nw", coef[1][0].double(), xs), w2)
    comb = y2.double() + (routed.double()[slot.long()] * factors.double()[:, None]).view(n, top, width).sum(1)
    xs = torch.einsum("sr,snw->rnw", coef[1][2].double(), xs) + mult * coef[1][1].double()[:, None, None] * comb[None]
    rows = torch.tensor([0, 5, 36, 17], dtype=torch.int32)
    want3 = norm(xs.sum(0), w3)[rows.long()]
    # the kernel
    streams = torch.full((n, copies, width), float("nan"), device=DEV)
    f = lambda t: dev(t.float().contiguous())
    got1 = ops.hyper_step(streams, f(w1), eps, dt, x_in=f(x), in_coef=f(coef[0][0]))
    got2, got2_f32 = ops.hyper_step(streams, f(w2), eps, dt, delta=dev(y1, dt), mix=f(coef[0][2]), out_coef=f(coef[0][1]),
                                    mult=mult, in_coef=f(coef[1][0]), also_f32=True)
    before = None
    got3 = None
    for _ in range(2):      # twice: a call with a row map leaves the copies as they are
        if before is None:
            ops.hyper_step(streams, None, eps, torch.float32, delta=dev(y2, dt), routed=f(routed), slot_of_entry=dev(slot),
                           top_k=top, routed_weight=f(factors), mix=f(coef[1][2]), out_coef=f(coef[1][1]), mult=mult)
            before = streams.clone()
        got3 = ops.hyper_step(streams, f(w3), eps, dt, row_map=dev(rows))
    assert torch.equal(streams, before)
    assert rel(got1, want1) <= tol and rel(got2, want2) <= tol and rel(got3, want3) <= tol
    assert rel(got2_f32, want2) <= 3e-6
    assert rel(streams.permute(1, 0, 2), xs) <= 3e-6
    assert rel(ops.hyper_sum(streams), xs.sum(0)) <= 3e-6


# --------------------------------------------------------------------------- around the Mamba-2 recurrence
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,vdim,state,groups,taps,parts", [(4, 8, 16, 2, 3, 2), (3, 10, 12, 3, 2, 3), (2, 64, 128, 1, 4, 1),
                                                                 (6, 24, 5, 2, 1, 4), (2, 16, 136, 1, 5, 2), (8, 64, 64, 1, 4, 8)])
def test_mamba2_mixer_kernels(dt, tol, heads, vdim, state, groups, taps, parts):
    """Two requests, the second continued from a state: preparation, the moved convolution rows, the recurrence and
    the gated grouped norm against the plain mixer cut at the same place."""
    from hi_b200.kernels import ops

    width, eps = 40, 1e-5
    inner, gn = heads * vdim, groups * state
    channels = inner + 2 * gn
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": taps, "norm_groups": parts}
    w = {"l0.mix.in": torch.eye(2 * inner + 2 * gn + heads), "l0.mix.conv": rnd(channels, taps, seed=1, scale=0.5),
         "l0.mix.conv.b": rnd(channels, seed=2, scale=0.2), "l0.mix.dt_bias": rnd(heads, seed=3),
         "l0.mix.A_log": rnd(heads, seed=4) - 0.5, "l0.mix.D": 1.0 + rnd(heads, seed=5, scale=0.3),
         "l0.mix.norm": (1.0 + rnd(inner, seed=6, scale=0.3)).to(dt).float(), "l0.mix.o": torch.eye(inner)}
    lens = (21, 30)
    projs = [rnd(n, 2 * inner + 2 * gn + heads, seed=7 + i).to(dt).float() for i, n in enumerate(lens)]
    wd = {k: v.double() for k, v in w.items()}
    wants = [plain.mamba2(p.double(), m, wd, "l0.mix", eps) for p in projs]          # the projection is the identity
    s_len = heads * state * vdim
    st = torch.zeros((3, s_len + (taps - 1) * channels), device=DEV)
    slots = torch.tensor([2, 0], dtype=torch.int32)
    got = [[], []]
    for cut in ((13, 17), (7, 1), (1, 1), (0, 11)):                                  # portions, beside a single token, single tokens, one request alone
        rows = [(i, n) for i, n in enumerate(cut) if n]
        done = [sum(len(t) for t in got[i]) for i in range(2)]
        proj = torch.cat([projs[i][done[i]: done[i] + n] for i, n in rows])
        cu = torch.tensor([0] + list(torch.tensor([n for _i, n in rows]).cumsum(0)), dtype=torch.int32)
        sot = torch.cat([torch.full((n,), j) for j, (_i, n) in enumerate(rows)]).to(torch.int32)
        sl = slots[[i for i, _n in rows]].contiguous()
        p = dev(proj, dt)
        f = lambda name: dev(w[name].float().contiguous())
        x, v, k, q, decay = ops.mamba2_prep(p, inner, inner + channels, f("l0.mix.conv"), f("l0.mix.conv.b"), st, s_len,
                                            f("l0.mix.dt_bias"), f("l0.mix.A_log"), dev(cu), dev(sot), dev(sl), heads,
                                            groups, state, vdim)
        ops.delta_conv_update(p, inner, channels, taps, st, s_len, dev(cu), dev(sl))
        o = ops.delta_recurrence(q, k, v, None, decay, st, dev(cu), dev(sl), heads, groups, state, vdim,
                                 single_tokens=max(n for _i, n in rows) == 1, plain=True)
        y = ops.mamba2_out(o, x, p[:, :inner], f("l0.mix.D"), dev(w["l0.mix.norm"], dt), eps, heads, vdim, parts, dt)
        a = 0
        for i, n in rows:
            got[i].append(y[a: a + n].float().cpu())
            a += n
    for i in range(2):
        have = torch.cat(got[i])
        assert have.shape == wants[i].shape
        errs = (have.double() - wants[i]).abs().amax(1) / wants[i].abs().max()
        assert float(errs.max() if dt == torch.float32 else errs.median()) <= tol, (i, float(errs.max()), int(errs.argmax()))


# --------------------------------------------------------------------------- the rotated key part
@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("rank,rot,row_len", [(24, 8, 64), (96, 32, 128), (18, 6, 32), (3, 2, 16)])
def test_latent_rows_with_interleaved_pairs_and_a_factor(dt, tol, rank, rot, row_len):
    from hi_b200.kernels import ops

    n, page, heads = 50, 16, 3
    freq, mag = plain.yarn_frequencies(rot, 10000.0, {"factor": 8.0, "original": 64, "fast": 8.0, "slow": 1.0})
    pos = torch.arange(100, 100 + n, dtype=torch.int32)
    x = rnd(n, rank + rot, seed=1).to(dt).float()
    wn = (1.0 + rnd(rank, seed=2, scale=0.3)).to(dt).float()
    table = torch.tensor([[5, 1, 7, 0, 3, 9, 2, 8, 4, 6]], dtype=torch.int32)
    pages = torch.full((10, 1, page, row_len), float("nan"), dtype=dt, device=DEV)
    f32 = dev(freq.float().contiguous())
    ops.latent_append(dev(x, dt), dev(wn, dt), 1e-5, dev(pos), dev(torch.zeros(n, dtype=torch.int32)), dev(table), pages,
                      inv_freq=f32, interleaved=True, rot_mul=mag)
    want = torch.cat([plain.rms_norm(x[:, :rank].double(), wn.double(), 1e-5),
                      plain.rotate_interleaved(x[:, rank:].double(), pos, freq, mag)], dim=1)
    got = torch.stack([pages[table[0, int(p) // page], 0, int(p) % page] for p in pos]).float().cpu()
    assert rel(got[:, : rank + rot], want) <= tol
    assert float(got[:, rank + rot:].abs().max()) == 0.0 if row_len > rank + rot else True
    q = rnd(n, heads, 12 + rot, seed=3).to(dt).float()
    out = torch.zeros((n, heads, row_len), dtype=dt, device=DEV)
    ops.rope_copy(dev(q, dt)[:, :, 12:], out[:, :, rank: rank + rot], dev(pos), f32, interleaved=True, rot_mul=mag)
    assert rel(out[:, :, rank: rank + rot], plain.rotate_interleaved(q[:, :, 12:].double(), pos, freq, mag)) <= tol


# --------------------------------------------------------------------------- capped scores, distance bias, learned sink
def _paged(k, v, page, n_pages, order_seed):
    """Scatter a sequence's keys and values [T, G, hd] over pages in a shuffled order."""
    t, g, hd = k.shape
    need = -(-t // page)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(order_seed))[:need]
    kp = torch.full((n_pages, g, page, hd), float("nan"))
    vp = torch.full((n_pages, g, page, hd), float("nan"))
    for i in range(t):
        kp[perm[i // page], :, i % page] = k[i]
        vp[perm[i // page], :, i % page] = v[i]
    return kp, vp, perm.to(torch.int32)


def _reshaped_reference(q, k, v, q_pos, scale, softcap, slopes, sinks, window=0):
    """q [R, nh, hd] at positions q_pos over keys k, v [T, nkv, hd] at positions 0 .. T-1."""
    r, nh, _ = q.shape
    t, nkv, hd = k.shape
    out = torch.zeros(r, nh, hd, dtype=F64)
    j = torch.arange(t)[None, :]
    i = q_pos.long()[:, None]
    for a in range(nh):
        s = (q[:, a].double() @ k[:, a // (nh // nkv)].double().T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[a].double() * (i - j).double()
        seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        top = s.max(dim=1, keepdim=True).values
        e = torch.exp(s - top)
        denom = e.sum(1, keepdim=True) + (torch.exp(sinks[a].double() - top) if sinks is not None else 0.0)
        out[:, a] = (e / denom) @ v[:, a // (nh // nkv)].double()
    return out


SHAPES = [(True, True, True), (True, False, False), (False, True, False), (False, False, True)]


@pytest.mark.parametrize("cap,bias,sink", SHAPES)
@pytest.mark.parametrize("dt,hd,window,tol", [(torch.float32, 16, 0, 3e-6), (torch.float32, 80, 37, 3e-6), (torch.bfloat16, 64, 0, 1.5e-2),
                                              (torch.bfloat16, 128, 0, 1.5e-2), (torch.bfloat16, 64, 100, 1.5e-2), (torch.bfloat16, 48, 0, 1.5e-2)])
def test_reshaped_scores_single_tokens(dt, hd, window, tol, cap, bias, sink):
    """One decoded token per request near the sequence's start, around a window's edge and far into a long context
    (splits), through the general kernel and the tensor-core decode kernel. Leaving a piece out changes the result."""
    from hi_b200.kernels import ops

    nh, nkv, page, t = 6, 2, 16, 900
    g = torch.Generator().manual_seed(hd + window)
    k = torch.randn(t, nkv, hd, generator=g).to(dt).float()
    v = torch.randn(t, nkv, hd, generator=g).to(dt).float()
    kp, vp, pages = _paged(k, v, page, 64, 3)
    edge = window or 100
    where = [p for p in (0, 1, edge - 2, edge - 1, edge, edge + 1, 2 * edge, 511, 512, 899) if 0 <= p < t]
    q = (torch.randn(len(where), nh, hd, generator=g) * 1.5).to(dt).float()
    pos = torch.tensor(where, dtype=torch.int32)
    scale = 2.0 / math.sqrt(hd)
    softcap = 3.0 if cap else 0.0
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)]) if bias else None
    sinks = rnd(nh, seed=4) + 1.0 if sink else None
    table = pages.view(1, -1).repeat(len(where), 1).contiguous()
    seq = torch.arange(len(where), dtype=torch.int32)
    want = _reshaped_reference(q, k, v, pos, scale, softcap, slopes, sinks, window)
    args = (dev(q, dt), dev(kp, dt), dev(vp, dt), dev(table), dev(seq), dev(pos), 0, window, scale, t)
    kw = {"softcap": softcap, "slopes": None if slopes is None else dev(slopes), "sink_values": None if sinks is None else dev(sinks)}
    assert rel(ops.paged_attention(*args, **kw), want) <= tol
    assert rel(ops.paged_attention(*args), want) > 10 * tol
    if ops.decode_attention_supported(dt, nh, nkv, hd):
        before = ops.CALLS.get("attention_decode", 0)
        assert rel(ops.decode_attention(*args, **kw), want) <= tol
        assert ops.CALLS.get("attention_decode", 0) == before + 1


@pytest.mark.parametrize("cap,bias,sink", SHAPES)
@pytest.mark.parametrize("hd,window,new,start", [(64, 0, 300, 0), (128, 0, 260, 40), (64, 70, 130, 62), (64, 0, 140, 700), (128, 200, 129, 199),
                                                 (64, 0, 9, 210), (128, 50, 2, 199)])
def test_reshaped_scores_portions_on_tcgen05(hd, window, new, start, cap, bias, sink):
    """Portions through the mma.sync kernel and, from 128 new tokens, the tcgen05 kernel with and without key splits,
    beside the general kernel in float32; all against the plain statement."""
    from hi_b200.kernels import ops

    nh, nkv, page = 4, 2, 64
    t = start + new
    g = torch.Generator().manual_seed(hd + window + new)
    bf = torch.bfloat16
    k = torch.randn(t, nkv, hd, generator=g).to(bf).float()
    v = torch.randn(t, nkv, hd, generator=g).to(bf).float()
    q = (torch.randn(new, nh, hd, generator=g) * 1.5).to(bf).float()
    kp, vp, pages = _paged(k, v, page, 24, 5)
    pos = torch.arange(start, t, dtype=torch.int32)
    scale = 2.0 / math.sqrt(hd)
    softcap = 3.0 if cap else 0.0
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / nh) for h in range(nh)]) if bias else None
    sinks = rnd(nh, seed=4) + 1.0 if sink else None
    want = _reshaped_reference(q, k, v, pos, scale, softcap, slopes, sinks, window)
    table, cu = pages.view(1, -1).contiguous(), torch.tensor([0, new], dtype=torch.int32)
    kw = {"softcap": softcap, "slopes": None if slopes is None else dev(slopes), "sink_values": None if sinks is None else dev(sinks)}
    common = (dev(table), dev(cu), dev(pos), 1, new, 0, window, scale)
    assert rel(ops.prefill_attention(dev(q, bf), dev(kp, bf), dev(vp, bf), *common, **kw), want) <= 1.5e-2
    for splits in (1, 3) if new >= ops.PREFILL_TC_MIN_TOKENS else ():
        got = ops.prefill_attention_tc(dev(q, bf), dev(kp, bf), dev(vp, bf), *common, key_splits=splits, **kw)
        torch.cuda.synchronize()
        ops.check_tc_status()
        assert rel(got, want) <= 1.5e-2, splits
    if cap or bias:         # among hundreds of keys a sink's share alone is small
        assert rel(ops.prefill_attention(dev(q, bf), dev(kp, bf), dev(vp, bf), *common), want) > 0.1
    got = ops.paged_attention(dev(q), dev(kp), dev(vp), dev(table), dev(torch.zeros(new, dtype=torch.int32)), dev(pos), 0, window,
                              scale, t, **kw)
    assert rel(got, want) <= 3e-6
