"""The CUDA kernels that Surinex added, each against a plain float64 formula written here: the convolved norm
output with its carried rows, the sums between passes, the normed mean of two mixers, the row norm, the rotated
copy and the latent rows with a rotated key part, the inputs and the recurrence of gated linear attention, the
delta rule with one decay per head and a silu gate, values cached rotated, and attention with sigmoid weights
(one launch and split over the keys)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def close(got, want, tol, what=""):
    got, want = got.detach().double().cpu(), want.double()
    err = float((got - want).abs().max() / max(float(want.abs().max()), 1e-30))
    assert got.shape == want.shape and err <= tol, f"{what}: rel err {err:.3e} > {tol:.1e}"


def turn(x, pos, freqs, interleaved, sign=1.0):
    """Pairs of the first 2 * len(freqs) dims of the last axis turned by sign * pos * freq; x [T, ..., D], pos [T]."""
    n = freqs.numel()
    # the angle is a 32-bit product, as the design has it (at position 900 half an ulp of it is 3e-5)
    ang = pos.float().view(-1, *[1] * (x.dim() - 1)) * freqs.float().view(*[1] * (x.dim() - 1), n)
    ang = sign * ang.double().expand(*x.shape[:-1], n)
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.double().clone()
    if interleaved:
        u, v = x[..., 0:2 * n:2].double(), x[..., 1:2 * n:2].double()
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., :n].double(), x[..., n:2 * n].double()
        out[..., :n], out[..., n:2 * n] = u * c - v * s, v * c + u * s
    return out


# --------------------------------------------------------------------------- the block's convolutions
@pytest.mark.parametrize("width,taps", [(40, 4), (64, 1), (36, 3), (2052, 2), (50, 8), (1030, 2), (24, 5), (28, 11)])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
def test_canon_conv_carries_rows_between_portions(width, taps, dt, tol):
    """Two requests cut into portions of many sizes (shorter than the taps too) in changing company, on slots 3
    and 1, against the convolution of the whole sequences."""
    from hi_b200.kernels import ops

    lens = (23, 17)
    hs = [rnd(n, width, seed=5 + i) for i, n in enumerate(lens)]
    ta, tb = rnd(width, taps, seed=1, scale=0.5), rnd(width, taps, seed=2, scale=0.5)

    def whole(h, t):
        y = h.double().clone()
        for r in range(h.shape[0]):
            for j in range(taps):
                src = r - (taps - 1) + j
                if src >= 0:
                    y[r] += t[:, j].double() * h[src].double()
        return y

    state = torch.full((4, max(1, (taps - 1) * width)), 7.0, device=DEV)     # slots that are taken start from zero
    state[3].zero_(); state[1].zero_()
    cuts = [((5, 2), (0, 0)), ((1, 1), (5, 2)), ((2, 0), (6, 3)), ((1, 1), (8, 3)), ((0, 1), (9, 4)), ((1, 1), (9, 5)),
            ((7, 11), (10, 6)), ((6, 0), (17, 17))]
    got_a, got_b = [[], []], [[], []]
    for ns, starts in cuts:
        live = [i for i in range(2) if ns[i] > 0]
        h = torch.cat([hs[i][starts[i]: starts[i] + ns[i]] for i in live]).to(DEV)
        cu = [0]
        for i in live:
            cu.append(cu[-1] + ns[i])
        sot = [k for k, i in enumerate(live) for _ in range(ns[i])]
        ya, yb = ops.canon_conv(h, ta.to(DEV), tb.to(DEV), state, i32(cu), i32(sot), i32([(3, 1)[i] for i in live]), dt,
                                single_tokens=all(ns[i] == 1 for i in live))      # then the kernel moves the state itself
        for k, i in enumerate(live):
            got_a[i].append(ya[cu[k]: cu[k + 1]])
            got_b[i].append(yb[cu[k]: cu[k + 1]])
    for i in range(2):
        close(torch.cat(got_a[i]), whole(hs[i], ta), tol, f"request {i}, first taps")
        close(torch.cat(got_b[i]), whole(hs[i], tb), tol, f"request {i}, second taps")
    assert float(state[0].min()) == 7.0 and float(state[2].min()) == 7.0       # other slots are not touched


@pytest.mark.parametrize("width,taps", [(64, 4), (36, 3), (8, 2)])
def test_canon_conv_of_a_long_step(width, taps):
    """Steps of more than a thousand rows (several rows a thread, a request's rows sliding through registers): three
    requests of unequal length side by side whose borders fall inside a thread's run of rows, then their next portions
    in a second such step; the state carries the rows between the two."""
    from hi_b200.kernels import ops

    lens = (1203, 7, 1001)
    hs = [rnd(n, width, seed=11 + i) for i, n in enumerate(lens)]
    ta, tb = rnd(width, taps, seed=3, scale=0.5), rnd(width, taps, seed=4, scale=0.5)
    state = torch.zeros((3, (taps - 1) * width), device=DEV)
    got_a, got_b = [[], [], []], [[], [], []]
    for ns, starts in (((601, 3, 499), (0, 0, 0)), ((602, 4, 502), (601, 3, 499))):
        h = torch.cat([hs[i][starts[i]: starts[i] + ns[i]] for i in range(3)]).to(DEV)
        cu = [0, ns[0], ns[0] + ns[1], sum(ns)]
        sot = [i for i in range(3) for _ in range(ns[i])]
        ya, yb = ops.canon_conv(h, ta.to(DEV), tb.to(DEV), state, i32(cu), i32(sot), i32([2, 0, 1]), torch.float32)
        for i in range(3):
            got_a[i].append(ya[cu[i]: cu[i + 1]])
            got_b[i].append(yb[cu[i]: cu[i + 1]])
    for i in range(3):
        for got, t in ((got_a, ta), (got_b, tb)):
            y = hs[i].double().clone()
            for j in range(taps):
                shift = taps - 1 - j
                y[shift:] += t[:, j].double() * hs[i][: lens[i] - shift].double()
            close(torch.cat(got[i]), y, 1e-6, f"request {i}")


def test_stream_add_and_normed_mean():
    from hi_b200.kernels import ops

    n, w = 19, 70
    x, d1, d2, e, v = rnd(n, w, seed=1), rnd(n, w, seed=2), rnd(n, w, seed=3), rnd(n, w, seed=4), rnd(w, seed=5)
    got = ops.stream_add(x.clone().to(DEV), d1.to(DEV).bfloat16(), d2.to(DEV), e.to(DEV), v.to(DEV))
    close(got, x.double() + d1.bfloat16().double() + d2.double() + e.double() + v.double(), 1e-6, "all terms")
    close(ops.stream_add(x.clone().to(DEV), vector=v.to(DEV)), x.double() + v.double(), 1e-6, "vector only")
    wa, wb = 1 + 0.3 * rnd(w, seed=6), 1 + 0.3 * rnd(w, seed=7)

    def norm(t, wt):
        t = t.double()
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-5) * wt.double()

    a, b = 3.0 * d1, 0.01 * d2
    close(ops.rmsnorm_mean2(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), 1e-5, torch.float32),
          0.5 * (norm(a, wa) + norm(b, wb)), 2e-6, "mean of two norms")
    # widths that the four-channels-a-thread kernel takes (two or four groups a thread) and one beyond it
    for w2 in (8, 72, 2048, 3000, 4100):
        a, b = 3.0 * rnd(5, w2, seed=w2), 0.01 * rnd(5, w2, seed=w2 + 1)
        wa2, wb2 = 1 + 0.3 * rnd(w2, seed=6), 1 + 0.3 * rnd(w2, seed=7)
        close(ops.rmsnorm_mean2(a.to(DEV), b.to(DEV), wa2.to(DEV), wb2.to(DEV), 1e-5, torch.float32),
              0.5 * (norm(a, wa2) + norm(b, wb2)), 2e-6, f"mean of two norms, width {w2}")
        ab, bb = a.bfloat16(), b.bfloat16()
        close(ops.rmsnorm_mean2(ab.to(DEV), bb.to(DEV), wa2.bfloat16().to(DEV), wb2.bfloat16().to(DEV), 1e-5, torch.bfloat16),
              0.5 * (norm(ab, wa2.bfloat16()) + norm(bb, wb2.bfloat16())), 8e-3, f"bfloat16, width {w2}")
    wide = rnd(n, 200, seed=8)
    close(ops.rmsnorm_rows(wide.to(DEV)[:, 30:100], wa.to(DEV), 1e-5), norm(wide[:, 30:100], wa), 2e-6, "rows of a slice")


# --------------------------------------------------------------------------- rotations
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_copy_and_latent_rows_with_a_rotated_key_part(interleaved):
    from hi_b200.kernels import ops

    n, heads, dim, rot, rank, page = 11, 3, 6, 10, 18, 4
    freqs = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)])
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 900, 901, 902])
    q = rnd(n, heads, dim + rot, seed=1)
    dst = torch.zeros(n, heads, 40, device=DEV)
    ops.rope_copy(q.to(DEV)[:, :, dim:], dst[:, :, rank: rank + rot], i32(pos.tolist()), freqs.to(DEV), interleaved)
    close(dst[:, :, rank: rank + rot], turn(q[:, :, dim:], pos, freqs, interleaved), 3e-6, "rotated copy")
    assert float(dst[:, :, :rank].abs().max()) == 0.0 and float(dst[:, :, rank + rot:].abs().max()) == 0.0
    # latent rows: [normed latent | rotated key part | zeros], at the token's place in its page
    x = rnd(n, 7 + rank + rot, seed=2)
    wgt = 1 + 0.3 * rnd(rank, seed=3)
    pages = torch.full((300, 1, page, 32), 5.0, device=DEV)
    table = torch.full((1, 230), -1, dtype=torch.int32)
    table[0, 0], table[0, 1], table[0, 225] = 9, 4, 17
    ops.latent_append(x.to(DEV)[:, 7:], wgt.to(DEV), 1e-5, i32(pos.tolist()), i32([0] * n), table.to(DEV), pages,
                      inv_freq=freqs.to(DEV), interleaved=interleaved)
    c = x[:, 7: 7 + rank].double()
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + 1e-5) * wgt.double()
    kr = turn(x[:, None, 7 + rank:], pos, freqs, interleaved)[:, 0]
    for t, p in enumerate(pos.tolist()):
        row = pages[int(table[0, p // page]), 0, p % page]
        close(row[:rank], c[t], 3e-6, f"latent of token {t}")
        close(row[rank: rank + rot], kr[t], 3e-6, f"key part of token {t}")
        assert float(row[rank + rot:].abs().max()) == 0.0


@pytest.mark.parametrize("hd,vdim,v_interleaved", [(16, 16, True), (32, 24, True), (16, 10, False)])
def test_values_are_cached_rotated(hd, vdim, v_interleaved):
    """qkv_post with a value rotation: every value row lands in its page turned by its own position over its first
    vdim dims; keys and queries are as without it."""
    from hi_b200.kernels import ops

    n, nh, nkv, page = 9, 2, 1, 4
    pos = [0, 1, 2, 3, 4, 5, 770, 771, 772]
    qkv = rnd(n, (nh + 2 * nkv) * hd, seed=4).to(DEV)
    vf = torch.tensor([50.0 ** (-2.0 * m / vdim) for m in range(vdim // 2)])
    table = torch.full((1, 200), -1, dtype=torch.int32)
    table[0, 0], table[0, 1], table[0, 192], table[0, 193] = 3, 0, 2, 1
    kp, vp = torch.zeros((4, nkv, page, hd), device=DEV), torch.zeros((4, nkv, page, hd), device=DEV)
    kp2, vp2 = torch.zeros_like(kp), torch.zeros_like(vp)
    args = (qkv, nh, nkv, hd, i32(pos), None, False, False, 1e-6, None, i32([0] * n), table.to(DEV))
    q1 = ops.qkv_post(*args, kp, vp, page, True, v_inv_freq=vf.to(DEV), v_interleaved=v_interleaved)
    q2 = ops.qkv_post(*args, kp2, vp2, page, True)
    assert torch.equal(q1, q2) and torch.equal(kp, kp2)
    v = qkv.view(n, nh + 2 * nkv, hd)[:, nh + nkv].cpu()
    want = turn(v[:, None], torch.tensor(pos), vf, v_interleaved)[:, 0]
    for t, p in enumerate(pos):
        close(vp[int(table[0, p // page]), 0, p % page], want[t], 3e-6, f"value of token {t}")


# --------------------------------------------------------------------------- sigmoid attention
def plain_sigmoid_attention(q, k, v, bias, scale, group, vf, v_interleaved, start):
    """q [n, nh, d] at positions start.., k / v [ctx, nkv, d] (values as cached: rotated already) -> [n, nh, d]."""
    n, nh, d = q.shape
    out = torch.zeros(n, nh, d, dtype=F64)
    for i in range(n):
        for a in range(nh):
            g = a // group
            s = (k[: start + i + 1, g].double() @ q[i, a].double()) * scale + float(bias[a])
            out[i, a] = torch.sigmoid(s) @ v[: start + i + 1, g].double()
    if vf is not None:
        out = turn(out, torch.arange(start, start + n), vf, v_interleaved, sign=-1.0)
    return out


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("nh,nkv,hd,vdim", [(4, 2, 16, 16), (3, 1, 24, 8), (2, 2, 64, 64), (8, 1, 96, 96), (2, 1, 264, 264)])
def test_sigmoid_attention_over_pages(dt, tol, nh, nkv, hd, vdim):
    """A portion and a single token far into a long context on scattered pages: one launch, and split over the keys."""
    from hi_b200.kernels import ops

    page, ctx_len = 16, 700
    g = torch.Generator().manual_seed(nh * hd)
    k = torch.randn(ctx_len, nkv, hd, generator=g).to(dt).float()
    v = torch.randn(ctx_len, nkv, hd, generator=g).to(dt).float()
    bias = torch.randn(nh, generator=g) - 3.0
    vf = torch.tensor([1000.0 ** (-2.0 * m / vdim) for m in range(vdim // 2)])
    n_pages = -(-ctx_len // page)
    perm = torch.randperm(n_pages + 5, generator=g)[:n_pages]
    kp = torch.zeros((n_pages + 5, nkv, page, hd), dtype=dt, device=DEV)
    vp = torch.zeros_like(kp)
    for p in range(ctx_len):
        kp[perm[p // page], :, p % page] = k[p].to(dt).to(DEV)
        vp[perm[p // page], :, p % page] = v[p].to(dt).to(DEV)
    table = perm.to(torch.int32).view(1, -1).to(DEV)
    for start, n in ((0, 40), (650, 50), (699, 1)):
        q = torch.randn(n, nh, hd, generator=g).to(dt).float()
        pos = i32(list(range(start, start + n)))
        want = plain_sigmoid_attention(q, k, v, bias, 0.2, nh // nkv, vf, True, start)
        for splits in (None, 64):
            got = ops.sigmoid_attention(q.to(dt).to(DEV), kp, vp, table, i32([0] * n), pos, 0, 0, 0.2, bias.to(DEV),
                                        start + n, v_inv_freq=vf.to(DEV), v_interleaved=True, split_size=splits)
            close(got, want, tol, f"start {start}, {n} tokens, split {splits}")


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 64), (8, 2, 128), (16, 1, 128), (6, 2, 192)])
def test_sigmoid_attention_on_the_tensor_cores(nh, nkv, hd, page):
    """bfloat16 heads of 64, 128 and 192: single tokens of three requests at different depths through the decode kernel
    (keys cut into splits), and portions of 130 to 300 new tokens at the start and far into a context through the
    tcgen05 kernel, one request bringing a single token beside them; all against the plain sum."""
    from hi_b200.kernels import ops

    dt, scale = torch.bfloat16, hd ** -0.5
    g = torch.Generator().manual_seed(nh + hd + page)
    lens = (900, 300, 65)
    per = -(-max(lens) // page)
    perm = torch.randperm(3 * per + 4, generator=g)[: 3 * per].view(3, per)
    kp = torch.zeros((3 * per + 4, nkv, page, hd), dtype=dt, device=DEV)
    vp = torch.zeros_like(kp)
    ks, vs = [], []
    for r, n in enumerate(lens):
        k, v = torch.randn(n, nkv, hd, generator=g).to(dt), torch.randn(n, nkv, hd, generator=g).to(dt)
        ks.append(k.float()); vs.append(v.float())
        for p in range(n):
            kp[perm[r, p // page], :, p % page] = k[p].to(DEV)
            vp[perm[r, p // page], :, p % page] = v[p].to(DEV)
    table = perm.to(torch.int32).to(DEV)
    bias = (torch.randn(nh, generator=g) - 4.0)
    vf = torch.tensor([1000.0 ** (-2.0 * m / hd) for m in range(hd // 2)])
    # single tokens: the last position of every request
    q = torch.randn(3, nh, hd, generator=g).to(dt)
    got = ops.sigmoid_decode_attention(q.to(DEV), kp, vp, table, i32([0, 1, 2]), i32([n - 1 for n in lens]), 0, 0, scale,
                                       bias.to(DEV), max(lens), vf.to(DEV), True)
    for r, n in enumerate(lens):
        want = plain_sigmoid_attention(q[r: r + 1].float(), ks[r], vs[r], bias, scale, nh // nkv, vf, True, n - 1)
        close(got[r: r + 1], want, 2e-2, f"single token of request {r}")
    # portions: request 0 brings positions 600..899, request 1 its first 130, request 2 one token
    news = ((600, 300), (0, 130), (64, 1))
    qs = [torch.randn(n, nh, hd, generator=g).to(dt) for _s, n in news]
    cu = [0, 300, 430, 431]
    pos = [p for s0, n in news for p in range(s0, s0 + n)]
    for skip in (False, True):
        got = ops.sigmoid_prefill_attention_tc(torch.cat(qs).to(DEV), kp, vp, table, i32(cu), i32(pos), 3, 300, 0, 0, scale,
                                               bias.to(DEV), skip_single=skip, v_inv_freq=vf.to(DEV), v_interleaved=True)
        for r, (s0, n) in enumerate(news):
            want = plain_sigmoid_attention(qs[r].float(), ks[r], vs[r], bias, scale, nh // nkv, vf, True, s0)
            if skip and n == 1:
                assert float(got[cu[r]: cu[r + 1]].abs().max()) == 0.0
            else:
                close(got[cu[r]: cu[r + 1]], want, 2e-2, f"portion of request {r}, skip {skip}")
    ops.check_tc_status()


# --------------------------------------------------------------------------- recurrences
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("nh,sliding", [(5, 0), (20, 0), (16, 150)])
def test_softmax_over_shared_rows_of_192(nh, sliding, page):
    """What latent attention with a rotated key part asks of the paged kernels in bfloat16: rows of 192 that are keys
    and values at once, one kv head under many query heads. Single tokens (the decode kernel, sixteen heads a call),
    portions of 2 to 70 tokens (mma.sync) and of 130 to 280 (tcgen05, with and without key splits), whole and far
    into a context, with a sliding window too; one row's first 8 numbers are made large so that the query that
    matches it puts nearly all its weight there (a row lost or shifted by one then shows)."""
    from hi_b200.kernels import ops

    hd, dt, scale = 192, torch.bfloat16, 0.09
    g = torch.Generator().manual_seed(nh + page + sliding)
    lens = (700, 281, 66)
    per = -(-max(lens) // page)
    perm = torch.randperm(3 * per + 3, generator=g)[: 3 * per].view(3, per)
    pool = torch.zeros((3 * per + 3, 1, page, hd), dtype=dt, device=DEV)
    rows = []
    for r, n in enumerate(lens):
        c = torch.randn(n, hd, generator=g).to(dt)
        c[n // 3, :8] = 6.0
        rows.append(c.float())
        for p in range(n):
            pool[perm[r, p // page], 0, p % page] = c[p].to(DEV)
    table = perm.to(torch.int32).to(DEV)

    def plain(q, c, start):
        out = torch.zeros(q.shape[0], nh, hd, dtype=torch.float64)
        for i in range(q.shape[0]):
            p = start + i
            lo = max(0, p - sliding + 1) if sliding else 0
            keys = c[lo: p + 1].double()
            w = torch.softmax(q[i].double() @ keys.T * scale, dim=-1)
            out[i] = w @ keys
        return out

    def queries(n):
        q = torch.randn(n, nh, hd, generator=g).to(dt)
        q[:, 0, :8] = 4.0                                    # head 0 asks for the planted row
        return q

    # single tokens: the last position of every request
    q = queries(3)
    got = torch.empty_like(q, device=DEV)
    for first in range(0, nh, 16):
        part = q[:, first: first + 16].contiguous().to(DEV)
        got[:, first: first + 16] = ops.decode_attention(part, pool, pool, table, i32([0, 1, 2]), i32([n - 1 for n in lens]),
                                                         0, sliding, scale, max(lens))
    for r, n in enumerate(lens):
        close(got[r: r + 1], plain(q[r: r + 1].float(), rows[r], n - 1), 2e-2, f"single token of request {r}")
    # portions
    for news in (((420, 280), (0, 130), (64, 2)), ((630, 70), (279, 2), (0, 66))):
        qs = [queries(n) for _s, n in news]
        cu = [0]
        for _s, n in news:
            cu.append(cu[-1] + n)
        pos = [p for s0, n in news for p in range(s0, s0 + n)]
        longest = max(n for _s, n in news)
        args = (torch.cat(qs).to(DEV), pool, pool, table, i32(cu), i32(pos), 3, longest, 0, sliding, scale)
        runs = [("mma.sync", ops.prefill_attention(*args))]
        if longest >= ops.PREFILL_TC_MIN_TOKENS:
            runs += [(f"tcgen05, {k} splits", ops.prefill_attention_tc(*args, key_splits=k)) for k in (1, 3)]
        for what, got in runs:
            for r, (s0, n) in enumerate(news):
                close(got[cu[r]: cu[r + 1]], plain(qs[r].float(), rows[r], s0), 2e-2, f"{what}: portion of request {r}")
    torch.cuda.synchronize()
    ops.check_tc_status()


@pytest.mark.parametrize("heads,dim,vdim,general", [(2, 16, 24, False), (3, 5, 7, False), (1, 136, 20, False), (2, 48, 32, True)])
def test_gated_linear_attention_inputs_and_recurrence(heads, dim, vdim, general):
    """gla_prep (scaled q, decay = sigmoid(z + b)^(1/tau)) and the recurrence without the delta rule's correction, two
    requests in portions on slots 2 and 0, against S <- diag(alpha) S + k v^T, o = S^T q."""
    from hi_b200.kernels import ops

    tau, lens = 4.0, (21, 9)
    hd, hv = heads * dim, heads * vdim
    projs = [rnd(n, 3 + 2 * hd + hv, seed=7 + i) for i, n in enumerate(lens)]
    zs = [rnd(n, hd, seed=9 + i, scale=2.0) for i, n in enumerate(lens)]
    bias = rnd(hd, seed=11)
    state = torch.zeros((3, heads * dim * vdim), device=DEV)
    cuts = [((6, 3), (0, 0)), ((1, 1), (6, 3)), ((14, 5), (7, 4))]
    got = [[], []]
    for ns, starts in cuts:
        proj = torch.cat([projs[i][s: s + n] for i, (n, s) in enumerate(zip(ns, starts))]).to(DEV)
        z = torch.cat([zs[i][s: s + n] for i, (n, s) in enumerate(zip(ns, starts))]).to(DEV)
        q, k, v, decay = ops.gla_prep(proj, 3, 3 + hd, 3 + 2 * hd, z, bias.to(DEV), tau, dim ** -0.5, hd, hv)
        o = ops.delta_recurrence(q, k, v, None, decay, state, i32([0, ns[0], ns[0] + ns[1]]), i32([2, 0]), heads, heads, dim,
                                 vdim, general=general, single_tokens=max(ns) == 1, plain=True)
        got[0].append(o[: ns[0]]); got[1].append(o[ns[0]:])
    for i, n in enumerate(lens):
        p = projs[i].double()
        q = p[:, 3: 3 + hd].view(n, heads, dim) * dim ** -0.5
        k, v = p[:, 3 + hd: 3 + 2 * hd].view(n, heads, dim), p[:, 3 + 2 * hd:].view(n, heads, vdim)
        alpha = (torch.sigmoid(zs[i].double() + bias.double()) ** (1.0 / tau)).view(n, heads, dim)
        want = torch.zeros(n, heads, vdim, dtype=F64)
        s = torch.zeros(heads, dim, vdim, dtype=F64)
        for t in range(n):
            s = alpha[t][:, :, None] * s + k[t][:, :, None] * v[t][:, None, :]
            want[t] = (s * q[t][:, :, None]).sum(1)
        close(torch.cat(got[i]).view(n, heads, vdim), want, 2e-5, f"request {i}")
        close(state[(2, 0)[i]].view(heads, dim, vdim), s, 2e-5, f"state of request {i}")


def test_delta_rule_with_one_decay_per_head_and_a_silu_gate():
    from hi_b200.kernels import ops

    heads, kvh, dim, vdim, taps, n = 4, 2, 8, 6, 3, 13
    chan = 2 * kvh * dim + heads * vdim
    proj = rnd(n, chan + heads, seed=1)
    conv = rnd(chan, taps, seed=2, scale=0.5)
    a_pre, dt_bias, a_log = rnd(n, heads, seed=3), rnd(heads, seed=4), rnd(heads, seed=5, scale=0.5)
    s_len = heads * dim * vdim
    state = torch.zeros((2, s_len + (taps - 1) * chan), device=DEV)
    outs = []
    for a, b in ((0, 5), (5, 6), (6, 13)):
        m = b - a
        q, k, v, beta, decay = ops.delta_prep(proj[a:b].to(DEV), 0, chan, conv.to(DEV), state, s_len, a_pre[a:b].contiguous().to(DEV),
                                              dt_bias.to(DEV), a_log.to(DEV), i32([0, m]), i32([0] * m), i32([1]), heads, kvh,
                                              dim, vdim, head_decay=True)
        ops.delta_conv_update(proj[a:b].to(DEV), 0, chan, taps, state, s_len, i32([0, m]), i32([1]))
        outs.append((q, k, v, beta, decay))
    q, k, v, beta, decay = (torch.cat([o[j] for o in outs]).cpu().double() for j in range(5))
    x = proj[:, :chan].double()
    y = torch.zeros_like(x)
    for t in range(n):
        for j in range(taps):
            if t - (taps - 1) + j >= 0:
                y[t] += conv[:, j].double() * x[t - (taps - 1) + j]
    y = y * torch.sigmoid(y)
    wq, wk = y[:, : kvh * dim].view(n, kvh, dim), y[:, kvh * dim: 2 * kvh * dim].view(n, kvh, dim)
    wq = wq / torch.sqrt((wq * wq).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    wk = wk / torch.sqrt((wk * wk).sum(-1, keepdim=True) + 1e-6)
    close(q.view(n, kvh, dim), wq, 1e-5, "q"); close(k.view(n, kvh, dim), wk, 1e-5, "k")
    close(v, y[:, 2 * kvh * dim:], 1e-5, "v")
    close(beta, torch.sigmoid(proj[:, chan:].double()), 1e-5, "beta")
    g = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(a_pre.double() + dt_bias.double()))
    close(decay.view(n, heads, dim), g[:, :, None].expand(n, heads, dim), 1e-5, "one decay for all channels of a head")
    o = rnd(n, heads * vdim, seed=6)
    gate = rnd(n, 5 + heads * vdim, seed=7)
    wn = 1 + 0.3 * rnd(vdim, seed=8)
    got = ops.delta_out_norm(o.to(DEV), gate.to(DEV)[:, 5:], wn.to(DEV), 1e-5, vdim, torch.float32, gate_silu=True)
    od = o.double().view(n, heads, vdim)
    gd = gate[:, 5:].double().view(n, heads, vdim)
    want = od / torch.sqrt((od * od).mean(-1, keepdim=True) + 1e-5) * wn.double() * gd * torch.sigmoid(gd)
    close(got.view(n, heads, vdim), want, 1e-5, "normed, gated read-out")
