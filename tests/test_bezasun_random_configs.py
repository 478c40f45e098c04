"""Bezasun configurations drawn at random (seeded): every size, constant, the order of layers, the number of copies of
the stream and what a configuration may leave out move at once, small odd sizes as well as sizes at which the
tensor-core kernels take over, and each draw goes through the four ways of cutting against the plain model, in 32-bit
and in bfloat16."""
import random

import pytest

import harness as h
from bezasun_configs import attention, config, latent, mamba, moe, write_model
from test_bezasun_engine import TOL, compare, replay, tokens

pytestmark = pytest.mark.gpu


def draw(rng: random.Random, large: bool) -> dict:
    layers = []
    for _ in range(rng.randrange(1, 6)):
        mlp = None
        if rng.random() < 0.8:
            experts = rng.choice([1, 2, 3, 4, 8, 16, 32]) if large else rng.choice([1, 2, 3, 5, 8, 12, 16, 33])
            top = rng.choice([t for t in (1, 2, 3, 4, 6, 8, 10) if t <= experts])
            ff = rng.choice([64, 96, 128]) if large else rng.choice([2, 8, 16]) * rng.randrange(1, 9)
            shared = rng.choice([None, ff, 2 * ff, 24])
            mlp = moe(experts, top, ff, shared=shared)
        kind = rng.choice(["latent", "mamba", "attention"])
        if kind == "latent":
            heads = rng.choice([1, 2, 3, 4, 8, 17])
            dim = rng.choice([8, 16, 32, 64]) if large else rng.choice([2, 6, 8, 16, 24, 40])
            rot_dim = rng.choice([16, 32, 64]) if large else rng.choice([2, 4, 6, 8, 16, 20])
            vdim = rng.choice([16, 32, 64]) if large else rng.choice([2, 4, 8, 12, 24, 36])
            kv_rank = rng.choice([32, 64, 96, 128, 160]) if large else rng.choice([3, 8, 16, 24, 50, 72, 130, 200])
            q_rank = rng.choice([4, 8, 24, 48, 96])
            scaling = rng.choice([None, (rng.choice([2.0, 4.0, 8.0, 40.0]), rng.choice([16, 64, 512, 4096]),
                                         rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0, 2.0]))])
            window = rng.choice([None, 1, 2, 7, 16, 33, 64, 96, 150, 1000])
            layers.append(latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, rng.choice([0.5, 1.0, 2.0]) * (dim + rot_dim) ** -0.5,
                                 rng.choice([100.0, 10000.0, 250000.0]), window=window, scaling=scaling, mlp=mlp))
        elif kind == "mamba":
            groups = rng.choice([1, 2, 3])
            heads = groups * rng.choice([1, 2, 4])
            vdim = rng.choice([32, 64]) if large else rng.choice([2, 4, 8, 16, 24, 48, 90])
            state = rng.choice([16, 64, 128]) if large else rng.choice([1, 3, 8, 16, 20, 32, 64, 130])
            parts = rng.choice([p for p in (1, 2, 3, 4, heads) if (heads * vdim) % p == 0])
            layers.append(mamba(heads, vdim, state, groups, rng.choice([1, 2, 3, 4, 5]), parts, mlp=mlp))
        else:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4, 6, 8])
            dim = rng.choice([64, 128]) if large else rng.choice([2, 8, 12, 16, 24, 40, 48, 64, 80, 96])
            vdim = dim if (large or rng.random() < 0.5) else rng.choice([4, 8, 20, 32, 48, 72])
            layers.append(attention(heads, kv, dim, vdim, rng.choice([0.5, 1.0, 2.0]) * dim ** -0.5,
                                    softcap=rng.choice([None, 2.0, 10.0, 30.0, 50.0]),
                                    q_temp=rng.choice([None, (rng.choice([0.1, 0.5, 1.0]), rng.choice([1, 5, 16, 100, 256]))]), mlp=mlp))
    width = rng.choice([256, 320, 384]) if large else rng.choice([2, 4, 8, 16]) * rng.randrange(3, 20)
    return config(rng.randrange(60, 900), width, rng.choice([1e-5, 1e-6, 3e-4]), layers,
                  streams=rng.choice([None, 1, 2, 3, 4, 4, 6, 8]), mult=rng.choice([None, 0.4, 0.7, 1.0, 1.5]),
                  embed_scale=rng.choice([None, 0.5, 2.0]), logit_scale=rng.choice([None, 0.5, 2.0]))


@pytest.mark.parametrize("seed,large", [(1, False), (2, False), (3, False), (4, False), (5, False), (6, False), (7, False), (8, False),
                                        (9, False), (10, False), (11, False), (12, False), (101, True), (102, True), (103, True),
                                        (104, True)])
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
            got, forced = replay(eng, steps, dtype)
            compare(cfg, weights, reqs, got, TOL[dtype], f"seed {seed} {cfg} page {page}: {dtype} {regime}", forced)
            assert not eng.manager.requests
            for p in eng.manager.pools:
                assert p.free == p.total, "pages were lost"
