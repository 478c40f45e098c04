"""Bezasun in the engine against the plain implementation: every mixer alone, whole prompts, decoding through the
cache and the states, portions down to two tokens, mixed batches with pages and slots used again, planted keys far
away, at page borders and on both sides of a window's edge, a peaked softmax, a sink that matters, the first tokens,
long decoding through captured steps, configurations of other sizes, generation through the entry point, the trace
replay and the command line."""
import numpy as np
import pytest
import torch

import harness as h
import plain_bezasun as plain
from bezasun_configs import CONFIGS, attention, config, latent, make_weights, moe, peaked, plain_logits, write_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# A position's error is the largest difference of its logits over the largest logit. The float32 runs are the sharp
# ones: rounding gives a few 1e-6 there, while a lost, doubled or shifted key, a lost state or convolution input, a
# copy of the stream mixed the wrong way round or a sink left out moves the logits by a thousand times that. In
# bfloat16 these small models magnify rounding, so there the MEDIAN error of a comparison's positions is held to the
# tolerance and no position may be wildly off.
TOL = {"float32": 5e-5, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("bezasun")
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(base / name)
        out[name] = (cfg, d, write_model(d, cfg, seed=40 + ord(name)))
    return out


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def engine(mdir, dtype, **kw):
    from hi_b200.engine.core import Engine

    kw.setdefault("kv_page_size", 16)
    kw.setdefault("kv_cache_tokens", 2048)
    kw.setdefault("max_active_requests", 4)
    return Engine.from_dir(mdir, dtype=dtype, **kw)


def compare(cfg, weights, requests, got, tol, what, forced=None):
    """Every wanted row against the plain model; names the first wrong token. ``forced``: the engine's own expert
    choices in a bfloat16 run (reduced precision may pick the other of two nearly equal scores; the logits are then
    compared given that choice)."""
    errs, over = [], []
    sharp = tol < 1e-3
    for rid, toks in requests.items():
        ref = plain_logits(cfg, weights, toks, forced=(forced or {}).get(rid))
        scale = float(ref.abs().max())
        rows = got.get(rid, {})
        assert rows, f"{what}: no logits came back for request {rid!r}"
        for p in sorted(rows):
            err = float(np.abs(rows[p].astype(np.float64) - ref[p].numpy()).max()) / scale
            assert np.isfinite(err), f"{what}: request {rid!r}, position {p}: not finite"
            assert err <= 8 * tol, f"{what}: request {rid!r} first differs at position {p} of {len(toks)}: rel err {err:.3e}"
            errs.append(err)
            if err > tol:
                over.append((rid, p, err))
    if sharp:
        # a norm over a handful of numbers that nearly cancel magnifies 32-bit rounding at single positions
        assert len(over) <= max(1, 0.02 * len(errs)), f"{what}: {len(over)} of {len(errs)} positions over {tol:.1e}; the first: {over[:3]}"
    else:
        assert float(np.median(errs)) <= tol, f"{what}: median error {float(np.median(errs)):.3e} of {len(errs)} positions"


def replay(eng, steps, dtype):
    got, forced = h.replay_in_process(eng, steps, record_routing=(dtype == "bfloat16"))
    return got, ({r: {k: v.long() for k, v in layers.items()} for r, layers in forced.items()} if dtype == "bfloat16" else None)


# --------------------------------------------------------------------------- every mixer alone
def _mixer_cases():
    cases = []
    for name, cfg in CONFIGS.items():
        for i, layer in enumerate(cfg["layers"]):
            cases.append(pytest.param(cfg, i, id=f"{name}{i}-{layer['type']}"))
    return cases


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("cfg,index", _mixer_cases())
def test_mixer_alone(dt, tol, cfg, index):
    """Two requests in four steps (a portion each, a portion beside a single token, single tokens, a single token
    beside a portion) on scattered pages and state slots 2 and 0, against the plain mixer on the whole inputs."""
    from hi_b200.config.bezasun import BezasunConfig
    from hi_b200.parts.bezasun import build_bezasun_spec
    from hi_b200.parts.context import CacheView
    from hi_b200.parts.registry import build
    from test_vinurax_engine import _ctx, _env

    width, page, eps = cfg["width"], 8, cfg["norm"]["eps"]
    layer = cfg["layers"][index]
    w = make_weights(cfg, 5 + index)
    spec = build_bezasun_spec(BezasunConfig.from_json(cfg)).layers[index].mixer
    part = build("mixer", spec, _env(dt, width), f"l{index}.mix")
    part.load(lambda name: w[name].to(DEV).to(dt) if name in w else None)
    cs = part.cache_spec()
    view = CacheView(group=0, writes=True)
    if cs.paged:
        view.k_pages = torch.zeros((12, cs.kv_heads, page, cs.head_dim), dtype=dt, device=DEV)
        view.v_pages = torch.zeros_like(view.k_pages) if cs.values else None
    if cs.state_shape:
        view.state = torch.zeros((3, *cs.state_shape), dtype=torch.float32, device=DEV)
    table = torch.tensor([[7, 2, 9, 4, 6], [1, 11, 0, 5, 3]], dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(n, width, generator=g).to(dt).float() for n in (33, 29)]
    cuts = [([13, 17], [0, 0]), ([18, 1], [13, 17]), ([1, 1], [31, 18]), ([1, 10], [32, 19])]
    got = [[], []]
    for lens, starts in cuts:
        x = torch.cat([xs[i][s: s + n] for i, (n, s) in enumerate(zip(lens, starts))])
        out = part.forward(x.to(DEV).to(dt), _ctx(lens, starts, page, table, [2, 0]), view)
        a = 0
        for i, n in enumerate(lens):
            got[i].append(out[a: a + n].float().cpu())
            a += n
    wd = {k: v.double() for k, v in w.items()}
    for i in range(2):
        want = plain.MIXERS[layer["type"]](xs[i].double(), layer["mixer"], wd, f"l{index}.mix", eps)
        have = torch.cat(got[i]).double()
        assert have.shape == want.shape
        errs = (have - want).abs().amax(dim=1) / want.abs().max()
        if dt == torch.float32:
            assert float(errs.max()) <= tol, f"request {i}: token {int(errs.argmax())}: rel err {float(errs.max()):.3e}"
        else:
            assert float(errs.median()) <= tol and float((errs > 8 * tol).float().mean()) <= 0.1, \
                f"request {i}: median rel err {float(errs.median()):.3e}, worst {float(errs.max()):.3e}"


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("name,index", [("A", 0), ("B", 1), ("C", 0), ("D", 0), ("D", 2), ("E", 0)])
def test_experts_alone(dt, tol, name, index):
    """The routed feed-forward with the engine's own choice of experts handed to the plain mixture: 3 and 150 tokens
    (the few-rows and the many-rows kernels)."""
    from hi_b200.config.bezasun import BezasunConfig
    from hi_b200.parts.bezasun import build_bezasun_spec
    from hi_b200.parts.context import Pending
    from hi_b200.parts.registry import build
    from test_vinurax_engine import _ctx, _env

    cfg = CONFIGS[name]
    width, mlp = cfg["width"], cfg["layers"][index]["mlp"]
    w = make_weights(cfg, 11)
    spec = build_bezasun_spec(BezasunConfig.from_json(cfg)).layers[index].feed_forward
    part = build("feed_forward", spec, _env(dt, width), f"l{index}.mlp")
    part.load(lambda n: w[n].to(DEV).to(dt) if n in w else None)
    wd = {k: v.double() for k, v in w.items()}
    for n in (3, 150):
        x = torch.randn(n, width, generator=torch.Generator().manual_seed(n)).to(dt).float()
        taps = {}
        ctx = _ctx([n], [0], 8, torch.zeros((1, 32), dtype=torch.int32), [0])
        ctx.tap = lambda k, t: taps.__setitem__(k, t.clone())
        out = part.forward(x.to(DEV).to(dt), ctx, normed_f32=x.to(DEV))
        assert isinstance(out, Pending)
        have = out.materialize(n).double().cpu()
        ids = taps[f"l{index}.mlp.router_ids"].long().cpu()
        own, _scores = plain.router_choice(x.double(), mlp, wd, f"l{index}.mlp")
        if dt == torch.float32:
            assert (own.sort(-1).values == ids.sort(-1).values).all()
        want = plain.mixture(x.double(), mlp, wd, f"l{index}.mlp", forced_ids=ids)
        err = float((have - want).abs().max() / want.abs().max())
        assert err <= tol, f"{n} tokens: rel err {err:.3e}"


# --------------------------------------------------------------------------- the model in the engine
@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_ways_of_cutting(name, dtype, models):
    cfg, mdir, weights = models[name]
    requests = {"p": tokens(cfg, 150, 1), "q": tokens(cfg, 37, 2), "r": tokens(cfg, 1, 3), "s": tokens(cfg, 2, 4),
                "t": tokens(cfg, 64, 5), "u": tokens(cfg, 97, 6)}
    eng = engine(mdir, dtype, kv_cache_tokens=352, debug_poison=True)
    prompt = {r: min(len(t), max(2, len(t) - 24)) for r, t in requests.items()}      # the rest is decoded token by token
    for what, steps in (("whole", h.trace_whole(requests)), ("decode", h.trace_tail_decode(requests, tail=20)),
                        ("portions", h.trace_portions(requests)),
                        ("mixed", h.trace_mixed(requests, max_tokens=352, page=16, seed=7, max_live=4, prefill_len=prompt))):
        got, forced = replay(eng, steps, dtype)
        compare(cfg, weights, requests, got, TOL[dtype], f"{name} {dtype} {what}", forced)
    assert len(eng.manager.requests) == 0


@pytest.mark.parametrize("name", ["A", "D"])
def test_mixed_batches_use_pages_and_slots_again(name, models):
    """More requests than slots and than the pool holds at once, in two orders: every request's logits equal the
    plain model's whatever ran beside it and whichever pages and slot it got. A slot that is handed out again
    starts from zero: the matrix memory and the convolution's inputs."""
    cfg, mdir, weights = models[name]
    requests = {i: tokens(cfg, n, 30 + i) for i, n in enumerate((70, 33, 48, 5, 90, 17, 64, 31, 2, 55))}
    for seed, live in ((1, 4), (2, 2)):
        eng = engine(mdir, "float32", kv_cache_tokens=272, max_active_requests=live, debug_poison=True)
        steps = h.trace_mixed(requests, max_tokens=272, page=16, seed=seed, max_live=live)
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, TOL["float32"], f"{name} mixed seed {seed}")
        assert eng.manager.snapshot()["groups"][0]["allocations"] > 272 // 16      # pages were handed out again


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_far_keys_and_window_edges_under_a_peaked_softmax(name, models, tmp_path):
    """Softmax scales times 8: nearly all weight on one key, so a key that is lost, doubled or shifted shows (the
    oldest key of a window, the one just outside it, a key hundreds of tokens back). A prompt over many pages whole,
    in portions whose edges fall inside pages and windows, and decoded at the end. The peaked scores magnify
    float32 rounding too (two cuttings of the same prompt differ by up to 1e-4 between themselves), so the bound is
    1e-3; a wrong key moves these logits by tenths."""
    cfg = peaked(CONFIGS[name], 8.0)
    mdir = str(tmp_path / "peaked")
    weights = write_model(mdir, cfg, seed=77)
    requests = {"long": tokens(cfg, 300, 8), "short": tokens(cfg, 90, 9)}
    eng = engine(mdir, "float32", kv_cache_tokens=1024)
    for what, steps in (("whole", h.trace_whole(requests)), ("decode", h.trace_tail_decode(requests, tail=60)),
                        ("portions", h.trace_portions(requests, sizes=(100, 3, 61, 2, 29, 17, 2, 50, 5))),
                        ("mixed", h.trace_mixed(requests, max_tokens=1024, page=16, seed=3, max_live=2))):
        got, _ = h.replay_in_process(eng, steps)
        compare(cfg, weights, requests, got, 9.9e-4, f"{name} peaked {what}")


def _planted_attention():
    """One attention layer made so that the last token's query matches exactly one earlier token's key: queries and
    keys read the token's identity through single dims, every other token's query and key are exactly zero, and only
    the answering token carries a value. The distance bias and the sink stay on."""
    cfg = config(16, 32, 1e-6, [attention(1, 1, 16, 16, 1.5, softcap=40.0, q_temp=(0.25, 64))], streams=2, mult=1.0)
    w = make_weights(cfg, 9)
    emb = torch.zeros(16, 32)
    emb[:, 8:] = 0.05 * torch.randn(16, 24, generator=torch.Generator().manual_seed(1))
    emb[1, 0], emb[2, 1], emb[2, 2] = 4.0, 4.0, 4.0
    w["embed"] = emb
    w["l0.norm1"] = torch.zeros(32)
    for nme in ("q", "k", "v"):
        w[f"l0.mix.{nme}"] = torch.zeros(16, 32)
    w["l0.mix.q"][12, 0] = 1.0           # token 1 asks ...
    w["l0.mix.k"][12, 1] = 1.0           # ... token 2 answers
    w["l0.mix.v"][:, 2] = torch.linspace(-1, 1, 16)  # and only token 2 carries a value worth reading
    w["l0.mix.q.norm"] = torch.ones(16)
    w["l0.mix.k.norm"] = torch.ones(16)
    w["l0.mix.sink"] = torch.tensor([2.0])
    return cfg, {k: v.to(torch.bfloat16).float() for k, v in w.items()}


@pytest.mark.parametrize("where", [0, 1, 15, 16, 17, 255, 256, 300])
def test_a_planted_key_far_away_and_at_page_borders(where, tmp_path):
    """The answering token at the sequence's first places, on both sides of a page's border and hundreds of tokens
    back: the engine agrees with the plain model whole, in portions and when the asking token is decoded alone, and
    the plain model's logits follow the planted value (they differ from a run without the answering token)."""
    cfg, w = _planted_attention()
    n = 400
    toks = [3 + (i % 11) for i in range(n)]
    toks[where], toks[-1] = 2, 1
    without = list(toks)
    without[where] = 3
    ref, ref_without = plain_logits(cfg, w, toks)[-1], plain_logits(cfg, w, without)[-1]
    assert float((ref - ref_without).abs().max()) > 0.05 * float(ref.abs().max())
    mdir = str(tmp_path / "planted")
    write_model(mdir, cfg, 0, weights=w)
    for what, steps in (("whole", h.trace_whole({"a": toks})), ("decode", h.trace_tail_decode({"a": toks}, tail=3)),
                        ("portions", h.trace_portions({"a": toks}, sizes=(15, 2, 1, 7, 230, 2, 44, 90, 9)))):
        got, _ = h.replay_in_process(engine(mdir, "float32", kv_cache_tokens=512), steps)
        compare(cfg, w, {"a": toks}, got, 5e-5, f"planted key at {where} {what}")


def test_the_sink_takes_its_share(tmp_path):
    """The planted model again with the sink's score raised until it outweighs the planted key: the read-out shrinks
    in the plain model, and the engine follows it."""
    cfg, w = _planted_attention()
    toks = [3 + (i % 11) for i in range(60)]
    toks[20], toks[-1] = 2, 1
    small = plain_logits(cfg, w, toks)[-1]
    w["l0.mix.sink"] = torch.tensor([30.0])
    large = plain_logits(cfg, w, toks)[-1]
    assert float((small - large).abs().max()) > 0.05 * float(small.abs().max())
    mdir = str(tmp_path / "sink")
    write_model(mdir, cfg, 0, weights=w)
    for steps in (h.trace_whole({"a": toks}), h.trace_tail_decode({"a": toks}, tail=3)):
        got, _ = h.replay_in_process(engine(mdir, "float32", kv_cache_tokens=128), steps)
        compare(cfg, w, {"a": toks}, got, 5e-5, "a sink that outweighs the keys")


WINDOW = 48


def _planted_latent():
    """One latent-attention layer with a window, made as :func:`_planted_attention`: the asking token's query and the
    answering token's latent have one entry each, every other token's are exactly zero (their norms leave zero as it
    is), and the value is read off the answering token's latent."""
    cfg = config(16, 32, 1e-6, [latent(1, 8, 4, 8, 8, 8, 2.0, 100.0, window=WINDOW, scaling=(2.0, 16, 4.0, 1.0))])
    w = make_weights(cfg, 9)
    emb = torch.zeros(16, 32)
    emb[:, 8:] = 0.05 * torch.randn(16, 24, generator=torch.Generator().manual_seed(1))
    emb[1, 0], emb[2, 1] = 4.0, 4.0
    w["embed"] = emb
    w["l0.norm1"] = torch.zeros(32)
    for nme in ("dq", "uq", "dkv", "uk"):
        w[f"l0.mix.{nme}"] = torch.zeros_like(w[f"l0.mix.{nme}"])
    w["l0.mix.dq"][0, 0] = 1.0           # token 1 asks ...
    w["l0.mix.uq"][0, 0] = 1.0
    w["l0.mix.dkv"][0, 1] = 1.0          # ... token 2 answers
    w["l0.mix.uk"][0, 0] = 1.0
    w["l0.mix.dq.norm"] = torch.ones(8)
    w["l0.mix.dkv.norm"] = torch.ones(8)
    return cfg, {k: v.to(torch.bfloat16).float() for k, v in w.items()}


@pytest.mark.parametrize("back", [0, 1, WINDOW - 2, WINDOW - 1, WINDOW, WINDOW + 1, 3 * WINDOW])
def test_a_planted_key_on_both_sides_of_the_window_edge(back, tmp_path):
    """The answering token ``back`` places before the asking one: read while back < window, and not at all from
    there on (the plain model's logits then equal those without it). The engine agrees whole, in portions that cut
    the window, and when the asking token is decoded alone (after other decoded tokens have moved the window)."""
    cfg, w = _planted_latent()
    n = 200
    toks = [3 + (i % 11) for i in range(n)]
    toks[-1] = 1
    without = list(toks)
    if back:
        toks[n - 1 - back] = 2
    else:
        without[-1] = 3
    ref, ref_without = plain_logits(cfg, w, toks)[-1], plain_logits(cfg, w, without)[-1]
    moved = float((ref - ref_without).abs().max()) / float(ref.abs().max())
    if 0 < back < WINDOW:
        assert moved > 0.05
    elif back:
        assert moved < 1e-12
    mdir = str(tmp_path / "planted")
    write_model(mdir, cfg, 0, weights=w)
    for what, steps in (("whole", h.trace_whole({"a": toks})), ("decode", h.trace_tail_decode({"a": toks}, tail=60)),
                        ("portions", h.trace_portions({"a": toks}, sizes=(15, 2, 1, 7, 100, 2, 44, 20, 9)))):
        got, _ = h.replay_in_process(engine(mdir, "float32", kv_cache_tokens=256), steps)
        compare(cfg, w, {"a": toks}, got, 5e-5, f"planted key {back} back {what}")


def test_long_decoding_and_first_tokens(models):
    """300 tokens decoded one by one after a two-token prompt (captured steps), beside a request that starts
    later; positions 0 and 1 are compared too."""
    cfg, mdir, weights = models["A"]
    requests = {"a": tokens(cfg, 300, 11), "b": tokens(cfg, 120, 12)}
    for dtype in ("float32", "bfloat16"):
        eng = engine(mdir, dtype)
        steps = [([("a", requests["a"][:2], [0, 1])], [])]
        for i in range(2, 300):
            entries = [("a", [requests["a"][i]], [0])]
            j = i - 100
            if 0 <= j < 120:
                entries.append(("b", [requests["b"][j]], [0]))
            steps.append((entries, [r for r, n in (("a", 299), ("b", 219)) if i == n]))
        got, forced = replay(eng, steps, dtype)
        compare(cfg, weights, requests, got, TOL[dtype], f"long decoding {dtype}", forced)
        assert len(eng._graphs) >= 1 and any(g.captured for g in eng._graphs.values())


def test_other_page_sizes_and_kernel_choices(models):
    """Page sizes 8 and 64; in bfloat16 a latent row (padded to 64, 128 or 192) goes through the tensor-core
    attention kernels with pages of 64 (single tokens, short portions, portions of 128 tokens and more)."""
    from hi_b200.kernels import ops

    for name in ("A", "B", "E"):
        cfg, mdir, weights = models[name]
        requests = {"x": tokens(cfg, 333, 14), "y": tokens(cfg, 40, 15)}
        for page in (8, 64):
            before = dict(ops.CALLS)
            eng = engine(mdir, "bfloat16", kv_page_size=page, kv_cache_tokens=1024)
            for steps in (h.trace_whole(requests), h.trace_tail_decode(requests, tail=8),
                          h.trace_portions(requests, sizes=(140, 5, 2, 150, 30))):
                got, forced = replay(eng, steps, "bfloat16")
                compare(cfg, weights, requests, got, TOL["bfloat16"], f"{name} page {page}", forced)
            used = {k for k, v in ops.CALLS.items() if v > before.get(k, 0)}
            if page == 64:
                assert all(any(k.startswith(w) for k in used) for w in ("attention_prefill_tc", "attention_decode")), sorted(used)
            every = {"hyper_step", "latent_append", "rope_copy", "rmsnorm_rows", "mamba2_prep", "delta_recurrence",
                     "mamba2_out", "router_plan"}
            assert every <= used, sorted(every - used)


def test_long_portions_beside_single_tokens(models):
    """Portions of a tile of new tokens and more (the tcgen05 kernel) in one step with single decoded tokens of other
    requests (the decode kernel), pages of 64: attention with reshaped scores over heads of 64 and latent rows of 128."""
    cfg, mdir, weights = models["B"]
    requests = {"a": tokens(cfg, 420, 31), "b": tokens(cfg, 200, 32), "c": tokens(cfg, 170, 33)}
    a, b, c = requests["a"], requests["b"], requests["c"]
    steps = [([("b", b[:60], list(range(60)))], []),
             ([("a", a[:150], list(range(150))), ("b", b[60:61], [0])], []),
             ([("a", a[150:300], list(range(150))), ("b", b[61:62], [0]), ("c", c[:129], list(range(129)))], []),
             ([("b", b[62:200], list(range(138))), ("a", a[300:301], [0]), ("c", c[129:130], [0])], ["b"]),
             ([("a", a[301:420], list(range(119))), ("c", c[130:170], list(range(40)))], ["a", "c"])]
    for dtype in ("float32", "bfloat16"):
        eng = engine(mdir, dtype, kv_page_size=64, kv_cache_tokens=1024)
        got, forced = replay(eng, steps, dtype)
        compare(cfg, weights, requests, got, TOL[dtype], f"long portions beside single tokens {dtype}", forced)


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_greedy_generation_through_the_entry_point(name, models):
    """hi_b200.generate (scheduler, sampler, launch-ahead) against greedy decoding of the plain model."""
    import hi_b200

    cfg, mdir, weights = models[name]
    prompts = [tokens(cfg, n, 40 + n) for n in (9, 1, 30, 17, 5)]
    outs = hi_b200.generate(mdir, prompts, hi_b200.SamplingParams(max_tokens=10, ignore_eos=True), dtype="float32",
                            kv_page_size=16, max_batch_size=3, kv_cache_tokens=512, max_batched_tokens=24)
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == 10
        ref = plain_logits(cfg, weights, list(prompt) + list(out.token_ids))
        for k, tok in enumerate(out.token_ids):
            logits = ref[len(prompt) - 1 + k]
            top2 = torch.topk(logits, 2).values
            if float(top2[0] - top2[1]) > 1e-3 * float(logits.abs().max()):
                assert tok == int(logits.argmax()), f"prompt of {len(prompt)}: token {k} is {tok}, plain model says {int(logits.argmax())}"


def test_trace_replay_as_a_user_runs_it(models, tmp_path):
    for name, dtype, seed in (("D", "float32", 5), ("B", "float32", 6)):
        cfg, mdir, weights = models[name]
        requests = {"a": tokens(cfg, 80, 21), "b": tokens(cfg, 33, 22), "c": tokens(cfg, 3, 23), "d": tokens(cfg, 50, 24),
                    "e": tokens(cfg, 20, 25)}
        steps = h.trace_mixed(requests, max_tokens=192, page=64, seed=seed, max_live=4)
        got = h.replay_subprocess(mdir, dtype, steps, max_tokens=192, out_dir=str(tmp_path / name), vocab=cfg["vocab"],
                                  extra=["--max-live", "4"])
        compare(cfg, weights, requests, got, TOL[dtype], f"trace_run {name} {dtype}")


def test_command_line_run_and_inspect(models, capsys):
    """``python -m hi_b200 run``: the next token, the top logits and greedy generation of a Bezasun folder."""
    import json

    from hi_b200.cli import main

    cfg, mdir, weights = models["D"]
    prompt = tokens(cfg, 12, 50)
    assert main(["run", mdir, "--tokens", ",".join(map(str, prompt)), "--max-tokens", "5", "--top-k", "3",
                 "--dtype", "float32", "--kv-page-size", "16", "--include-logits"]) == 0
    report = json.loads(capsys.readouterr().out)
    ref = plain_logits(cfg, weights, prompt)[-1]
    assert report["next_token"] == int(ref.argmax()) and report["logit_count"] == cfg["vocab"]
    assert float((torch.tensor(report["logits"], dtype=torch.float64) - ref).abs().max()) <= 3e-5 * float(ref.abs().max())
    assert [t["token_id"] for t in report["top_logits"]] == torch.topk(ref, 3).indices.tolist()
    assert len(report["generated_tokens"]) == 5 and report["generated_tokens"][0] == report["next_token"]
    assert main(["inspect", models["A"][1]]) == 0
    text = capsys.readouterr().out
    assert "hyper_connections" in text and "mamba2" in text and "latent_attention" in text and "routed_experts" in text
