"""Surinex without a GPU: the plain implementation's mechanisms against closed forms and against each other, the
configuration reader, and the ModelSpec the builder makes (schedule of a looped range, cache slots, state sizes)."""
import math

import pytest
import torch

import plain_surinex as plain
from surinex_configs import CONFIGS, SX_A, SX_B, SX_C, SX_D, SX_E, make_weights, plain_logits

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# --------------------------------------------------------------------------- mechanisms of the plain model
def test_time_convolution_reads_the_past_only():
    x, taps = rnd(9, 5, seed=1), rnd(5, 4, seed=2)
    y = plain.time_convolution(x, taps)
    # the last column weighs the token itself; the first token sees nothing else
    assert torch.allclose(y[0], taps[:, 3] * x[0])
    assert torch.allclose(y[5], taps[:, 0] * x[2] + taps[:, 1] * x[3] + taps[:, 2] * x[4] + taps[:, 3] * x[5])
    x2 = x.clone()
    x2[6:] += 1.0
    assert torch.equal(plain.time_convolution(x2, taps)[:6], y[:6])


def test_pair_frequencies_stretch_slow_pairs_only():
    plainf = plain.pair_frequencies(10000.0, 16)
    assert torch.allclose(plainf, torch.tensor([10000.0 ** (-2.0 * i / 16) for i in range(8)], dtype=F64))
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    f = plain.pair_frequencies(10000.0, 16, sc)
    lengths = 2 * math.pi / plainf
    for i in range(8):
        if lengths[i] < 64 / 4.0:
            assert f[i] == plainf[i]
        elif lengths[i] > 64 / 1.0:
            assert torch.isclose(f[i], plainf[i] / 4.0)
        else:
            assert plainf[i] / 4.0 < f[i] < plainf[i]
    assert any(16 <= l <= 64 for l in lengths.tolist())          # the blend is exercised


@pytest.mark.parametrize("layout", ["interleaved", "halves"])
def test_rotation_keeps_lengths_and_turns_back(layout):
    x, pos = rnd(7, 3, 12, seed=3), torch.arange(7) * 5
    f = plain.pair_frequencies(100.0, 8)
    y = plain.rotate(x, pos, f, layout)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    assert torch.allclose(plain.rotate(y, pos, f, layout, sign=-1.0), x)
    # dot products of two rotated vectors depend on the distance of their positions only
    a, b = plain.rotate(x[:1].expand(7, 3, 12), pos, f, layout), plain.rotate(x[1:2].expand(7, 3, 12), pos + 11, f, layout)
    d = (a * b).sum(-1)
    assert torch.allclose(d, d[:1].expand_as(d))
    u = torch.zeros(1, 1, 12, dtype=F64)
    u[0, 0, 0] = 1.0
    turned = plain.rotate(u, torch.tensor([1]), f, layout)[0, 0]
    partner = 1 if layout == "interleaved" else 4
    assert torch.isclose(turned[0], torch.cos(f[0])) and torch.isclose(turned[partner], torch.sin(f[0]))


def test_gated_linear_attention_equals_its_sum_form():
    """o_t = sum_{s<=t} (q_t * prod_{s<r<=t} alpha_r) . k_s v_s, written out without a state."""
    cfg = {"heads": 2, "dim": 3, "vdim": 4, "tau": 2.0}
    t_len, width = 6, 5
    w = {"m.q": rnd(6, width, seed=1), "m.k": rnd(6, width, seed=2), "m.v": rnd(8, width, seed=3), "m.g": rnd(8, width, seed=4),
         "m.o": torch.eye(8, dtype=F64), "m.norm": torch.ones(4, dtype=F64), "m.a1": rnd(2, width, seed=5),
         "m.a2": rnd(6, 2, seed=6), "m.a2.b": rnd(6, seed=7)}
    h = rnd(t_len, width, seed=8)
    got = plain.gated_linear_attention(h, cfg, w, "m", 1e-5)
    q = (h @ w["m.q"].T).view(t_len, 2, 3) * 3 ** -0.5
    k, v = (h @ w["m.k"].T).view(t_len, 2, 3), (h @ w["m.v"].T).view(t_len, 2, 4)
    alpha = (torch.sigmoid((h @ w["m.a1"].T) @ w["m.a2"].T + w["m.a2.b"]) ** 0.5).view(t_len, 2, 3)
    out = torch.zeros(t_len, 2, 4, dtype=F64)
    for t in range(t_len):
        for s in range(t + 1):
            keep = torch.ones(2, 3, dtype=F64)
            for r in range(s + 1, t + 1):
                keep = keep * alpha[r]
            out[t] += ((q[t] * keep * k[s]).sum(-1, keepdim=True)) * v[s]
    out = plain.rms_norm(out, None, 1e-5).reshape(t_len, 8) * plain.silu(h @ w["m.g"].T)
    assert torch.allclose(got, out, atol=1e-12)


def test_delta_rule_overwrites_a_repeated_key():
    """With beta = 1, no decay and the same unit key twice, the second write replaces the first value: the
    read-out with that key returns the second value alone."""
    k = torch.tensor([0.6, 0.8], dtype=F64)
    s = torch.zeros(2, 3, dtype=F64)
    for v in (torch.tensor([1.0, 2.0, 3.0], dtype=F64), torch.tensor([-4.0, 0.5, 9.0], dtype=F64)):
        u = 1.0 * (v - s.T @ k)
        s = s + torch.outer(k, u)
    assert torch.allclose(s.T @ k, torch.tensor([-4.0, 0.5, 9.0], dtype=F64))


def test_sigmoid_attention_weights_are_not_normalised_and_values_turn_with_distance():
    """One head, keys and queries fixed so that every visible weight is sigmoid(pb): the output at position i is
    sigmoid(pb) times the sum of the values turned by (j - i)."""
    p = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0, "rot": {"base": 50.0, "dims": 2}}
    t_len, width = 5, 4
    w = {"m.q": torch.zeros(4, width, dtype=F64), "m.k": torch.zeros(4, width, dtype=F64), "m.v": torch.eye(4, dtype=F64),
         "m.q.norm": torch.ones(4, dtype=F64), "m.k.norm": torch.ones(4, dtype=F64), "m.pb": torch.tensor([-0.7], dtype=F64),
         "m.o": torch.eye(4, dtype=F64)}
    h = rnd(t_len, width, seed=4)
    got = plain.sigmoid_attention(h, p, w, "m", 1e-5)
    fv = plain.pair_frequencies(50.0, 4)
    sig = 1.0 / (1.0 + math.exp(0.7))
    for i in range(t_len):
        want = torch.zeros(4, dtype=F64)
        for j in range(i + 1):
            want += plain.rotate(h[j].view(1, 1, 4), torch.tensor([j - i]), fv, "interleaved")[0, 0]
        assert torch.allclose(got[i], sig * want, atol=1e-12)


def test_latent_attention_first_token_returns_its_own_value():
    cfg = SX_A["layers"][2]["mixer"]
    w = {k[len("l2."):]: v.double() for k, v in make_weights(SX_A, 3).items() if k.startswith("l2.mix")}
    h = rnd(4, SX_A["width"], seed=6)
    out = plain.latent_attention(h, cfg, w, "mix", 1e-5)
    c = plain.rms_norm((h[:1] @ w["mix.dkv"].T)[:, : cfg["kv_rank"]], w["mix.dkv.norm"], 1e-5)
    assert torch.allclose(out[0], (c @ w["mix.uv"].T) @ w["mix.o"].T, atol=1e-10)


def test_layer_order_and_pass_offsets():
    assert plain.layer_order(SX_A) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.layer_order(SX_C) == [(0, None), (1, None)]
    assert plain.layer_order(SX_D) == [(0, None), (1, None), (2, 0)]
    # the vector of a pass reaches the logits; so does the embedding output that later passes add again
    w = make_weights(SX_A, 5)
    toks = [3, 9, 27, 81, 5]
    base = plain_logits(SX_A, w, toks)
    w2 = dict(w)
    w2["loop.step"] = w["loop.step"].clone()
    w2["loop.step"][1] += 1.0
    assert float((plain_logits(SX_A, w2, toks) - base).abs().max()) > 1e-3


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_token_depends_on_the_past_only(name):
    cfg = CONFIGS[name]
    w = make_weights(cfg, 11)
    toks = torch.randint(0, cfg["vocab"], (14,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = plain_logits(cfg, w, toks)
    assert torch.isfinite(whole).all()
    assert torch.allclose(plain_logits(cfg, w, toks[:9]), whole[:9], atol=1e-9)


# --------------------------------------------------------------------------- configuration and ModelSpec
def test_config_reader_takes_every_size_from_the_json():
    from hi_b200.config.surinex import SurinexConfig, sizes_from_tensors

    cfg = SurinexConfig.from_json(SX_D)
    assert (cfg.vocab, cfg.width, cfg.taps, cfg.eps) == (90, 40, 8, 1e-5)
    left, right = cfg.layers[2].mixer
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.rot.dims, left.rot.scaling) == (2, 2, 8, 40, 4, (2.0, 0.5, 4.0, 16.0))
    assert (right.heads, right.kv_heads, right.dim, right.vdim, right.conv) == (4, 1, 24, 8, 5)
    assert cfg.layers[0].ff is None and cfg.layers[1].ff == 56 and cfg.loop.times == 1
    lat = cfg.layers[1].mixer
    assert (lat.kv_rank, lat.q_rank, lat.rot_dim, lat.rot.base) == (12, 40, 16, 100.0)
    assert SurinexConfig.from_json(SX_C).loop is None
    sized = sizes_from_tensors(SurinexConfig.from_json(SX_E), {"l1.mix.a1": (3, 50), "l3.mix.a1": (9, 50)})
    assert sized.layers[1].mixer.decay_rank == 3 and sized.layers[3].mixer.decay_rank == 9


@pytest.mark.parametrize("path,value,word", [
    (("canon", "taps"), 0, "canon.taps"), (("layers", 0, "type"), "conv", "type"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 2, "mixer", "rot", "dims"), 6, "rot.dims"),
    (("loop", "stop"), 9, "loop"), (("layers", 1, "mixer", "left", "rot", "scaling", "factor"), -1.0, "scaling")])
def test_config_errors_name_the_key(path, value, word):
    import copy

    from hi_b200.config.base import ConfigError
    from hi_b200.config.surinex import SurinexConfig

    raw = copy.deepcopy(SX_A)
    node = raw
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        SurinexConfig.from_json(raw)


def test_spec_runs_looped_layers_with_caches_of_their_own():
    from hi_b200.config.surinex import SurinexConfig
    from hi_b200.parts.surinex import build_surinex_spec

    spec = build_surinex_spec(SurinexConfig.from_json(SX_A))
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [e.cache for e in spec.schedule] == list(range(6))
    assert [(e.interlude, e.interlude_arg) for e in spec.schedule] == [(None, 0), (0, 0), (None, 0), (0, 1), (None, 0), (None, 0)]
    assert spec.interludes[0].kind == "pass_offset" and spec.interludes[0].params["times"] == 2
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.kind == "dense_swiglu"
    assert spec.layers[1].mixer.kind == "mixer_pair" and spec.layers[1].mixer.params["right"]["params"]["decay_per"] == "head"
    flat = build_surinex_spec(SurinexConfig.from_json(SX_C))
    assert flat.interludes == () and all(e.interlude is None for e in flat.schedule)


def test_model_declares_every_tensor_of_the_checkpoint_and_its_state():
    from hi_b200.config.surinex import SurinexConfig
    from hi_b200.parts.model import Model
    from hi_b200.parts.surinex import build_surinex_spec, normalize_surinex_tensor_name

    for cfg in CONFIGS.values():
        model = Model(build_surinex_spec(SurinexConfig.from_json(cfg)), torch.float32, "cpu")
        want = {normalize_surinex_tensor_name(k): tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
        have = {t.name: tuple(t.shape) for t in model.tensor_specs() if t.init != "absent"}
        assert have == want
    model = Model(build_surinex_spec(SurinexConfig.from_json(SX_A)), torch.float32, "cpu")
    taps, width = SX_A["canon"]["taps"], SX_A["width"]
    assert model.block_state_sizes == {slot: (taps - 1) * width for slot in range(6)}
    pair = model.cache_specs[1]
    assert pair.paged and pair.kv_heads == 2 and pair.state_shape and model.cache_specs[1] == model.cache_specs[3]
    assert model.cache_specs[0].state_shape == (2 * 16 * 24,) and not model.cache_specs[0].paged
    assert model.cache_specs[2].paged and not model.cache_specs[2].values
    assert Model(build_surinex_spec(SurinexConfig.from_json(SX_C)), torch.float32, "cpu").block_state_sizes == {}
