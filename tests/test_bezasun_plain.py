"""Bezasun without a GPU: the plain implementation's mechanisms against closed forms and against each other, the
configuration reader, and the ModelSpec the builder makes (parts, cache needs, tensor names)."""
import copy
import math

import pytest
import torch

import plain_bezasun as plain
from bezasun_configs import BZ_A, BZ_C, BZ_D, BZ_E, CONFIGS, make_weights, plain_logits

F64 = torch.float64


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# --------------------------------------------------------------------------- mechanisms of the plain model
def test_convolution_reads_the_past_only_and_adds_its_bias():
    x, taps, bias = rnd(9, 5, seed=1), rnd(5, 4, seed=2), rnd(5, seed=3)
    y = plain.causal_convolution(x, taps, bias)
    assert torch.allclose(y[0], bias + taps[:, 3] * x[0])
    assert torch.allclose(y[5], bias + taps[:, 0] * x[2] + taps[:, 1] * x[3] + taps[:, 2] * x[4] + taps[:, 3] * x[5])
    x2 = x.clone()
    x2[6:] += 1.0
    assert torch.equal(plain.causal_convolution(x2, taps, bias)[:6], y[:6])


def test_ramped_frequencies_slow_the_slow_pairs_only():
    f0, one = plain.yarn_frequencies(32, 10000.0, None)
    assert one == 1.0 and torch.allclose(f0, torch.tensor([10000.0 ** (-2.0 * i / 32) for i in range(16)], dtype=F64))
    sc = {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}
    f, mag = plain.yarn_frequencies(32, 10000.0, sc)
    assert math.isclose(mag, 0.1 * math.log(8.0) + 1.0)
    turns = 512 * f0 / (2 * math.pi)                       # turns of a pair over the original length
    assert torch.equal(f[turns > 40.0], f0[turns > 40.0])   # clearly fast pairs stay
    assert torch.allclose(f[turns < 0.8], f0[turns < 0.8] / 8.0)
    mid = (turns > 1.5) & (turns < 25.0)
    assert bool(mid.any()) and bool(((f[mid] < f0[mid]) & (f[mid] > f0[mid] / 8.0)).all())


def test_interleaved_rotation_turns_neighbours():
    x, pos = rnd(7, 3, 8, seed=3), torch.arange(7) * 5
    f, _ = plain.yarn_frequencies(8, 100.0, None)
    y = plain.rotate_interleaved(x, pos, f, 1.0)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    u = torch.zeros(1, 1, 8, dtype=F64)
    u[0, 0, 2] = 1.0                                        # dim 2 is the first of pair 1: it turns into dim 3
    t = plain.rotate_interleaved(u, torch.tensor([1]), f, 1.0)[0, 0]
    assert math.isclose(float(t[2]), math.cos(float(f[1]))) and math.isclose(float(t[3]), math.sin(float(f[1])))
    assert float(t[[0, 1, 4, 5, 6, 7]].abs().max()) == 0.0
    # a factor on cos and sin scales the turned vector
    assert torch.allclose(plain.rotate_interleaved(x, pos, f, 1.3), 1.3 * y)
    # dot products depend on the distance of the positions only
    a = plain.rotate_interleaved(x[:1].expand(7, 3, 8), pos, f, 1.0)
    b = plain.rotate_interleaved(x[1:2].expand(7, 3, 8), pos + 11, f, 1.0)
    d = (a * b).sum(-1)
    assert torch.allclose(d, d[:1].expand_as(d))


def _one_layer(layer, **kw):
    cfg = {"architecture": "Bezasun", "vocab": 19, "width": 24, "norm": {"eps": 1e-5}, "layers": [layer], **kw}
    return cfg, {k: v.double() for k, v in make_weights(cfg, 3).items()}


def test_latent_attention_sees_its_window_only():
    from bezasun_configs import latent

    cfg, w = _one_layer(latent(2, 8, 4, 6, 10, 7, 0.4, 100.0, window=5))
    m = cfg["layers"][0]["mixer"]
    h = rnd(20, 24, seed=5)
    y = plain.latent_attention(h, m, w, "l0.mix", 1e-5)
    h2 = h.clone()
    h2[:10] += 1.0                                           # tokens 0..9: outside the window of 14 and later
    y2 = plain.latent_attention(h2, m, w, "l0.mix", 1e-5)
    assert torch.allclose(y2[14:], y[14:], atol=1e-12) and not torch.allclose(y2[13], y[13])
    m_all = {k: v for k, v in m.items() if k != "mask"}
    assert not torch.allclose(plain.latent_attention(h2, m_all, w, "l0.mix", 1e-5)[19], y[19])


def test_mamba2_is_its_recurrence_and_carries_a_state():
    from bezasun_configs import mamba

    cfg, w = _one_layer(mamba(4, 6, 5, 2, 3, 2))
    m = cfg["layers"][0]["mixer"]
    h = rnd(12, 24, seed=6)
    y = plain.mamba2(h, m, w, "l0.mix", 1e-5)
    h2 = h.clone()
    h2[8:] += 1.0
    assert torch.equal(plain.mamba2(h2, m, w, "l0.mix", 1e-5)[:8], y[:8])          # causal
    h3 = h.clone()
    h3[0] += 1.0
    assert not torch.allclose(plain.mamba2(h3, m, w, "l0.mix", 1e-5)[11], y[11])   # the state remembers
    # a very negative dt bias switches the recurrence off: what is left is the skip through D
    w2 = dict(w)
    w2["l0.mix.dt_bias"] = torch.full((4,), -60.0, dtype=F64)
    proj = h @ w["l0.mix.in"].T
    inner = 24
    xbc = plain.silu(plain.causal_convolution(proj[:, inner: 2 * inner + 20], w["l0.mix.conv"], w["l0.mix.conv.b"]))
    skip = (xbc[:, :inner].view(12, 4, 6) * w["l0.mix.D"][None, :, None]).reshape(12, inner) * plain.silu(proj[:, :inner])
    want = plain.rms_norm(skip.view(12, 2, 12), None, 1e-5).reshape(12, inner) * w["l0.mix.norm"] @ w["l0.mix.o"].T
    assert torch.allclose(plain.mamba2(h, m, w2, "l0.mix", 1e-5), want, atol=1e-9)


def test_attention_bias_sink_cap_and_temperature_each_matter():
    from bezasun_configs import attention

    cfg, w = _one_layer(attention(4, 2, 8, 6, 0.8, softcap=3.0, q_temp=(0.5, 4)))
    m = cfg["layers"][0]["mixer"]
    h = rnd(15, 24, seed=7)
    y = plain.attention(h, m, w, "l0.mix", 1e-5)
    h2 = h.clone()
    h2[9:] += 1.0
    assert torch.equal(plain.attention(h2, m, w, "l0.mix", 1e-5)[:9], y[:9])       # causal
    for change in ({"softcap": None}, {"q_temp": None}, {"softcap": 30.0}, {"q_temp": {"coef": 0.5, "every": 5}}):
        assert not torch.allclose(plain.attention(h, {**m, **change}, w, "l0.mix", 1e-5), y)
    # the temperature is 1 before the first step of `every` positions
    assert torch.allclose(plain.attention(h, {**m, "q_temp": None}, w, "l0.mix", 1e-5)[:3], y[:3])
    w2 = dict(w)
    w2["l0.mix.sink"] = w["l0.mix.sink"] - 50.0              # a sink that weighs nothing: an ordinary softmax
    no_sink = plain.attention(h, m, w2, "l0.mix", 1e-5)
    assert not torch.allclose(no_sink, y)
    # the first token sees itself and the sink only: its output is its own value times 1 / (1 + e^(sink - score))
    q = plain.rms_norm((h[:1] @ w["l0.mix.q"].T).view(1, 4, 8), w["l0.mix.q.norm"], 1e-5)
    k = plain.rms_norm((h[:1] @ w["l0.mix.k"].T).view(1, 2, 8), w["l0.mix.k.norm"], 1e-5)
    v = (h[:1] @ w["l0.mix.v"].T).view(2, 6)
    outs = []
    for a in range(4):
        s = 3.0 * torch.tanh((q[0, a] @ k[0, a // 2]) * 0.8 / 3.0)
        outs.append(v[a // 2] / (1.0 + torch.exp(w["l0.mix.sink"][a] - s)))
    assert torch.allclose(y[0], torch.cat(outs) @ w["l0.mix.o"].T, atol=1e-10)


def test_mixture_weighs_by_unnormalised_softmax_scores():
    from bezasun_configs import latent, moe

    cfg, w = _one_layer(latent(1, 8, 2, 8, 8, 8, 0.3, 100.0, mlp=moe(5, 2, 7, shared=9)))
    mlp = cfg["layers"][0]["mlp"]
    h = rnd(6, 24, seed=8)
    ids, scores = plain.router_choice(h, mlp, w, "l0.mlp")
    full = torch.softmax(h @ w["l0.mlp.router"].T, dim=1)
    assert torch.equal(ids, torch.topk(full, 2, dim=1).indices) and bool((scores.sum(1) < 1.0).all())
    y = plain.mixture(h, mlp, w, "l0.mlp")
    t = 4
    want = sum(scores[t, r] * plain.expert(h[t: t + 1], w, f"l0.mlp.e{int(ids[t, r])}")[0] for r in range(2))
    assert torch.allclose(y[t], want + plain.expert(h[t: t + 1], w, "l0.mlp.shared")[0])


def test_copies_of_the_stream_with_unit_coefficients_are_one_stream():
    """One copy with in = out = mix = 1 is the plain pre-norm block; so are S copies whose mix is the identity and
    whose `in` picks one copy, read at that copy."""
    cfg = copy.deepcopy(BZ_C)
    w = make_weights(cfg, 4)
    toks = [5, 9, 33, 2, 17, 40, 8]
    base = plain_logits(cfg, w, toks)
    one = copy.deepcopy(cfg)
    one["streams"] = 1
    w1 = dict(w)
    for i, layer in enumerate(cfg["layers"]):
        for q in (1, 2) if layer["mlp"] else (1,):
            w1[f"l{i}.hc{q}.in"] = torch.ones(1)
            w1[f"l{i}.hc{q}.out"] = torch.ones(1)
            w1[f"l{i}.hc{q}.mix"] = torch.ones(1, 1)
    assert torch.allclose(plain_logits(one, w1, toks), base, atol=1e-10)
    # the update of all copies reads the old ones: mix is indexed [from, to]
    two = copy.deepcopy(cfg)
    two["streams"] = 2
    w2 = dict(w)
    for i, layer in enumerate(cfg["layers"]):
        for q in (1, 2) if layer["mlp"] else (1,):
            w2[f"l{i}.hc{q}.in"] = torch.tensor([1.0, 0.0])
            w2[f"l{i}.hc{q}.out"] = torch.tensor([1.0, 0.0])
            w2[f"l{i}.hc{q}.mix"] = torch.tensor([[1.0, 1.0], [0.0, 0.0]])      # copy 0 feeds both, copy 1 feeds nothing
    x = {k: v.double() for k, v in w2.items()}
    outs = []
    plain.forward(two, x, toks, layer_outputs=outs)
    ref = []
    plain.forward(cfg, {k: v.double() for k, v in w.items()}, toks, layer_outputs=ref)
    # copy 0 follows the plain stream; copy 1 is copy 0 before the last sub-layer's result: their sum is not twice it
    assert not torch.allclose(outs[-1], 2.0 * ref[-1])


def test_multipliers_scale_what_they_say():
    cfg = copy.deepcopy(BZ_A)
    w = make_weights(cfg, 5)
    toks = [3, 99, 14, 60, 7]
    base = plain_logits(cfg, w, toks)
    doubled = copy.deepcopy(cfg)
    doubled["logit_scale"] = 2.0 * cfg["logit_scale"]
    assert torch.allclose(plain_logits(doubled, w, toks), 2.0 * base)
    for key, value in (("residual_mult", 0.3), ("embedding", {"scale": 1.1})):
        other = copy.deepcopy(cfg)
        other[key] = value
        assert not torch.allclose(plain_logits(other, w, toks), base)


# --------------------------------------------------------------------------- configuration and spec
def test_config_reader_takes_every_size_and_names_the_key():
    from hi_b200.config.base import ConfigError
    from hi_b200.config.bezasun import BezasunConfig

    cfg = BezasunConfig.from_json(BZ_A)
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.residual_mult, cfg.embedding_scale, cfg.logit_scale) == (131, 64, 3, 0.7, 0.5, 2.0)
    lat, mam, att = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[2].mixer
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.q_rank, lat.window) == (2, 16, 8, 16, 24, 20, 40)
    assert lat.rot.scaling == (4.0, 64.0, 8.0, 1.0)
    assert (mam.heads, mam.vdim, mam.state, mam.groups, mam.conv, mam.norm_groups) == (4, 8, 16, 2, 3, 2)
    assert (att.heads, att.kv_heads, att.softcap, att.q_temp) == (4, 2, 20.0, (0.5, 32.0))
    assert (cfg.layers[0].mlp.experts, cfg.layers[0].mlp.top, cfg.layers[0].mlp.ff, cfg.layers[0].mlp.shared_ff) == (8, 2, 24, 32)
    bare = BezasunConfig.from_json(BZ_C)
    assert bare.streams is None and bare.residual_mult == 1.0 and bare.embedding_scale == 1.0 and bare.logit_scale == 1.0
    assert bare.layers[0].mixer.window is None and bare.layers[0].mixer.rot.scaling is None
    assert bare.layers[1].mlp is None and bare.layers[1].mixer.softcap is None and bare.layers[1].mixer.q_temp is None
    assert bare.layers[0].mlp.shared_ff is None
    for path, value, word in ((("layers", 0, "mixer", "kv_rank"), None, "kv_rank"), (("layers", 1, "mixer", "groups"), 3, "groups"),
                              (("layers", 2, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
                              (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"), (("norm",), None, "norm"),
                              (("layers", 0, "type"), "conv", "type"), (("streams",), 40, "streams")):
        bad = copy.deepcopy(BZ_A)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            BezasunConfig.from_json(bad)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_spec_asks_for_exactly_the_checkpoints_tensors(name):
    from hi_b200.config.registry import lookup
    from hi_b200.parts.model import Model

    cfg = CONFIGS[name]
    arch = lookup(cfg)
    assert arch.name == "bezasun"
    model = Model(arch.build_spec(arch.parse_config(cfg, None)), torch.float32, "cpu")
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs() if s.init != "absent"}
    have = {arch.normalize_tensor_name(k): tuple(v.shape) for k, v in make_weights(cfg, 1).items()}
    assert specs == have
    assert model.graph_safe


def test_spec_parts_and_cache_needs():
    from hi_b200.config.registry import lookup
    from hi_b200.parts.model import Model

    arch = lookup(BZ_A)
    spec = arch.build_spec(arch.parse_config(BZ_A, None))
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "mamba2", "attention", "latent_attention"]
    assert all(l.arrangement.kind == "hyper_connections" and l.arrangement.params["streams"] == 3 for l in spec.layers)
    assert all(l.feed_forward.kind == "routed_experts" and l.feed_forward.params["score"] == "softmax"
               and l.feed_forward.params["scale"] == "output" for l in spec.layers)
    assert spec.final_norm.params["one_plus"] and spec.head.params["scale"] == 2.0
    model = Model(spec, torch.float32, "cpu")
    c = model.cache_specs
    assert c[0].paged and not c[0].values and c[0].window == ("sliding", 40) and c[3].window == ("sliding", 23)
    assert not c[1].paged and c[1].state_shape == (4 * 16 * 8 + 2 * (32 + 2 * 2 * 16),)
    assert c[2].paged and c[2].values and c[2].kv_heads == 2 and c[2].window is None
    plain_stream = arch.build_spec(arch.parse_config(BZ_C, None))
    assert all(not l.arrangement.params["learned"] and l.arrangement.params["streams"] == 1 for l in plain_stream.layers)
    assert plain_stream.layers[1].feed_forward is None and plain_stream.layers[1].norm_feed_forward is None
    wide = Model(arch.build_spec(arch.parse_config(BZ_D, None)), torch.float32, "cpu")
    assert wide.cache_specs[0].head_dim == 16 and wide.cache_specs[3].head_dim == 32      # value and key sizes padded to one row
    assert Model(arch.build_spec(arch.parse_config(BZ_E, None)), torch.float32, "cpu").cache_specs[2].head_dim == 224


def test_random_weights_folder_round_trip(tmp_path):
    """The framework's own random-weights writer makes a folder the loader's tensor list accepts."""
    from hi_b200.config.registry import load_architecture
    from hi_b200.weights import write_random_model
    from hi_b200.weights.safetensors_io import Checkpoint

    d = write_random_model(BZ_D, str(tmp_path / "m"), seed=3, std=0.05)
    arch, cfg, _raw = load_architecture(d)
    assert arch.name == "bezasun" and cfg.streams == 5
    names = set(Checkpoint(d).names())
    assert {"embed.weight", "head", "final.norm", "l0.hc1.mix", "l1.mix.conv.b", "l0.mix.sink", "l2.mlp.shared.down", "l2.mlp.e6.up"} <= names
