"""CPU tests of the Vinurax pieces that need no GPU: the configuration reader, the model as data, the
names the parts ask for, and the plain implementation against itself (a sequence fed whole, in portions
and token by token must give the same logits) and against hand-computable cases."""
import json
import math

import pytest
import torch

import plain_vinurax as plain
from vinurax_configs import VX_A, VX_B, VX_C, VX_D, VX_E, config, delta, latent, make_weights, write_model


@pytest.mark.parametrize("cfg", [VX_A, VX_B, VX_C, VX_D, VX_E])
def test_plain_model_portions_equal_whole(cfg):
    w = make_weights(cfg, 5)
    m = plain.PlainVinurax(cfg, w)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg["vocab"], (41,), generator=g).tolist()
    whole = m.logits(toks)
    seq, rows, pos = m.new_sequence(), [], 0
    for n in (5, 1, 2, 1, 1, 9, 2, 20):
        rows.append(m.forward(seq, toks[pos: pos + n]))
        pos += n
    assert pos == len(toks)
    assert float((torch.cat(rows) - whole).abs().max()) < 1e-9 * float(whole.abs().max())
    assert float(whole.std()) > 0.3          # the weights give logits of order one


def test_hand_computable_pieces():
    x = torch.tensor([[3.0, -4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms(x, 0.0), x / math.sqrt(12.5))
    w = {"n": torch.tensor([2.0, 1.0]), "n.b": torch.tensor([0.5, -0.5]), "n.alpha": torch.tensor(0.5)}
    want = torch.tanh(torch.tensor([1.5, -2.0])) * torch.tensor([2.0, 1.0]) + torch.tensor([0.5, -0.5])
    assert torch.allclose(plain.dynamic_tanh(x.float(), w, "n"), want[None])
    act = torch.tensor([0.0, 0.0], dtype=torch.float64)           # softplus(0) = ln 2
    z = torch.tensor([2.0, -1.0, 0.0], dtype=torch.float64)
    ln2 = math.log(2.0)
    want = torch.tensor([ln2 * 4 + 1.0, (0.5 + ln2) * (math.exp(-1) - 1 + 1) - 0.5, 0.0], dtype=torch.float64)
    assert torch.allclose(plain.xielu(z, act), want)
    # the convolution's last tap is the token's own; zeros before the start
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=torch.float64)
    xs = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    y, carry = plain.short_conv(xs, taps, torch.zeros(2, 1, dtype=torch.float64))
    raw = torch.tensor([100.0, 210.0, 321.0], dtype=torch.float64)
    assert torch.allclose(y[:, 0], raw * torch.sigmoid(raw)) and carry[:, 0].tolist() == [2.0, 3.0]


def test_delta_rule_writes_then_reads_the_token():
    """One head, key = query direction, beta = 1, no decay: the read-out of the token that was just written is
    its own value times q.k, and a second token with an orthogonal key does not disturb the first."""
    cfg = config(4, 2, 1e-5, [delta(1, 1, 2, 2, 1)])
    w = {k: torch.zeros_like(v, dtype=torch.float64) for k, v in make_weights(cfg, 0).items()}
    p = "l0.mix"
    w[p + ".q"] = w[p + ".k"] = torch.eye(2, dtype=torch.float64)
    w[p + ".v"] = torch.eye(2, dtype=torch.float64) * 2
    for n in "qkv":
        w[f"{p}.{n}.conv"] = torch.ones(2, 1, dtype=torch.float64)
    w[p + ".dt_bias"] = torch.full((2,), -50.0, dtype=torch.float64)      # softplus -> 0: decay 1
    w[p + ".b"] = torch.full((1, 2), 50.0, dtype=torch.float64)           # beta -> 1 for positive inputs
    w[p + ".norm"] = torch.ones(2, dtype=torch.float64)
    w[p + ".o"] = torch.eye(2, dtype=torch.float64)
    h = torch.tensor([[3.0, 0.0], [0.0, 5.0], [3.0, 0.0]], dtype=torch.float64)
    out, state = plain.channel_delta(h, None, w, p, cfg["layers"][0]["mixer"], 0.0)
    silu = lambda t: t * torch.sigmoid(t)
    S = state["S"][0]
    # rows of S are key channels: token 0 wrote silu(2*3) along key (1, 0), token 1 silu(2*5) along (0, 1)
    assert torch.allclose(S[0], torch.tensor([float(silu(torch.tensor(6.0))), 0.0], dtype=torch.float64), atol=1e-6)
    assert torch.allclose(S[1], torch.tensor([0.0, float(silu(torch.tensor(10.0)))], dtype=torch.float64), atol=1e-6)
    # the third token repeats the first: nothing to correct, the state stays
    assert out.shape == (3, 2)


def test_config_reader_and_spec():
    from hi_b200.config.base import ConfigError
    from hi_b200.config.registry import lookup
    from hi_b200.parts.model import Model

    arch = lookup(VX_A)
    cfg = arch.parse_config(VX_A, None)
    assert [l.kind for l in cfg.layers] == [l["type"] for l in VX_A["layers"]] and cfg.layers[3].ff is None
    spec = arch.build_spec(cfg)
    assert [(e.cache, e.writes_cache) for e in spec.schedule] == [(0, True), (1, True), (1, False), (3, True), (4, True)]
    model = Model(spec, torch.bfloat16, "cpu")
    assert model.cache_specs[1].head_dim == 64 and not model.cache_specs[1].values and model.cache_specs[4].head_dim == 64
    assert model.cache_specs[0].state_shape == (4 * 16 * 24 + 3 * (2 * 2 * 16 + 4 * 24),)
    for bad, word in (({**VX_A, "layers": [latent(2, 8, 8, 16, 0.1, kv_from=0)]}, "kv_from"),
                      ({**VX_A, "layers": [delta(3, 2, 8, 8, 2)]}, "kv_heads"),
                      ({**VX_A, "layers": [{"type": "other", "mixer": {}}]}, "type"),
                      ({k: v for k, v in VX_A.items() if k != "norm"}, "norm"),
                      ({**VX_A, "layers": [latent(2, 8, 8, 16, 0.1), latent(2, 8, 8, 24, 0.1, kv_from=0)]}, "kv_rank")):
        with pytest.raises(ConfigError, match=word):
            arch.parse_config(bad, None)


def test_inner_sizes_come_from_the_checkpoint_and_names_bind(tmp_path):
    from hi_b200.config.registry import load_architecture
    from hi_b200.parts.model import Model
    from hi_b200.weights.loader import check_names
    from hi_b200.weights.safetensors_io import Checkpoint

    for k, cfg in enumerate((VX_A, VX_B, VX_C, VX_D, VX_E)):
        d = str(tmp_path / f"m{k}")
        weights = write_model(d, cfg, 3, decay_rank=7, gate_rank=3)
        arch, typed, _raw = load_architecture(d)
        for layer in typed.layers:
            if layer.kind == "channel_delta":
                assert (layer.decay_rank, layer.gate_rank) == (7, 3)
        model = Model(arch.build_spec(typed), torch.bfloat16, "cpu")
        ck = Checkpoint(d)
        check_names(model.tensor_specs(), {arch.normalize_tensor_name(n): ck.describe(n)[1] for n in ck.names()}, d)
        assert len(weights) == len(ck.names())


def test_random_weights_writer_and_inspect(tmp_path, capsys):
    from hi_b200.cli import main

    cfg_path = tmp_path / "c.json"
    cfg_path.write_text(json.dumps(VX_B))
    assert main(["random-weights", str(cfg_path), str(tmp_path / "m"), "--seed", "4"]) == 0
    capsys.readouterr()
    assert main(["inspect", str(tmp_path / "m")]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["architecture"] == "vinurax" and report["tensors"]["status"] == "ok"
    assert [l["mixer"] for l in report["layers"]] == [l["type"] for l in VX_B["layers"]]
    assert report["schedule_cache_slots"] == [0, 1, 0, 3, 4]
