"""Norusun without a GPU: the registry, the generator of made-up checkpoints, the packing of the residual streams' numbers,
and the plain restatement's mechanisms on cases with closed forms (what the GPU tests compare the kernels with)."""

import json
import math

import pytest
import torch

from oracle import norusun as O
from tiny_llm_b200.layer_norm import ResidualStreams
from tiny_llm_b200.models import ARCHITECTURES
from tiny_llm_b200.synthetic import norusun_config, save_norusun, synthetic_norusun

D64 = torch.float64


def test_registry_names_the_design():
    assert ARCHITECTURES["Norusun"] == ("tiny_llm_b200.norusun", "NorusunModel")


def test_generator_spells_the_stack_and_round_trips_through_a_directory(tmp_path):
    config = norusun_config(pattern="WnLdPd", width=96, wkv_heads=3, wkv_dim=32, streams=3, canon_taps=2)
    assert [l["type"] for l in config["layers"]] == ["wkv", "latent_attention", "parallel"]
    assert config["layers"][0]["mlp"] is None and config["layers"][1]["mlp"]["kind"] == "dense"
    tensors = synthetic_norusun(config, seed=3)
    assert tensors["l0.norm1"].shape == () and tensors["final.norm"].shape == ()
    assert tensors["l1.hc2.mix"].shape == (3, 3) and tensors["l0.canon1"].shape == (96, 2)
    assert "l0.norm2" not in tensors and "l0.hc2.in" not in tensors
    right = config["layers"][2]["mixer"]["right"]
    inner = right["heads"] * right["vdim"]
    assert tensors["l2.mix.right.in"].shape[0] == 2 * inner + 2 * right["groups"] * right["state"] + right["heads"]
    save_norusun(config, tensors, tmp_path / "m")
    from tiny_llm_b200.checkpoint import read_tensors

    again = read_tensors(tmp_path / "m")
    assert set(again) == set(tensors) and json.loads((tmp_path / "m" / "config.json").read_text()) == config
    assert all(torch.equal(again[k], tensors[k]) for k in tensors)
    plain = norusun_config(pattern="Ld", streams=0, canon_taps=0)
    assert "streams" not in plain and "canon" not in plain
    assert not any(".hc" in k or "canon" in k for k in synthetic_norusun(plain))
    with pytest.raises(ValueError):
        norusun_config(pattern="Xd")


def test_sites_of_the_residual_streams_pack_their_numbers():
    s = ResidualStreams(3, 1e-6, torch.float32, "cpu")
    read = s.read_site(torch.tensor(1.5), torch.tensor([0.5, 0.25, 2.0]))
    assert read.tolist() == [0.5, 0.25, 2.0, 1.5]
    mix = torch.arange(9.0).reshape(3, 3)
    write = s.write_site(mix, torch.tensor([1.0, 2.0, 3.0]))
    assert write.tolist() == list(range(9)) + [1.0, 2.0, 3.0]          # [from, to] row by row, then the output weights
    one = ResidualStreams(1, 1e-6, torch.float32, "cpu")                  # the plain residual sum
    assert one.read_site(torch.tensor(0.75)).tolist() == [1.0, 0.75] and one.write_site().tolist() == [1.0, 1.0]
    with pytest.raises(ValueError):
        ResidualStreams(9, 1e-6, torch.float32, "cpu")
    with pytest.raises(ValueError):
        s.read_site(torch.ones(4), None)


def test_streams_with_identity_mixing_are_the_ordinary_residual():
    g = torch.Generator().manual_seed(0)
    xs, y = torch.randn(3, 5, 7, generator=g, dtype=D64), torch.randn(5, 7, generator=g, dtype=D64)
    out = O.streams_write(xs, y, torch.eye(3, dtype=D64), torch.ones(3, dtype=D64))
    assert torch.allclose(out, xs + y[None])
    mix = torch.tensor([[0.0, 1.0], [1.0, 0.0]], dtype=D64)               # [from, to]: the streams swap places
    out = O.streams_write(xs[:2], y, mix, torch.zeros(2, dtype=D64))
    assert torch.equal(out[0], xs[1]) and torch.equal(out[1], xs[0])
    assert torch.allclose(O.streams_read(xs, torch.tensor([1.0, 0.0, -2.0], dtype=D64)), xs[0] - 2 * xs[2])


def test_causal_convolution_by_hand():
    x = torch.tensor([[1.0], [2.0], [4.0], [8.0]], dtype=D64)
    taps = torch.tensor([[100.0, 10.0, 1.0]], dtype=D64)                  # the last column is the current token's
    assert O.causal_conv(x, taps).reshape(-1).tolist() == [1.0, 12.0, 124.0, 248.0]
    assert O.causal_conv(x, taps, torch.tensor([0.5], dtype=D64))[0].item() == 1.5


def test_masks_at_their_edges():
    assert O.visible(39, 0, "window", 40) and not O.visible(40, 0, "window", 40) and O.visible(40, 1, "window", 40)
    assert O.visible(23, 0, "chunk", 24) and not O.visible(24, 23, "chunk", 24) and O.visible(24, 24, "chunk", 24)
    assert not O.visible(3, 4, "window", 40) and not O.visible(3, 4, "chunk", 24)


def test_bonus_reaches_only_the_current_token_and_the_read_comes_before_the_update():
    r = torch.ones(3, 1, 1, dtype=D64)
    k = torch.ones(3, 1, 1, dtype=D64)
    v = torch.tensor([1.0, 10.0, 100.0], dtype=D64).reshape(3, 1, 1)
    w = torch.full((3, 1, 1), 0.5, dtype=D64)
    u = torch.tensor([[3.0]], dtype=D64)
    out = O.wkv_sum(r, k, v, w, u).reshape(-1).tolist()
    # o_0 = 3*1; S = 1; o_1 = 1 + 3*10; S = 0.5 + 10; o_2 = 10.5 + 3*100
    assert out == [3.0, 31.0, 310.5]


def test_sink_takes_weight_without_giving_a_value_and_sigmoid_weights_do_not_sum_to_one():
    q = torch.zeros(2, 1, 2, dtype=D64)
    k = torch.zeros(2, 1, 2, dtype=D64)
    v = torch.tensor([[[2.0]], [[4.0]]], dtype=D64)
    out = O.sink_softmax_attention(q, k, v, torch.tensor([0.0], dtype=D64), scale=1.0, kind="window", size=8)
    assert torch.allclose(out.reshape(-1), torch.tensor([1.0, 2.0], dtype=D64))            # 2/2, (2+4)/3
    big = O.sink_softmax_attention(q, k, v, torch.tensor([math.log(8.0)], dtype=D64), scale=1.0, kind="window", size=8)
    assert torch.allclose(big.reshape(-1), torch.tensor([2.0 / 9, 6.0 / 10], dtype=D64))
    out = O.sigmoid_attention(q, k, v, torch.tensor([0.0], dtype=D64), scale=1.0, kind="chunk", size=8)
    assert torch.allclose(out.reshape(-1), torch.tensor([1.0, 3.0], dtype=D64))            # every key weighs one half
    out = O.sigmoid_attention(q, k, v, torch.tensor([0.0], dtype=D64), scale=1.0, kind="chunk", size=1)
    assert torch.allclose(out.reshape(-1), torch.tensor([1.0, 2.0], dtype=D64))            # position 1 starts a new chunk


def test_state_space_step_decays_by_the_step_size_and_adds_the_skip():
    x = torch.tensor([1.0, 0.0, 0.0], dtype=D64).reshape(3, 1, 1)
    B = torch.ones(3, 1, 1, dtype=D64)
    C = torch.ones(3, 1, 1, dtype=D64)
    dt = torch.full((3, 1), 0.5, dtype=D64)
    out = O.state_space_sum(x, B, C, dt, torch.tensor([2.0], dtype=D64), torch.tensor([7.0], dtype=D64)).reshape(-1)
    d = math.exp(-2.0 * 0.5)
    assert torch.allclose(out, torch.tensor([0.5 + 7.0, 0.5 * d, 0.5 * d * d], dtype=D64))


def test_clamped_feed_forward_limits_gate_from_above_and_the_other_half_on_both_sides():
    w = {"p.gate": torch.tensor([[1.0]], dtype=D64), "p.gate.b": torch.zeros(1, dtype=D64), "p.up": torch.tensor([[1.0]], dtype=D64),
         "p.up.b": torch.zeros(1, dtype=D64), "p.down": torch.tensor([[1.0]], dtype=D64), "p.down.b": torch.tensor([0.25], dtype=D64)}
    h = torch.tensor([[10.0], [-10.0], [1.0]], dtype=D64)
    out = O.clamped_ff(h, w, "p.", 2.0).reshape(-1)
    sig = lambda z: 1 / (1 + math.exp(-z))
    want = [2 * sig(1.702 * 2) * 3 + 0.25, -10 * sig(-17.02) * (-2 + 1) + 0.25, sig(1.702) * 2 + 0.25]
    assert torch.allclose(out, torch.tensor(want, dtype=D64))


def test_plain_model_runs_every_mixer_and_is_causal():
    config = norusun_config(pattern="LdPdWn", width=64, wkv_heads=2, wkv_dim=32, vocab=50, ff=48)
    tensors = synthetic_norusun(config, seed=1)
    ids = torch.randint(0, 50, (30,), generator=torch.Generator().manual_seed(2)).tolist()
    tap = []
    full = O.forward(ids, tensors, config, tap=tap)
    assert full.shape == (30, 50) and len(tap) == 3 and torch.isfinite(full).all()
    assert torch.allclose(O.forward(ids[:17], tensors, config), full[:17], atol=1e-9)
