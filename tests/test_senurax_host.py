"""Senurax without a GPU: the order of layer runs, the configuration generator and registry, a checkpoint round trip,
and the plain restatement's mechanisms (oracle/senurax.py) on cases with closed forms."""

import math

import pytest
import torch

from oracle import senurax as O
from tiny_llm_b200.models import ARCHITECTURES
from tiny_llm_b200.synthetic import save_senurax, senurax_config, synthetic_senurax


def test_registry_names_the_design():
    assert ARCHITECTURES["Senurax"] == ("tiny_llm_b200.senurax", "SenuraxModel")


def test_layer_runs_repeat_the_looped_layers_and_mark_the_first_of_each_pass():
    config = senurax_config(pattern="RdCmCdPm", loop=(1, 3, 2))
    assert O.layer_runs(config) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False)]
    assert O.layer_runs(senurax_config(pattern="RdCm", loop=None)) == [(0, None, False), (1, None, False)]
    assert O.layer_runs(senurax_config(pattern="RdCm", loop=(0, 2, 1))) == [(0, 0, True), (1, 0, False)]


def test_product_and_oracle_agree_on_the_order_of_runs():
    import ast
    from pathlib import Path

    # the product's function is pure host code; load it without importing the GPU extension
    source = (Path(__file__).resolve().parent.parent / "tiny-llm_b200" / "tiny_llm_b200" / "senurax.py").read_text()
    fn = next(n for n in ast.parse(source).body if isinstance(n, ast.FunctionDef) and n.name == "layer_runs")
    scope: dict = {}
    exec(compile(ast.Module([fn], []), "layer_runs", "exec"), scope)
    for loop in (None, (0, 1, 3), (1, 4, 2), (2, 5, 1), (0, 5, 2)):
        config = senurax_config(pattern="RdCmCdPmRn", loop=loop)
        assert scope["layer_runs"](5, config.get("loop")) == O.layer_runs(config)
    with pytest.raises(ValueError):
        scope["layer_runs"](3, {"start": 2, "stop": 5, "times": 2})


def test_generator_spells_layers_and_weights_round_trip(tmp_path):
    config = senurax_config(pattern="PnRdCm", loop=None, rot_factor=1.0, softcap=None, identity=0)
    assert [l["type"] for l in config["layers"]] == ["parallel", "retention", "channel_delta"]
    assert config["layers"][0]["mlp"] is None and "loop" not in config and "logit_softcap" not in config
    assert "scaling" not in config["layers"][0]["mixer"]["left"]["rot"]
    tensors = synthetic_senurax(config, seed=3)
    assert "l0.norm2" not in tensors and tensors["l2.mlp.router"].shape[0] == config["layers"][2]["mlp"]["router"]["experts"]
    save_senurax(config, tensors, tmp_path / "m")
    from tiny_llm_b200.checkpoint import read_tensors

    back = read_tensors(tmp_path / "m")
    assert set(back) == set(tensors) and all(torch.equal(back[k], tensors[k]) for k in tensors)
    logits = O.forward([1, 2, 3, 4], tensors, config)
    assert logits.shape == (4, config["vocab"]) and torch.isfinite(logits).all()
    assert torch.allclose(O.forward([1, 2, 3, 4, 5], tensors, config)[:4], logits)  # causal


def test_short_convolution_is_causal_and_starts_from_zeros():
    x = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    taps = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)  # the last column multiplies the current token
    y = O.short_conv_silu(x, taps)
    pre = torch.tensor([2.0, 4.0 - 1.0, 6.0 - 2.0 + 0.5])
    assert torch.allclose(y[:, 0], (pre * torch.sigmoid(pre)).double())


def test_rotation_depends_on_the_distance_only_and_leaves_the_rest():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 12, generator=g, dtype=torch.float64), torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    for layout in ("half", "interleaved"):
        scores = []
        for at in (0, 5):
            qs, ks = torch.zeros(at + 4, 1, 12, dtype=torch.float64), torch.zeros(at + 4, 1, 12, dtype=torch.float64)
            qs[at + 3], ks[at] = q[0], k[0]
            qr, kr = (O.rotate(t, dims=8, base=100.0, factor=2.0, layout=layout) for t in (qs, ks))
            scores.append(float(qr[at + 3, 0] @ kr[at, 0]))
            assert torch.equal(qr[at + 3, 0, 8:], q[0, 0, 8:])
        assert abs(scores[0] - scores[1]) < 1e-12
    one = O.rotate(torch.tensor([[[1.0, 0.0]]] * 3, dtype=torch.float64), dims=2, base=10.0, factor=4.0, layout="half")
    assert torch.allclose(one[2, 0], torch.tensor([math.cos(0.5), math.sin(0.5)], dtype=torch.float64))


def test_delta_rule_replaces_a_value_and_retention_sums_with_decay():
    e = torch.eye(4, dtype=torch.float64)
    k = torch.stack([e[0], e[1], e[0]])[:, None]
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)[:, None]
    out = O.delta_rule(k, k, v, torch.ones(3, 1, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(out[:, 0], v[:, 0])  # the third token reads its own write, not 1 + 5
    half = O.delta_rule(k, k, v, torch.full((3, 1), 0.5, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(half[2, 0], 0.5 * v[0, 0] + 0.5 * (v[2, 0] - 0.5 * v[0, 0]))
    kept = O.retained_sum(k, k, v, [0.5])
    assert torch.allclose(kept[2, 0], 0.25 * v[0, 0] + v[2, 0])


def test_router_chooses_by_corrected_scores_and_weighs_by_plain_ones():
    h = torch.eye(3, dtype=torch.float64)[:1]
    w = {"router": torch.tensor([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0], [0.0, 0, 0]], dtype=torch.float64),
         "correction": torch.tensor([0.0, 0.0, 1.0, 0.0], dtype=torch.float64)}
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0, 0.0], dtype=torch.float64), 0)
    chosen, weight = O.route(h, w, "", {"top": 2, "scale": 3.0})
    assert chosen.tolist() == [[2, 0]]
    assert torch.allclose(weight[0], 3.0 * torch.stack([s[2], s[0]]) / (s[2] + s[0]))
    # output 2 and 3 are identity experts of a mixture with two real ones
    for e in range(2):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = torch.ones(2, 3, dtype=torch.float64), torch.ones(2, 3, dtype=torch.float64), torch.ones(3, 2, dtype=torch.float64)
    y = O.expert_mixture(h, w, "", {"router": {"experts": 2, "identity": 2, "top": 2, "scale": 3.0}})
    expert = (O.silu(torch.tensor(1.0, dtype=torch.float64)) * 1.0) * 2 * torch.ones(3, dtype=torch.float64)
    assert torch.allclose(y[0], weight[0, 0] * h[0] + weight[0, 1] * expert)
