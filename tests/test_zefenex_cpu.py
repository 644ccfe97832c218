"""Host-side checks of the Zefenex model class (no GPU): the registry, the configuration reader, and the oracle's own mechanisms."""
import importlib

import pytest
import torch

import zefenex_oracle as ref
from util import b200


def test_registry_names_the_design():
    models = importlib.import_module("llm-inference-engine_b200.models")
    assert "zefenex" in models.architectures()
    assert models.architecture_of({"architecture": "Zefenex"}) == "Zefenex"


def test_layer_specs_follow_the_configuration():
    m = b200()
    z = importlib.import_module("llm-inference-engine_b200.models.zefenex")
    config = ref.make_config([ref.latent_layer(heads=3, dim=10, rot_dim=6, rot_dims=4, vdim=7, kv_rank=9, window=11, scale=0.5, base=77.0, mlp=ref.dense(ff=13)),
                              ref.latent_layer(kv_from=0, mlp=ref.moe(experts=4, identity=2, top=3, ff=5, shared_ff=0)), ref.latent_layer()])
    a, b, c = z.layer_specs(config)
    assert (a["mixer"], a["norm"], a["heads"], a["dim"], a["rot_dim"], a["rot_dims"], a["vdim"], a["kv_rank"], a["window"], a["kv_from"]) == \
        (m.MIXER_LATENT, m.NORM_DYT_PRE_POST, 3, 10, 6, 4, 7, 9, 11, -1)
    assert a["scale"] == 0.5 and a["rot_base"] == 77.0 and (a["mlp"], a["expert_ff"], a["act"], a["gated"]) == (m.MLP_DENSE, 13, m.ACT_RELU2, 0)
    assert (b["kv_from"], b["mlp"], b["route"], b["experts"], b["identity"], b["top"], b["expert_ff"], b["shared_ff"], b["act"], b["gated"]) == \
        (0, m.MLP_MOE, m.ROUTE_SOFTMAX, 4, 2, 3, 5, 0, m.ACT_SILU, 1)
    assert c["mlp"] == m.MLP_NONE
    with pytest.raises(ValueError):
        z.layer_specs(ref.make_config([{"type": "conv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}]))
    with pytest.raises(ValueError):
        z.layer_specs(ref.make_config([ref.latent_layer(kv_from=0)]))   # a layer cannot borrow from itself
    with pytest.raises(ValueError):
        z.layer_specs(ref.make_config([ref.latent_layer(mlp={"kind": "glu"})]))


def test_oracle_window_and_rotation():
    see = ref.visible(6, 3)
    assert see[5].tolist() == [False, False, False, True, True, True] and see[1].tolist() == [True, True, False, False, False, False]
    assert ref.visible(4, 0)[3].all()
    v = torch.arange(12, dtype=torch.float64).view(2, 6) + 1
    out = ref.rotate(v, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(out[0], v[0])                       # position 0 turns nothing
    assert torch.equal(out[1, 4:], v[1, 4:])               # past `dims`: unchanged
    assert torch.allclose(out[1, :4].norm(), v[1, :4].norm())
    c, s = torch.cos(torch.tensor(3.0, dtype=torch.float64)), torch.sin(torch.tensor(3.0, dtype=torch.float64))
    assert torch.allclose(out[1, 0], v[1, 0] * c - v[1, 2] * s) and torch.allclose(out[1, 2], v[1, 2] * c + v[1, 0] * s)


def test_oracle_router_weights_sum_to_one_and_identity_returns_its_input():
    config = ref.make_config([ref.latent_layer(mlp=ref.moe(experts=1, identity=1, top=2, shared_ff=0))])
    W, _ = ref.make_weights(config, seed=2)
    h = torch.randn(9, config["width"], dtype=torch.float64)
    chosen, weight = ref.route(h, W, "l0.mlp.", config["layers"][0]["mlp"])
    assert torch.allclose(weight.sum(-1), torch.ones(9, dtype=torch.float64))
    y = ref.feed_forward_moe(h, W, "l0.mlp.", config["layers"][0]["mlp"])
    w_id = torch.where(chosen == 1, weight, torch.zeros_like(weight)).sum(-1, keepdim=True)
    assert torch.allclose(y, w_id * h + (1 - w_id) * ref.gated_expert(h, W, "l0.mlp.e0."))
