"""Goletar on the CPU: configuration, registry, checkpoint adapter and the one error for a checkpoint that does not
fit; and the plain restatement against itself (a recurrence carried over a cut, the softmax's sink, the experts'
limits)."""
import json
import os

import pytest
import torch

import goletar_models as gm
import plain_goletar as pg


def test_config_json_round_trip_and_registry(tmp_path):
    from fms_b200 import models
    from fms_b200.models import get_model
    from fms_b200.models.goletar import Goletar

    assert "goletar" in models.list_models() and "tiny" in models.list_variants("goletar")
    cfg = gm.CONFIGS["p"]
    folder = gm.write_folder(str(tmp_path / "p"), cfg, gm.tensors(cfg, 1))
    model = get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")  # found by "architecture"
    assert isinstance(model, Goletar) and model.config_json() == cfg
    spec = model.decoder_spec()
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "mingru", "latent_attention", "mingru"]
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.kind == "routed_experts"
    assert dict(spec.layers[0].mixer.options)["rot_dims"] == 4 and spec.embedding.kind == "pair_hash"
    sd = model.state_dict()
    assert sd["layers.0.mlp.gate_up"].shape == (5, 40, 48) and sd["layers.1.mix.zxg_fused.weight"].shape == (120, 48)
    assert sd["layers.1.mix.zxg_fused.bias"][80:].abs().max() == 0 and sd["layers.0.norm1.weight"].shape == ()
    assert "layers.1.norm2.weight" not in sd
    requests = model.decoder.cache_requests()
    assert requests[0].planes == 1 and requests[0].head_dim == 24 + 8 and requests[1].shape == (40,)
    assert model.decoder.named_cache_requests()["embedding"].dtype == torch.int32
    assert model.cache_bytes_per_token() == 2 * (24 + 8) * 4


def test_a_checkpoint_that_does_not_fit_is_refused_with_one_error(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    cfg = gm.CONFIGS["q"]
    weights = gm.tensors(cfg, 2)
    del weights["l1.mlp.e3.up"], weights["l2.mix.sink"]
    weights["l0.mix.o"] = weights["l0.mix.o"][:, :-1]
    weights["stray"] = torch.zeros(3, dtype=torch.bfloat16)
    folder = gm.write_folder(str(tmp_path / "q"), cfg, weights)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    assert "layers.2.mix.sink" in e.value.missing and "layers.1.mlp.gate_up" in e.value.missing
    assert "stray" in e.value.unexpected and any(n == "layers.0.mix.dense.weight" for n, _, _ in e.value.wrong_shapes)


def test_config_json_of_another_design_or_with_unknown_layers_is_refused():
    from fms_b200.models.goletar import Goletar

    with pytest.raises(ValueError):
        Goletar.config_from_json({"architecture": "Other"})
    bad = json.loads(json.dumps(gm.CONFIGS["r"]))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError, match="convolution"):
        Goletar.config_from_json(bad)


def test_random_weights_of_a_registered_variant():
    from fms_b200.models import get_model

    model = get_model("goletar", "tiny", device_type="cpu", data_type="fp32", seed=4)
    names = {t.name for t in model.checkpoint_layout()}
    assert {"embed", "bigram", "final.norm", "head", "l0.mix.z.b", "l1.mix.dkv.norm", "l1.mlp.e3.down"} <= names


def test_plain_recurrence_carried_over_a_cut_and_plain_sink():
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    wz, bz, wx, bx, wg, wo = r(6, 5), r(6), r(6, 5), r(6), r(6, 5), r(5, 6)
    h = r(9, 5)
    whole = pg.mingru(h, wz, bz, wx, bx, wg, wo)
    # the state after four tokens, taken from the recurrence itself, carries the rest
    z, u = torch.sigmoid(h @ wz.T + bz), h @ wx.T + bx
    s = torch.zeros(6, dtype=torch.float64)
    for t in range(4):
        s = (1 - z[t]) * s + z[t] * torch.where(u[t] >= 0, u[t] + 0.5, torch.sigmoid(u[t]))
    torch.testing.assert_close(pg.mingru(h[4:], wz, bz, wx, bx, wg, wo, state=s), whole[4:])
    m = gm.latent(2, 4, 4, 3, 6, 10.0, None)["mixer"]
    args = (r(16, 5), r(10, 5), r(6), r(8, 6), r(6, 6))
    sink = torch.tensor([30.0, -30.0], dtype=torch.float64)
    _, p = pg.latent_attention(h, m, 1e-5, *args, sink, r(2, 5), r(5, 6))
    assert p[0].sum(-1).max() < 1e-6 and (p[1].sum(-1) - 1).abs().max() < 1e-9


def test_plain_experts_limits_and_weights_on_the_input():
    router = torch.tensor([[4.0, 0.0], [0.0, 4.0], [-9.0, -9.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.5]], dtype=torch.float64)
    out, chosen = pg.routed_experts(h, router, [eye * 10] * 3, [eye * 10] * 3, [eye] * 3, 2, 1.25)
    assert chosen == [[0, 1]]
    # both products pass the limit whatever the (positive) weight: g = 1.25, u = 1.25 for every value
    one = 1.25 / (1 + torch.exp(torch.tensor(-1.702 * 1.25, dtype=torch.float64))) * 2.25
    torch.testing.assert_close(out, torch.full((1, 2), 2 * one.item(), dtype=torch.float64))
