"""Niletar on the CPU: configuration, registry, checkpoint adapter, layers that share weights, the cache's entries for
mixers that ask for several things, and the one error for a checkpoint that does not fit; and the plain restatement
against itself (recurrences carried over a cut, the softmax's sink, the scaled frequencies)."""
import json
import math

import pytest
import torch

import niletar_models as nm
import plain_niletar as pn


def test_config_json_round_trip_registry_and_shared_layers(tmp_path):
    from fms_b200 import models
    from fms_b200.cache.requests import KVRequest, StateRequest
    from fms_b200.models import get_model
    from fms_b200.models.niletar import Niletar

    assert "niletar" in models.list_models() and "tiny" in models.list_variants("niletar")
    cfg = nm.CONFIGS["p"]
    folder = nm.write_folder(str(tmp_path / "p"), cfg, nm.tensors(cfg, nm.RANKS["p"], 1))
    model = get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")  # found by "architecture"
    assert isinstance(model, Niletar)
    spec = model.decoder_spec()
    assert [b.mixer.kind for b in spec.layers] == ["selective_state_space", "parallel", "parallel", "selective_state_space"]
    assert [b.weights_of for b in spec.layers] == [None, None, 1, 0] and all(b.arrangement == "post_norm" for b in spec.layers)
    assert dict(spec.layers[0].options)["alpha"] == 2.5
    right = dict(dict(spec.layers[1].mixer.options)["right"].options)
    assert (right["decay_rank"], right["gate_rank"]) == nm.RANKS["p"]  # read from the checkpoint's shapes
    blocks = model.decoder.blocks
    assert blocks[2] is blocks[1] and blocks[3] is blocks[0] and blocks[0] is not blocks[1]
    sd = model.state_dict()
    assert not any(k.startswith(("layers.2.", "layers.3.")) for k in sd)
    assert sd["layers.1.mix.left.in_proj.weight"].shape == (4 * 24 + 24 + 8 + 4 * 8, 48)
    assert sd["layers.1.mix.left.in_proj.bias"][-32:].abs().max() == 0
    assert sd["layers.1.mix.right.in_proj.weight"].shape == (2 * 12 + 2 * 12 + 4 * 20 + 4, 48)
    assert sd["layers.1.mix.right.conv"].shape == (2 * 12 + 2 * 12 + 4 * 20, 2)
    assert sd["layers.0.mlp.wg1_fused.weight"].shape == (80, 48)
    # every layer has cache entries of its own, also those that share weights
    requests = model.decoder.cache_requests()
    assert len(requests) == 4 and all(isinstance(r, tuple) for r in requests)
    kv, matrix, tail = requests[1]
    assert isinstance(kv, KVRequest) and kv.head_dim == 32 and kv.kvheads == 1  # heads of 24 and 8, padded to 32
    assert isinstance(matrix, StateRequest) and matrix.shape == (4, 20, 12) and tail.shape == (1, 2 * 12 + 2 * 12 + 4 * 20)
    assert requests[0][0].shape == (3, 8, 5) and requests[0][1].shape == (2, 3 * 8 + 2 * 5)
    assert model.cache_bytes_per_token() == 2 * (2 * 1 * 32 * 4)  # two attention layers, keys and values, float32
    out = json.loads(json.dumps(model.config_json()))
    for layer in out["layers"]:  # what the loader read from the shapes is the only thing added
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank", None), layer["mixer"]["right"].pop("gate_rank", None)
    assert out == cfg


def test_cache_entries_of_a_layer_that_asks_for_several_things():
    from fms_b200.cache import Cache
    from fms_b200.cache.requests import KVRequest, StateRequest

    kv, a, b = KVRequest(2, 16), StateRequest((3, 4), torch.float32, "m"), StateRequest((2, 5), torch.float32, "t")
    cache = Cache([(kv, a, b), (a, b), None, (kv, a, b)], 256, 256, torch.float32, "cpu", max_slots=3)
    v0, v1, v3 = cache.layer_view(0), cache.layer_view(1), cache.layer_view(3)
    assert cache.layer_view(2) is None and len(v0) == 3 and len(v1) == 2
    assert v0[0].keys.shape[-1] == 16 and v0[1].state.shape == (4, 3, 4) and v1[1].state.shape == (4, 2, 5)
    # equal requests share a group, every layer has rows of its own in it
    v0[1].state.fill_(1.0), v3[1].state.fill_(3.0)
    assert float(v1[0].state.sum()) == 0 and float(cache.layer_view(0)[1].state.mean()) == 1.0
    (slot,) = cache.begin(1)
    assert float(cache.layer_view(3)[1].state[slot].sum()) == 0 and float(cache.layer_view(3)[1].state.sum()) > 0


def test_a_checkpoint_that_does_not_fit_is_refused_with_one_error(tmp_path):
    from fms_b200.models import get_model
    from fms_b200.weights import WeightError

    cfg = nm.CONFIGS["q"]
    weights = nm.tensors(cfg, nm.RANKS["q"], 2)
    del weights["l0.mix.left.sink"], weights["l2.mix.right.k.conv"]
    weights["l1.mix.o"] = weights["l1.mix.o"][:, :-1]
    weights["stray"] = torch.zeros(3, dtype=torch.bfloat16)
    folder = nm.write_folder(str(tmp_path / "q"), cfg, weights)
    with pytest.raises(WeightError) as e:
        get_model("hf_pretrained", model_path=folder, device_type="cpu", data_type="fp32")
    assert "layers.0.mix.left.sink" in e.value.missing and "layers.2.mix.right.conv" in e.value.missing
    assert "stray" in e.value.unexpected and any(n == "layers.1.mix.dense.weight" for n, _, _ in e.value.wrong_shapes)


def test_config_json_of_another_design_or_with_unknown_layers_is_refused():
    from fms_b200.models.niletar import Niletar

    with pytest.raises(ValueError):
        Niletar.config_from_json({"architecture": "Other"})
    bad = json.loads(json.dumps(nm.CONFIGS["r"]))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError, match="convolution"):
        Niletar.config_from_json(bad)
    chained = json.loads(json.dumps(nm.CONFIGS["p"]))
    chained["layers"].append(dict(chained["layers"][2], weights_of=2))  # the weights of a layer that takes another's
    spec = Niletar(Niletar.config_from_json(chained)).decoder_spec()
    assert [b.weights_of for b in spec.layers] == [None, None, 1, 0, 1]
    bad = json.loads(json.dumps(nm.CONFIGS["p"]))
    bad["layers"][2]["weights_of"] = 0  # a layer of another type
    with pytest.raises(ValueError, match="weights_of"):
        Niletar.config_from_json(bad)


def test_random_weights_of_a_registered_variant():
    from fms_b200.models import get_model

    model = get_model("niletar", "tiny", device_type="cpu", data_type="fp32", seed=4)
    names = {t.name for t in model.checkpoint_layout()}
    assert {"embed", "final.norm", "head", "l0.mix.left.q.b", "l0.mix.right.a2", "l1.mix.conv.b", "l1.mlp.down"} <= names
    assert float(model.state_dict()["layers.0.norm1.weight"].abs().max()) <= 0.1  # stored around zero


def test_plain_recurrences_carried_over_a_cut():
    """The restatement's scans restarted from the middle with the state and the convolution's inputs of the first half
    give the second half: what a step function must carry is exactly that."""
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, w, b = r(11, 6), r(6, 3), r(6)
    whole = pn.causal_conv(x, w, b)
    torch.testing.assert_close(pn.causal_conv(x[5:], w, b, before=x[3:5]), whole[5:])
    torch.testing.assert_close(whole[0], x[0] * w[:, 2] + b)  # zeros before the start; the last column is the current row's


def test_plain_sink_and_scaled_frequencies():
    g = torch.Generator().manual_seed(1)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    m = nm.left(2, 1, 4, 3, 2, 10.0, 0.5)
    t = {"q": r(8, 5), "q.b": r(8), "k": r(4, 5), "k.b": r(4), "v": r(3, 5), "v.b": r(3), "g": torch.zeros(6, 5, dtype=torch.float64),
         "o": torch.eye(6, dtype=torch.float64), "sink": torch.tensor([40.0, -40.0], dtype=torch.float64)}
    h = r(7, 5)
    out = pn.sink_attention(h, m, 1e-5, t, "")
    v = h @ t["v"].T + t["v.b"]
    assert out[:, :3].abs().max() < 1e-12  # the sink took everything
    torch.testing.assert_close(out[0, 3:], 0.5 * v[0])  # the first token sees itself only; the gate is sigmoid(0)
    f = pn.rotary_frequencies(8, 10000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 100})
    plain = [10000.0 ** (-2 * i / 8) for i in range(4)]
    assert f[0] == plain[0] and f[3] == plain[3] / 4  # short waves stay, long ones are slowed
    wl = 2 * math.pi / plain[1]  # the second lies between the two: 100 / 4 < 62.8 < 100
    s = (100 / wl - 1.0) / 3.0
    assert abs(f[1] - ((1 - s) * plain[1] / 4 + s * plain[1])) < 1e-15
