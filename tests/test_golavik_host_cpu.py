"""Host side of the Golavik path without a GPU: configuration reading and validation, the order of layer runs under a
loop, the registry, the rotary frequency table against the restatement's."""
import json

import pytest
import torch

import golavik_oracle as go


def _cfg(loop=None, layers=None):
    moe = {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 2, "scale": 1.0,
                                                           "groups": {"count": 2, "keep": 1}}}
    layers = layers or [
        {"type": "general_delta", "mixer": {"heads": 2, "dim": 4}, "mlp": None},
        {"type": "latent_attention", "mlp": moe,
         "mixer": {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 6, "kv_rank": 5, "scale": 0.3, "mask": {"size": 3},
                   "rot": {"base": 100.0, "dims": 4}}},
        {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "conv": 2}, "mlp": moe}]
    return {"architecture": "Golavik", "vocab": 11, "width": 12, "norm": {"eps": 1e-5, "groups": 3},
            "canon": {"taps": 2}, "loop": loop, "layers": layers}


def test_config_round_trip_and_layer_runs():
    from llark_b200.models.golavik import GolavikConfig

    c = GolavikConfig.from_dict(_cfg({"start": 1, "stop": 3, "times": 2}))
    assert (c.vocab, c.width, c.groups, c.taps, c.eps) == (11, 12, 3, 2, 1e-5)
    assert c.layer_runs() == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False)]
    assert [(i, t, f) for i, t, f in go.layer_runs(_cfg({"start": 1, "stop": 3, "times": 2}))] == c.layer_runs()
    assert GolavikConfig.from_dict(json.loads(json.dumps(c.to_dict()))).to_dict() == c.to_dict()
    assert GolavikConfig.from_dict(_cfg(None)).layer_runs() == [(0, None, False), (1, None, False), (2, None, False)]
    one = GolavikConfig.from_dict(_cfg({"start": 0, "stop": 3, "times": 1}))
    assert one.layer_runs() == [(0, 0, True), (1, 0, False), (2, 0, False)]
    assert GolavikConfig.from_dict(_cfg({"start": 2, "stop": 2, "times": 5})).loop is None


@pytest.mark.parametrize("bad", [
    lambda d: d.update(architecture="Other"),
    lambda d: d["layers"][0].update(type="hgrn2"),
    lambda d: d["layers"][1]["mlp"].update(kind="dense"),
    lambda d: d["norm"].update(groups=5),
    lambda d: d.update(loop={"start": 2, "stop": 1, "times": 2}),
    lambda d: d.update(loop={"start": 0, "stop": 4, "times": 2}),
    lambda d: d.update(loop={"start": 0, "stop": 2, "times": 0}),
])
def test_config_validation(bad):
    from llark_b200.models.golavik import GolavikConfig

    d = json.loads(json.dumps(_cfg()))
    bad(d)
    with pytest.raises(ValueError):
        GolavikConfig.from_dict(d)


def test_registry_names_the_class():
    from llark_b200.models.registry import model_class_for

    assert model_class_for({"architecture": "Golavik"}).__name__ == "GolavikForCausalLM"
    assert model_class_for({"architecture": "Kelutar"}).__name__ == "KelutarForCausalLM"
    with pytest.raises(ValueError):
        model_class_for({"architecture": "Nothing"})


def test_mixer_tables():
    from llark_b200.mixers import FEED_FORWARDS, MIXERS

    assert {"latent_attention", "channel_delta", "general_delta", "attention", "hgrn2"} <= set(MIXERS)
    assert hasattr(FEED_FORWARDS["moe"], "residual")


def test_rotary_frequencies_match_the_restatement():
    from llark_b200.mixers import rotary_frequencies

    for dims, base, sc in ((2, 10.0, None), (8, 100.0, None),
                           (32, 5e5, {"factor": 6.0, "original": 2048, "fast": 16.0, "slow": 2.0}),
                           (24, 500.0, {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}),
                           (64, 10000.0, {"factor": 40.0, "original": 4096, "fast": 32, "slow": 1})):
        f, m = rotary_frequencies(dims, base, sc)
        f2, m2 = go.yarn_frequencies(dims, base, sc)
        assert f.shape == (dims // 2,) and torch.allclose(f, f2, rtol=1e-12) and abs(m - m2) < 1e-12
    f, _ = rotary_frequencies(8, 100.0, {"factor": 2.0, "original": 64, "fast": 1e9, "slow": 1e-9})  # ramp covers all
    plain, _ = rotary_frequencies(8, 100.0)
    assert (f <= plain + 1e-15).all() and (f >= plain / 2.0 - 1e-15).all()
