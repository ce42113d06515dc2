"""Lanizen's configuration on the CPU: every size comes from config.json, branches the design names are data in the
model's description, and what does not fit is refused by name."""
import copy
import json

import pytest
import torch

import citlali_b200 as cb
import plain_lanizen as plain
from citlali_b200.engine.model import cache_requirements_of
from lanizen_models import CONFIGS, config, make_weights


def test_round_trip_and_registry(tmp_path):
    for name, d in CONFIGS.items():
        c = config(name)
        (tmp_path / name).mkdir()
        (tmp_path / name / "config.json").write_text(json.dumps(c.to_dict()))
        assert cb.config_from_model_dir(str(tmp_path / name)) == c
        assert c.vocab == d["vocab"] and c.width == d["width"] and c.streams == d.get("streams")


def test_spec_is_data():
    spec = config("P").to_model_spec()
    assert spec.residual_streams == 2 and spec.embedding_scale == 2.0 and spec.tie_head_to_embedding is False
    assert [l.block for l in spec.layers] == ["hyper_connection"] * 4
    assert [l.part("mixer").kind for l in spec.layers] == ["gated_delta", "latent_attention"] * 2
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[0].part("feed_forward").kind == "relu_squared"
    assert [(s.layer, s.cache_of) for s in spec.schedule] == [(0, None), (1, None), (2, None), (3, 1)]
    owner, reader = spec.layers[1].part("mixer").params, spec.layers[3].part("mixer").params
    assert owner["window"] == 9 and owner["cache_window"] == 20 and reader["window"] == 20 and not reader["kv_projection"]
    reqs = cache_requirements_of(spec)
    assert reqs[1] == cb.KVRequirement(1, 48, 20, value_dim=0) and reqs[3] is None
    assert reqs[0] == cb.StateRequirement((4 * 16 * 24 + 3 * (2 * 2 * 16 + 4 * 24),), torch.float32)
    plain_spec = config("Q").to_model_spec()
    assert plain_spec.residual_streams is None and plain_spec.layers[0].block == "pre_norm_residual"
    assert plain_spec.layers[0].part("mixer").params["window"] is None
    assert plain_spec.layers[0].part("mixer").params["rot_dims"] == 8
    names = {t.name for t in cb.expected_tensors(plain_spec)}
    assert "l0.mix.dkv" in names and "l0.hc1.in" not in names and "l2.norm2" not in names


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][0].update(type="conv"), "type 'conv' is unknown"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=41), "kv_rank differs"),
    (lambda d: d["layers"][1]["mlp"].update(kind="gated"), "mlp.kind"),
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d.update(streams=0), "streams"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
])
def test_rejections_name_the_key(change, message):
    d = copy.deepcopy(CONFIGS["P"])
    change(d)
    with pytest.raises(cb.CitlaliError, match=message):
        cb.config_from_dict(d)


def test_plain_identities():
    """The plain implementation against elementary facts: one stream with unit mixtures is the residual sum; a window of
    the whole length is no window; a sink far below every score is a plain softmax; the delta rule with beta = 1 and
    g = 1 stores v under k exactly."""
    d = copy.deepcopy(CONFIGS["S"])
    cfg = cb.config_from_dict(d)
    w = {k: v.float() for k, v in make_weights(cfg, 3).items()}
    for n in list(w):
        if ".hc" in n:
            w[n] = torch.ones_like(w[n])
    toks = [5, 9, 77, 3, 100, 8]
    a = plain.forward(cfg.to_dict(), w, toks)
    no_streams = {k: v for k, v in cfg.to_dict().items() if k != "streams"}
    assert torch.allclose(a, plain.forward(no_streams, w, toks), atol=1e-12)
    wide = copy.deepcopy(cfg.to_dict())
    wide["layers"][1]["mixer"]["mask"]["size"] = 4
    unmasked = copy.deepcopy(wide)
    del unmasked["layers"][1]["mixer"]["mask"]
    assert torch.allclose(plain.forward(wide, w, toks[:4]), plain.forward(unmasked, w, toks[:4]), atol=1e-12)
    assert not torch.allclose(plain.forward(wide, w, toks)[5], plain.forward(unmasked, w, toks)[5], atol=1e-6)
    scores = torch.randn(4, 4, dtype=torch.float64)
    vis = torch.tril(torch.ones(4, 4, dtype=torch.bool))
    p = plain.sink_softmax_attention(scores, vis, torch.tensor(-200.0, dtype=torch.float64))
    assert torch.allclose(p, torch.softmax(scores.masked_fill(~vis, float("-inf")), -1), atol=1e-12)
    assert float(plain.sink_softmax_attention(scores, vis, torch.tensor(50.0, dtype=torch.float64)).abs().max()) < 1e-15
    k = torch.nn.functional.normalize(torch.randn(1, 8, dtype=torch.float64), dim=-1)
    v = torch.randn(1, 5, dtype=torch.float64)
    o = plain.delta_rule(k, k, v, torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64))
    assert torch.allclose(o, v, atol=1e-12)
