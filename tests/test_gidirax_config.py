"""The Gidirax configuration on the CPU: read, written back, described as data; rejections name the key; sizes that only
tensor shapes give; the cache's bookkeeping for windows with kept first tokens and for mixers with several caches; and the
plain implementation against elementary identities."""
import json

import pytest
import torch

import citlali_b200 as cb
import plain_gidirax as plain
from citlali_b200.cache import KVRequirement, SequenceCache, StateRequirement
from gidirax_models import CONFIGS, config, make_weights


def test_round_trip_and_spec_as_data():
    for name, d in CONFIGS.items():
        cfg = config(name)
        assert cb.config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
        spec = cfg.to_model_spec()
        assert spec.architecture == "Gidirax" and spec.tie_head_to_embedding is True
        assert len(spec.layers) == len(d["layers"]) == len(spec.schedule)
        for layer, described in zip(spec.layers, d["layers"]):
            assert layer.block == "sublayer_output_norm"
            assert layer.parts["mixer"].kind == {"mamba2": "state_space", "parallel": "parallel",
                                                 "channel_delta": "gated_delta"}[described["type"]]
            assert ("feed_forward" in layer.parts) == (described["mlp"] is not None)
        names = [t.name for t in cb.expected_tensors(spec)]
        assert len(names) == len(set(names)) and "embed" in names and "final.norm" in names


def test_constants_reach_the_parts():
    spec = config("K").to_model_spec()
    par = spec.layers[0].parts["mixer"].params
    left = par["left"]["params"]
    assert (par["left_scale"], par["right_scale"]) == (1.3, 0.7)
    assert (left["window"], left["keep_first"], left["rot_dims"], left["rot_base"], left["scale"]) == (9, 2, 8, 1e4, 0.25)
    assert left["qk_norm_eps"] == 1e-5 and par["right"]["params"]["blocks"] == 3
    ff = spec.layers[0].parts["feed_forward"].params
    assert (ff["experts"], ff["top"], ff["groups"], ff["keep_groups"], ff["intermediate_size"]) == (8, 2, 4, 2, 32)
    assert spec.layers[1].parts["feed_forward"].params["groups"] is None


def test_ranks_come_from_tensor_shapes():
    d = json.loads(json.dumps(CONFIGS["K"]))
    for key in ("decay_rank", "gate_rank"):
        del d["layers"][2]["mixer"][key]
    cfg = cb.config_from_dict(d).with_tensor_shapes({"l2.mix.a1": (12, 64), "l2.mix.g1": (20, 64)})
    p = cfg.to_model_spec().layers[2].parts["mixer"].params
    assert (p["decay_rank"], p["gate_rank"]) == (12, 20)
    with pytest.raises(cb.CitlaliError, match="decay_rank"):
        config("K").with_tensor_shapes({"l2.mix.a1": (12, 64)})


@pytest.mark.parametrize("edit,match", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["layers"][0].update(type="conv"), "type 'conv'"),
    (lambda d: d["layers"][1]["mixer"].pop("state"), "state"),
    (lambda d: d["layers"][1]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(blocks=5), "blocks"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=0), "keep"),
    (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
])
def test_rejections_name_the_key(edit, match):
    d = json.loads(json.dumps(CONFIGS["K"]))
    edit(d)
    with pytest.raises(cb.CitlaliError, match=match):
        cb.config_from_dict(d)


def test_cache_keeps_the_pages_of_kept_tokens_and_nests_views():
    kv = KVRequirement(2, 16, window=70, value_dim=24, keep_first=3)
    reqs = [((kv, StateRequirement((10,))), StateRequirement((7,))), None, StateRequirement((7,))]
    cache = SequenceCache(reqs, num_slots=2, capacity_tokens=64 * 5, max_sequence_tokens=1024, dtype=torch.float32,
                          device="cpu", page_size=64)
    slot = cache.acquire()
    (left_kv, left_state), right = cache.view(0)
    assert left_kv.values.shape[-1] == 24 and left_kv.keys.shape[-1] == 16
    assert tuple(left_state.storage.shape) == (2, 10) and tuple(right.storage.shape) == (2, 7)
    assert not cache.has_view(1) and tuple(cache.view(2).storage.shape) == (2, 7)
    assert cache.view(2).storage.data_ptr() != right.storage.data_ptr()
    length = 0
    for n in [200] + [1] * 400:
        cache.reserve(slot, length + n)
        length += n
        cache.commit(slot, length)
        held = sorted(cache.kv_groups[0].held[slot])
        first_visible = max(0, length - 70 + 1) // 64
        assert held[0] == 0, "the page of the kept first tokens was given back"
        assert held[1:] == list(range(max(first_visible, 1), (length + 63) // 64))
    cache.release(slot)
    assert cache.pages_held() == 0


def test_plain_identities():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    w = torch.ones(12)
    y = plain.layer_norm(x, w, 0.0)
    assert float(y.mean(-1).abs().max()) < 1e-12 and float(((y * y).mean(-1) - 1).abs().max()) < 1e-12
    # one tap of one is no convolution; a window that covers everything is no window; keeping every token neither
    assert torch.equal(plain.causal_conv(x, torch.ones(12, 1)), x)
    assert torch.equal(plain.visible(9, 100, 0), plain.visible(9, None, 0))
    assert torch.equal(plain.visible(9, 2, 9), plain.visible(9, None, 0))
    assert plain.visible(9, 3, 1)[8].tolist() == [True, False, False, False, False, False, True, True, True]
    # no rotation at position 0; a rotation keeps lengths
    q = torch.randn(6, 2, 8, dtype=torch.float64)
    r = plain.rotate_interleaved(q, 4, 100.0)
    assert torch.equal(r[0], q[0]) and torch.allclose(r.norm(dim=-1), q.norm(dim=-1)) and torch.equal(r[..., 4:], q[..., 4:])
    # with every decay one and beta one, the delta rule returns the value just written for a unit key
    k = torch.nn.functional.normalize(torch.randn(4, 6, dtype=torch.float64), dim=-1)
    v = torch.randn(4, 3, dtype=torch.float64)
    o = plain.channel_delta_rule(k, k, v, torch.ones(4, 6, dtype=torch.float64), torch.ones(4, dtype=torch.float64))
    assert torch.allclose(o, v)
    # the state-space scan with a zero step size passes D x
    xs = torch.randn(4, 3, dtype=torch.float64)
    ys = plain.ssm_scan(xs, torch.randn(4, 5, dtype=torch.float64), torch.randn(4, 5, dtype=torch.float64),
                        torch.zeros(4, dtype=torch.float64), torch.tensor(1.0, dtype=torch.float64), 2.0)
    assert torch.allclose(ys, 2.0 * xs)
    # routing: top = experts takes all; one kept group of neighbours holds every choice
    s = torch.softmax(torch.randn(20, 12, dtype=torch.float64), -1)
    assert sorted(plain.route(s, 12, None, 1)[0].tolist()) == list(range(12))
    chosen = plain.route(s, 2, 4, 1)
    assert bool(((chosen // 3)[:, 0] == (chosen // 3)[:, 1]).all())
    assert bool(((chosen // 3)[:, 0] == s.view(20, 4, 3).max(-1).values.argmax(-1)).all())


def test_plain_model_runs_on_every_configuration():
    for name in CONFIGS:
        cfg = config(name)
        w = make_weights(cfg, 1)
        toks = list(range(1, 40))
        layers = []
        logits = plain.forward(cfg.to_dict(), w, toks, layers)
        assert logits.shape == (39, CONFIGS[name]["vocab"]) and bool(torch.isfinite(logits).all())
        # causality: a later token changes no earlier logits
        again = plain.forward(cfg.to_dict(), w, toks[:20] + [0] + toks[21:])
        assert torch.equal(again[:20], logits[:20]) and not torch.equal(again[20:], logits[20:])
