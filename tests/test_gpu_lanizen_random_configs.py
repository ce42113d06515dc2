"""Lanizen configurations drawn at random with a fixed seed: layer orders, stream counts, head counts and group sizes,
head / value / latent sizes (odd ones, and ones the tensor-core kernels take), taps, windows shorter and longer than
the prompts, readers of earlier caches, layers without feed-forward, widths and vocabularies that are no multiples
of 8.  Two unequal prompts in one step, then tokens one by one, against the plain implementation, in both dtypes."""
import json
import os
import random

import pytest
import torch

import citlali_b200 as cb
import plain_lanizen as plain
import replay
from helpers import random_tokens
from lanizen_models import make_weights

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(seed)
    width = rng.choice([24, 40, 52, 64, 72, 100, 128])
    layers, owners = [], []
    for i in range(rng.randint(2, 5)):
        ff = None if rng.random() < 0.25 else rng.choice([32, 50, 96, 136])
        mlp = None if ff is None else {"kind": "dense", "ff": ff}
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            m = {"heads": kv * rng.choice([1, 2, 4]), "kv_heads": kv, "dim": rng.choice([4, 12, 16, 32, 36, 64, 72]),
                 "vdim": rng.choice([4, 8, 20, 32, 48]), "conv": rng.choice([1, 2, 3, 4, 5])}
            layers.append({"type": "delta", "mixer": m, "mlp": mlp})
        else:
            m = {"heads": rng.choice([1, 2, 5, 8, 17]), "dim": rng.choice([4, 8, 16, 24, 32]), "vdim": rng.choice([4, 8, 16, 40]),
                 "q_rank": rng.choice([8, 12, 24, 40]), "scale": rng.choice([0.1, 0.25, 0.5])}
            if owners and rng.random() < 0.4:
                src = rng.choice(owners)
                m.update(kv_from=src, kv_rank=layers[src]["mixer"]["kv_rank"], rot_dim=layers[src]["mixer"]["rot_dim"])
                if "rot" in layers[src]["mixer"]:
                    m["rot"] = dict(layers[src]["mixer"]["rot"])
            else:
                rank, rot = rng.choice([(64, 16), (128, 32), (20, 6), (48, 8), (64, 0), (33, 4)])
                m.update(kv_rank=rank, rot_dim=rot)
                if rot and rng.random() < 0.85:
                    m["rot"] = {"base": rng.choice([100.0, 1e4, 5e5]), "dims": rot if rng.random() < 0.7 else rot // 4 * 2}
                owners.append(i)
            if rng.random() < 0.8:
                m["mask"] = {"size": rng.choice([1, 3, 17, 64, 90, 300])}
            layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    d = {"architecture": "Lanizen", "vocab": rng.choice([97, 256, 333, 1000]), "width": width,
         "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}
    if rng.random() < 0.8:
        d["streams"] = rng.choice([1, 2, 3, 5])
    if rng.random() < 0.7:
        d["embedding"] = {"scale": rng.choice([0.5, 2.0, 4.0])}
    return d


@pytest.mark.parametrize("seed", range(10))
def test_random_configuration(seed, tmp_path):
    d = draw(1000 + seed)
    cfg = cb.config_from_dict(json.loads(json.dumps(d)))
    w = make_weights(cfg, seed)
    path = str(tmp_path / "m")
    os.makedirs(path)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    cb.write_safetensors(os.path.join(path, "model.safetensors"), lambda: iter(w.items()), metadata={"format": "pt"})
    reqs = [("a", random_tokens(d["vocab"], 70, seed)), ("b", random_tokens(d["vocab"], 23, seed + 1)),
            ("c", random_tokens(d["vocab"], 131, seed + 2))]
    want = {rid: plain.forward(cfg.to_dict(), w, toks) for rid, toks in reqs}
    steps = replay.batched(reqs, [50, 9, 100], 3)
    # 32-bit: every row within rounding of the exact evaluation.  bfloat16: rounding to 8 bits at every product's operands;
    # tiny layers of unit-scale random weights amplify it at single rows, so the mean over the rows is held too
    for dtype, worst_allowed, mean_allowed in (("float32", 4e-5, 4e-5), ("bfloat16", 1.2e-1, 2.5e-2)):
        s = cb.InferenceSession().load_model(path, max_context=256, dtype=dtype, max_batch=3)
        got = replay.run_in_process(s, steps)
        errs = []
        for (rid, pos), row in got.items():
            ref = want[rid][pos]
            errs.append(float((row.double() - ref).abs().max()) / float(ref.abs().max()))
        assert max(errs) <= worst_allowed and sum(errs) / len(errs) <= mean_allowed, \
            f"seed {seed} {dtype}: worst {max(errs):.3e}, mean {sum(errs) / len(errs):.3e}\n{d}"
