"""Small Lanizen configurations and weights for tests.

The configurations differ from one another in every size and option: streams (none, 1, 2, 4), head counts and group
sizes of the delta rule, head sizes that are no multiple of 32, value sizes that are no multiple of 32, 1 to 4
convolution taps, latent ranks, windows (none, shorter than a page, a page and one, reaching over several pages), a
reader of another layer's cache with a wider window than its owner's, partial rotation, layers without feed-forward,
widths and vocabularies that are no multiples of 8.  Weights are drawn so that every mechanism matters to the logits
(unit-scale activations, decays well inside (0, 1), sinks of the size of the scores, stream mixtures away from the
identity), stored in bfloat16 so that both compute paths and the plain implementation read the same numbers.
"""
import json
import os

import torch

import citlali_b200 as cb


def _delta(heads, kv_heads, dim, vdim, conv, ff):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim}
    if conv is not None:
        m["conv"] = conv
    return {"type": "delta", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, ff, kv_from=None, rot_dims=None, base=1e4, scale=0.25):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # two streams; a reader (layer 3) of layer 1's cache with a wider window than its owner's
    "P": {"architecture": "Lanizen", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
          "streams": 2, "layers": [
              _delta(4, 2, 16, 24, 4, 96),
              _latent(3, 16, 8, 16, 24, 40, 9, 96),
              _delta(2, 2, 32, 32, 2, None),
              _latent(2, 24, 8, 40, 16, 40, 20, 80, kv_from=1)]},
    # one plain residual, no embedding scale, no window, a partial rotation, one tap, odd width and vocabulary
    "Q": {"architecture": "Lanizen", "vocab": 333, "width": 60, "norm": {"eps": 1e-6}, "layers": [
              _latent(5, 12, 16, 20, 36, 48, None, 100, rot_dims=8, base=5e5, scale=0.3),
              _delta(3, 3, 20, 44, 1, 70),
              _delta(6, 2, 48, 16, 3, None)]},
    # four streams, windows around a page's edge, four query heads a key head, a head size over 64
    "R": {"architecture": "Lanizen", "vocab": 512, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
          "streams": 4, "layers": [
              _latent(4, 32, 32, 32, 64, 96, 65, 128, base=1e6, scale=0.125),
              _delta(8, 2, 80, 40, 4, 128),
              _latent(2, 16, 32, 48, 32, 96, 130, None, kv_from=0, base=1e6, scale=0.2),
              _latent(3, 8, 4, 8, 16, 12, 1, 64, scale=1.0)]},
    # one stream that still passes its three mixtures
    "S": {"architecture": "Lanizen", "vocab": 128, "width": 32, "norm": {"eps": 1e-5}, "streams": 1, "layers": [
              _delta(1, 1, 8, 8, 2, 48),
              _latent(1, 8, 2, 8, 8, 8, 4, 48, scale=0.5),
              _delta(2, 2, 8, 12, None, None)]},
}


def config(name):
    return cb.config_from_dict(json.loads(json.dumps(CONFIGS[name])))


def make_weights(cfg, seed):
    """{name: bfloat16 tensor} for every tensor the model reads."""
    g = torch.Generator().manual_seed(seed)
    S = cfg.streams
    out = {}
    for spec in cb.expected_tensors(cfg.to_model_spec()):
        n, shape = spec.name, tuple(spec.shape)
        r = torch.randn(shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith((".norm1", ".norm2")) or n == "final.norm":
            t = 0.3 * r                                    # the factor is 1 + w
        elif n.endswith((".mix.norm", ".dq.norm", ".dkv.norm")):
            t = 1.0 + 0.3 * r
        elif n.endswith(".conv"):
            t = 0.6 * r
        elif n.endswith(".A_log"):
            t = -1.0 + 0.7 * r
        elif n.endswith(".dt_bias"):
            t = r
        elif n.endswith(".sink"):
            t = 1.5 * r
        elif n.endswith((".in",)):
            t = 1.0 / S + 0.3 * r
        elif n.endswith(".out"):
            t = 1.0 + 0.3 * r
        elif n.endswith(".hc1.mix") or n.endswith(".hc2.mix"):
            t = torch.eye(S) + 0.25 * r
        elif n.endswith((".mix.b", ".mix.a")):
            t = 2.0 * r / shape[1] ** 0.5
        else:
            t = r / shape[1] ** 0.5                        # matrices [out, in]
        out[n] = t.to(torch.bfloat16)
    return out


def write_model(path, name, seed):
    cfg = config(name)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    w = make_weights(cfg, seed)
    cb.write_safetensors(os.path.join(path, "model.safetensors"), lambda: iter(w.items()), metadata={"format": "pt"})
    return cfg, w
