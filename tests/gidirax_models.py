"""Small Gidirax configurations and weights for tests.

The configurations differ from one another in every size and option: layer orders, head counts and group sizes, head sizes
that are no multiple of 32, key and value sizes that differ, 1 to 4 convolution taps or none, state sizes, norm groups,
windows (shorter than a page, a page and one, several pages), kept first tokens (none, some, more than the window),
partial rotation, gate blocks, expert counts and groups (no groups, every group kept, one expert a group), ranks, layers
without a feed-forward, widths and vocabularies that are no multiples of 8.  Weights are drawn so that every mechanism
matters to the logits (unit-scale activations, decays well inside (0, 1), routers that spread their choices), stored in
bfloat16 so that both compute paths and the plain implementation read the same numbers.
"""
import json
import os

import torch

import citlali_b200 as cb


def moe(experts, top, ff, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def ssm(heads, vdim, state, groups, norm_groups, conv, mlp):
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups}
    if conv is not None:
        m["conv"] = conv
    return {"type": "mamba2", "mixer": m, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp, decay_rank=8, gate_rank=8):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "decay_rank": decay_rank, "gate_rank": gate_rank}
    if conv is not None:
        m["conv"] = conv
    return {"type": "channel_delta", "mixer": m, "mlp": mlp}


def par(heads, kv_heads, dim, vdim, conv, window, keep_first, rot_dims, base, scale, width, blocks, rconv, mlp,
        left_scale=1.0, right_scale=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        left["conv"] = conv
    if window is not None:
        left["mask"] = {"size": window, "keep_first": keep_first}
    if rot_dims is not None:
        left["rot"] = {"dims": rot_dims, "base": base}
    right = {"width": width, "blocks": blocks}
    if rconv is not None:
        right["conv"] = rconv
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


CONFIGS = {
    # every kind of layer; a window shorter than a page with kept tokens; groups of which some are dropped
    "K": {"architecture": "Gidirax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        par(4, 2, 16, 24, 3, 9, 2, 8, 1e4, 0.25, 48, 3, 4, moe(8, 2, 32, 4, 2), 1.3, 0.7),
        ssm(4, 8, 16, 2, 2, 4, moe(6, 3, 16)),
        delta(4, 2, 16, 24, 4, moe(4, 1, 48, 2, 1), 8, 16),
        ssm(2, 24, 40, 1, 1, 2, None)]},
    # odd width and vocabulary, no groups, a window of a page and one with more kept tokens than a tap reaches, one tap,
    # a head size over 64, one query head a key head
    "L": {"architecture": "Gidirax", "vocab": 333, "width": 60, "norm": {"eps": 1e-6}, "layers": [
        delta(3, 3, 20, 44, 1, moe(5, 2, 24), 4, 12),
        par(3, 3, 80, 12, 1, 65, 5, 80, 5e5, 0.1, 64, 1, 2, None, 0.5, 2.0),
        delta(6, 2, 48, 16, 3, moe(12, 4, 16, 3, 2), 16, 8)]},
    # windows over several pages, no kept tokens, no rotation on one layer and all of the head on another, no convolutions,
    # every group kept, one expert a group, top = experts
    "M": {"architecture": "Gidirax", "vocab": 512, "width": 96, "norm": {"eps": 1e-6}, "layers": [
        par(8, 2, 32, 32, None, 130, 0, 32, 1e6, 0.125, 96, 4, None, moe(4, 4, 32, 4, 4)),
        ssm(6, 16, 32, 3, 3, None, moe(8, 2, 16, 8, 3)),
        par(2, 1, 24, 40, 4, 1, 3, None, None, 0.2, 32, 2, 3, moe(16, 4, 16, 4, 3), 1.0, 1.0),
        par(2, 2, 16, 16, 2, None, 0, 4, 1e2, 0.3, 16, 1, 1, None)]},
}


def config(name):
    return cb.config_from_dict(json.loads(json.dumps(CONFIGS[name])))


def make_weights(cfg, seed):
    """{name: bfloat16 tensor} for every tensor the model reads."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in cb.expected_tensors(cfg.to_model_spec()):
        if spec.optional:
            continue
        n, shape = spec.name, tuple(spec.shape)
        r = torch.randn(shape, generator=g)
        if n == "embed":
            t = r
        elif n.endswith((".norm1", ".norm2", ".mix.norm", ".q.norm", ".k.norm")) or n == "final.norm":
            t = 1.0 + 0.3 * r
        elif n.endswith(".conv"):
            t = 0.6 * r
        elif n.endswith(".b") and len(shape) == 1 or n.endswith((".ra.b", ".ri.b")):
            t = 0.3 * r                                    # biases
        elif n.endswith(".A_log"):
            t = -1.0 + 0.7 * r
        elif n.endswith(".dt_bias"):
            t = r
        elif n.endswith(".D"):
            t = 1.0 + 0.3 * r
        elif n.endswith(".lam"):
            t = -1.5 + r                                   # decays a = exp(-8 r softplus(lam)) inside (0, 1)
        elif n.endswith((".ra", ".ri")):
            t = 1.5 * r / shape[2] ** 0.5
        elif n.endswith(".router"):
            t = 3.0 * r / shape[1] ** 0.5
        elif n.endswith(".mix.b"):
            t = 2.0 * r / shape[1] ** 0.5
        else:
            t = r / shape[-1] ** 0.5                       # matrices [out, in]
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
