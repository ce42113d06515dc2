"""Configuration of the Gidirax decoder, read from its own config.json keys.

Gidirax is a decoder whose layers differ and whose norms sit on the sub-layers' outputs: x <- x + LN(mixer(x)), then
x <- x + LN(ff(x)), with a layer norm that has a weight and no bias.  config ``layers`` lists the layers in order, each
with a ``type`` that names its mixer, the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none):

* ``mamba2``: a state-space mixer (heads, vdim, state, groups, norm_groups, conv);
* ``channel_delta``: a gated delta rule with a decay per key channel, low-rank decay and gate projections and a sigmoid
  gate (heads, kv_heads, dim, vdim, conv);
* ``parallel``: two mixers side by side, ``left`` an attention over a sliding window that keeps the first tokens, behind a
  short convolution (heads, kv_heads, dim, vdim, conv, scale, mask {size, keep_first}, rot {dims, base}), ``right`` a
  recurrent block around a gated linear recurrent unit (width, blocks, conv), summed with ``left_scale`` and ``right_scale``.

The feed-forward is a mixture of experts (``mlp``: {kind: "moe", expert: {ff}, router: {experts, top, groups: {count,
keep}}}).  The head is the embedding table.  Every size and every constant that can differ between models comes from
config.json or from a tensor's shape (the ranks of the low-rank projections are read from the checkpoint's shapes when a
folder is loaded; a configuration built from a dictionary may name them as ``mixer.decay_rank`` / ``mixer.gate_rank``).

Tensor names: ``embed``, ``final.norm``; layer i's tensors start with ``l<i>.``: ``norm1``, ``norm2``, ``mix.*``,
``mlp.router``, ``mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..errors import require
from .lanizen import _int, _number
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

ARCHITECTURE = "Gidirax"
MAX_POSITIONS = 1 << 24          # positions are exact as float32 up to here; the design itself sets no limit
DEFAULT_RANK = 32                # of the low-rank projections, where neither the configuration nor a checkpoint says

_LAYER_TYPES = ("mamba2", "parallel", "channel_delta")


def _optional_conv(m, where):
    if m.get("conv") is not None:
        _int(m, "conv", where)


def _check_attention(m, where):
    heads = _int(m, "heads", where)
    kv = _int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
    require(heads % kv == 0, f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(m, "dim", where)
    if m.get("vdim") is not None:                 # absent: values have the keys' size
        _int(m, "vdim", where)
    _number(m, "scale", where)
    _optional_conv(m, where)
    if m.get("mask") is not None:
        _int(m["mask"], "size", where + ".mask")
        if m["mask"].get("keep_first") is not None:
            _int(m["mask"], "keep_first", where + ".mask", minimum=0)
    if m.get("rot") is not None:
        dims = _int(m["rot"], "dims", where + ".rot", minimum=0)
        _number(m["rot"], "base", where + ".rot")
        require(dims % 2 == 0 and dims <= dim, f"config.json: {where}.rot.dims {dims} must be even and at most dim {dim}")


def _check_recurrent(m, where):
    width = _int(m, "width", where)
    blocks = _int(m, "blocks", where)
    require(width % blocks == 0, f"config.json: {where}.width {width} does not split into {blocks} blocks")
    _optional_conv(m, where)


@dataclass(frozen=True)
class GidiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, validated

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GidiraxConfig":
        vocab = _int(d, "vocab", "the top level")
        width = _int(d, "width", "the top level")
        eps = _number(d.get("norm"), "eps", "norm")
        layers = d.get("layers")
        require(isinstance(layers, list) and len(layers) > 0, "config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            require(isinstance(layer, dict), f"config.json: {where} must be an object")
            kind = layer.get("type")
            require(kind in _LAYER_TYPES, f"config.json: {where}.type '{kind}' is unknown; known: {', '.join(_LAYER_TYPES)}")
            m, mw = layer.get("mixer"), where + ".mixer"
            require(isinstance(m, dict), f"config.json: {where} lacks 'mixer'")
            if kind == "mamba2":
                heads = _int(m, "heads", mw)
                _int(m, "vdim", mw), _int(m, "state", mw)
                groups = _int(m, "groups", mw) if m.get("groups") is not None else 1
                ng = _int(m, "norm_groups", mw) if m.get("norm_groups") is not None else 1
                require(heads % groups == 0, f"config.json: {mw}.heads {heads} is not a multiple of groups {groups}")
                require((heads * m["vdim"]) % ng == 0, f"config.json: {mw}: heads * vdim does not split into {ng} norm groups")
                _optional_conv(m, mw)
            elif kind == "channel_delta":
                heads = _int(m, "heads", mw)
                kv = _int(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
                require(heads % kv == 0, f"config.json: {mw}.heads {heads} is not a multiple of kv_heads {kv}")
                _int(m, "dim", mw), _int(m, "vdim", mw)
                _optional_conv(m, mw)
                for key in ("decay_rank", "gate_rank"):
                    if m.get(key) is not None:
                        _int(m, key, mw)
            else:
                require(isinstance(m.get("left"), dict) and isinstance(m.get("right"), dict),
                        f"config.json: {mw} needs 'left' and 'right'")
                _check_attention(m["left"], mw + ".left")
                _check_recurrent(m["right"], mw + ".right")
                for key in ("left_scale", "right_scale"):
                    if m.get(key) is not None:
                        _number(m, key, mw, positive=False)
            mlp = layer.get("mlp")
            if mlp is not None:
                lw = where + ".mlp"
                require(isinstance(mlp, dict) and mlp.get("kind") == "moe", f"config.json: {lw}.kind must be 'moe'")
                _int(mlp.get("expert"), "ff", lw + ".expert")
                r = mlp.get("router")
                experts, top = _int(r, "experts", lw + ".router"), _int(r, "top", lw + ".router")
                require(top <= experts, f"config.json: {lw}.router.top {top} exceeds experts {experts}")
                g = r.get("groups")
                if g is not None:
                    count, keep = _int(g, "count", lw + ".router.groups"), _int(g, "keep", lw + ".router.groups")
                    require(experts % count == 0 and keep <= count and keep * (experts // count) >= top,
                            f"config.json: {lw}.router.groups: {keep} of {count} groups of {experts} experts cannot give {top}")
            checked.append(copy.deepcopy(layer))
        return cls(vocab, width, eps, tuple(checked))

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "GidiraxConfig":
        """The sizes that only a checkpoint's tensors give: the ranks of the low-rank decay and gate projections."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            if layer["type"] != "channel_delta":
                continue
            for key, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                if name in shapes:
                    rank = int(shapes[name][0])
                    require(layer["mixer"].get(key) in (None, rank),
                            f"config.json: layers[{i}].mixer.{key} {layer['mixer'].get(key)} differs from the rows of {name}, {rank}")
                    layer["mixer"][key] = rank
        return GidiraxConfig(self.vocab, self.width, self.norm_eps, tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "layers": copy.deepcopy(list(self.layers))}

    def describe(self) -> Dict[str, Any]:
        kinds = [l["type"] + ("" if l.get("mlp") else " (no feed-forward)") for l in self.layers]
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps,
                "layers": ", ".join(kinds)}

    # ---- the architecture as data ----------------------------------------------------------------------------------
    def _mixer(self, i: int, layer) -> PartSpec:
        m, mp, eps = layer["mixer"], f"l{i}.mix", self.norm_eps
        if layer["type"] == "mamba2":
            return PartSpec("state_space", {
                "hidden_size": self.width, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                "groups": m.get("groups") or 1, "norm_groups": m.get("norm_groups") or 1, "conv": m.get("conv"),
                "norm_eps": eps,
                "names": {"in": f"{mp}.in", "conv": f"{mp}.conv", "conv_bias": f"{mp}.conv.b", "dt_bias": f"{mp}.dt_bias",
                          "a_log": f"{mp}.A_log", "skip": f"{mp}.D", "norm": f"{mp}.norm", "o": f"{mp}.o"}}, mp)
        if layer["type"] == "channel_delta":
            return PartSpec("gated_delta", {
                "hidden_size": self.width, "heads": m["heads"], "kv_heads": m.get("kv_heads") or m["heads"],
                "dim": m["dim"], "vdim": m["vdim"], "conv": m.get("conv"), "norm_eps": eps, "decay": "channel",
                "decay_rank": m.get("decay_rank") or DEFAULT_RANK, "gate_rank": m.get("gate_rank") or DEFAULT_RANK,
                "gate_act": "sigmoid",
                "names": {"q": f"{mp}.q", "k": f"{mp}.k", "v": f"{mp}.v", "b": f"{mp}.b", "a1": f"{mp}.a1", "a2": f"{mp}.a2",
                          "g1": f"{mp}.g1", "g2": f"{mp}.g2", "q_conv": f"{mp}.q.conv", "k_conv": f"{mp}.k.conv",
                          "v_conv": f"{mp}.v.conv", "a_log": f"{mp}.A_log", "dt_bias": f"{mp}.dt_bias", "norm": f"{mp}.norm",
                          "o": f"{mp}.o"}}, mp)
        l, r = m["left"], m["right"]
        lp, rp = f"{mp}.left", f"{mp}.right"
        mask, rot = l.get("mask"), l.get("rot")
        left = {"kind": "window_attention", "prefix": lp, "params": {
            "hidden_size": self.width, "heads": l["heads"], "kv_heads": l.get("kv_heads") or l["heads"], "dim": l["dim"],
            "vdim": l.get("vdim") or l["dim"], "conv": l.get("conv"), "qk_norm_eps": eps, "scale": l["scale"],
            "rot_dims": rot["dims"] if rot is not None else 0, "rot_base": rot["base"] if rot is not None else 1.0,
            "window": mask["size"] if mask is not None else None,
            "keep_first": (mask.get("keep_first") or 0) if mask is not None else 0,
            "names": {"q": f"{lp}.q", "k": f"{lp}.k", "v": f"{lp}.v", "q_conv": f"{lp}.q.conv", "k_conv": f"{lp}.k.conv",
                      "v_conv": f"{lp}.v.conv", "q_norm": f"{lp}.q.norm", "k_norm": f"{lp}.k.norm", "o": f"{lp}.o"}}}
        right = {"kind": "gated_recurrent", "prefix": rp, "params": {
            "hidden_size": self.width, "width": r["width"], "blocks": r["blocks"], "conv": r.get("conv"),
            "names": {"y": f"{rp}.y", "y_bias": f"{rp}.y.b", "x": f"{rp}.x", "x_bias": f"{rp}.x.b", "conv": f"{rp}.conv",
                      "conv_bias": f"{rp}.conv.b", "gate_a": f"{rp}.ra", "gate_a_bias": f"{rp}.ra.b", "gate_i": f"{rp}.ri",
                      "gate_i_bias": f"{rp}.ri.b", "lam": f"{rp}.lam", "o": f"{rp}.o"}}}
        return PartSpec("parallel", {"left": left, "right": right,
                                     "left_scale": 1.0 if m.get("left_scale") is None else m["left_scale"],
                                     "right_scale": 1.0 if m.get("right_scale") is None else m["right_scale"]}, mp)

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            p = f"l{i}"
            norm = {"size": self.width, "eps": self.norm_eps}
            parts = {"mixer_norm": PartSpec("layer_norm", dict(norm, tensor=f"{p}.norm1"), f"{p}.norm1"),
                     "mixer": self._mixer(i, layer)}
            mlp = layer.get("mlp")
            if mlp is not None:
                r = mlp["router"]
                g = r.get("groups")
                parts["feed_forward_norm"] = PartSpec("layer_norm", dict(norm, tensor=f"{p}.norm2"), f"{p}.norm2")
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden_size": self.width, "experts": r["experts"], "top": r["top"],
                    "intermediate_size": mlp["expert"]["ff"], "groups": g["count"] if g is not None else None,
                    "keep_groups": g["keep"] if g is not None else None}, f"{p}.mlp")
            layers.append(LayerSpec(block="sublayer_output_norm", parts=parts))
            schedule.append(ScheduleStep(i))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule),
            final_norm=PartSpec("layer_norm", {"size": self.width, "eps": self.norm_eps, "tensor": "final.norm"}, "final.norm"),
            head_name="head", tie_head_to_embedding=True, stop_token_ids=())
        spec.validate()
        return spec
