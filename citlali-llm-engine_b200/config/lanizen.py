"""Configuration of the Lanizen decoder, read from its own config.json keys.

Lanizen is a decoder whose layers differ: config ``layers`` lists them in order, each with a ``type`` (``delta``: a
gated delta-rule mixer with a recurrent state; ``latent_attention``: attention through a cached latent with a sliding
window, a sink and an output gate, optionally reading an earlier layer's cache through ``kv_from``), the mixer's sizes
(``mixer``) and its feed-forward (``mlp``: ``{"kind": "dense", "ff": n}``, or null for none).  The residual is kept
as ``streams`` parallel streams joined by small learned mixtures (absent: the plain residual sum).  The layer norms are
RMS norms whose stored weight lies around zero (factor 1 + w); the embedding rows are multiplied by
``embedding.scale``.  Every size comes from config.json; what it does not mention does not exist (no mask: every
earlier token is seen; no ``rot``: no rotation).

Tensor names: ``embed``, ``head``, ``final.norm``; layer i's tensors start with ``l<i>.``: ``norm1``, ``norm2``,
``mix.*``, ``mlp.up``, ``mlp.down``, ``hc1.{in,out,mix}``, ``hc2.{in,out,mix}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import require
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

ARCHITECTURE = "Lanizen"
MAX_POSITIONS = 1 << 24          # positions are exact as float32 up to here; the design itself sets no limit

_LAYER_TYPES = ("delta", "latent_attention")
_MLP_KINDS = ("dense",)


def _int(d, key, where, minimum=1):
    require(isinstance(d, dict) and key in d, f"config.json: {where} lacks '{key}'")
    v = d[key]
    require(isinstance(v, int) and not isinstance(v, bool) and v >= minimum,
            f"config.json: {where}.{key} must be an integer of at least {minimum}, got {v!r}")
    return v


def _number(d, key, where, positive=True):
    require(isinstance(d, dict) and key in d, f"config.json: {where} lacks '{key}'")
    v = d[key]
    require(isinstance(v, (int, float)) and not isinstance(v, bool) and (v > 0 or not positive),
            f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class LanizenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: Optional[float]
    streams: Optional[int]
    layers: Tuple[Dict[str, Any], ...]          # as config.json lists them, validated

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LanizenConfig":
        vocab = _int(d, "vocab", "the top level")
        width = _int(d, "width", "the top level")
        eps = _number(d.get("norm"), "eps", "norm")
        emb = d.get("embedding")
        scale = None if emb is None or emb.get("scale") is None else _number(emb, "scale", "embedding", positive=False)
        streams = None if d.get("streams") is None else _int(d, "streams", "the top level")
        require(streams is None or streams <= 8, f"config.json: streams must be at most 8, got {streams}")
        layers = d.get("layers")
        require(isinstance(layers, list) and len(layers) > 0, "config.json: 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            require(isinstance(layer, dict), f"config.json: {where} must be an object")
            kind = layer.get("type")
            require(kind in _LAYER_TYPES, f"config.json: {where}.type '{kind}' is unknown; known: {', '.join(_LAYER_TYPES)}")
            m = layer.get("mixer")
            mw = where + ".mixer"
            if kind == "delta":
                heads = _int(m, "heads", mw)
                kv = _int(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
                require(heads % kv == 0, f"config.json: {mw}.heads {heads} is not a multiple of kv_heads {kv}")
                _int(m, "dim", mw), _int(m, "vdim", mw)
                if m.get("conv") is not None:
                    _int(m, "conv", mw)
            else:
                for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _int(m, key, mw)
                _int(m, "rot_dim", mw, minimum=0)
                _number(m, "scale", mw)
                if m.get("mask") is not None:
                    _int(m["mask"], "size", mw + ".mask")
                if m.get("rot") is not None:
                    dims = _int(m["rot"], "dims", mw + ".rot", minimum=0)
                    _number(m["rot"], "base", mw + ".rot")
                    require(dims % 2 == 0 and dims <= m["rot_dim"],
                            f"config.json: {mw}.rot.dims {dims} must be even and at most rot_dim {m['rot_dim']}")
                src = m.get("kv_from")
                if src is not None:
                    require(isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i
                            and layers[src].get("type") == "latent_attention" and layers[src]["mixer"].get("kv_from") is None,
                            f"config.json: {mw}.kv_from must name an earlier latent_attention layer with a latent of its own, "
                            f"got {src!r}")
                    other = layers[src]["mixer"]
                    for key in ("kv_rank", "rot_dim", "rot"):
                        require(other.get(key) == m.get(key),
                                f"config.json: {mw}.{key} differs from that of layer {src}, whose cache it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                require(isinstance(mlp, dict) and mlp.get("kind") in _MLP_KINDS,
                        f"config.json: {where}.mlp.kind must be one of: {', '.join(_MLP_KINDS)}")
                _int(mlp, "ff", where + ".mlp")
            checked.append(copy.deepcopy(layer))
        return cls(vocab, width, eps, scale, streams, tuple(checked))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.embedding_scale is not None:
            d["embedding"] = {"scale": self.embedding_scale}
        if self.streams is not None:
            d["streams"] = self.streams
        return d

    def describe(self) -> Dict[str, Any]:
        kinds = [l["type"] + ("" if l.get("mlp") else " (no feed-forward)") for l in self.layers]
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm_eps": self.norm_eps,
                "embedding_scale": self.embedding_scale, "streams": self.streams, "layers": ", ".join(kinds)}

    # ---- the architecture as data ----------------------------------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        readers: Dict[int, list] = {}                 # layer -> the windows of the layers that read its cache
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                owner = i if m.get("kv_from") is None else m["kv_from"]
                readers.setdefault(owner, []).append(m["mask"]["size"] if m.get("mask") is not None else None)
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}", layer["mixer"]
            offset_norm = {"size": self.width, "eps": self.norm_eps, "offset": 1.0}
            parts = {"mixer_norm": PartSpec("rms_norm", dict(offset_norm, tensor=f"{p}.norm1"), f"{p}.norm1")}
            if layer["type"] == "delta":
                mp = f"{p}.mix"
                parts["mixer"] = PartSpec("gated_delta", {
                    "hidden_size": self.width, "heads": m["heads"], "kv_heads": m.get("kv_heads") or m["heads"],
                    "dim": m["dim"], "vdim": m["vdim"], "conv": m.get("conv"), "norm_eps": self.norm_eps,
                    "names": {"q": f"{mp}.q", "k": f"{mp}.k", "v": f"{mp}.v", "gate": f"{mp}.g", "b": f"{mp}.b",
                              "a": f"{mp}.a", "q_conv": f"{mp}.q.conv", "k_conv": f"{mp}.k.conv", "v_conv": f"{mp}.v.conv",
                              "a_log": f"{mp}.A_log", "dt_bias": f"{mp}.dt_bias", "norm": f"{mp}.norm", "o": f"{mp}.o"},
                }, mp)
                schedule.append(ScheduleStep(i))
            else:
                mp = f"{p}.mix"
                own = m.get("kv_from") is None
                windows = readers[i] if own else []
                parts["mixer"] = PartSpec("latent_attention", {
                    "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                    "vdim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"],
                    "norm_eps": self.norm_eps, "window": m["mask"]["size"] if m.get("mask") is not None else None,
                    "cache_window": None if (not own or None in windows) else max(windows),
                    "rot_dims": m["rot"]["dims"] if m.get("rot") is not None else 0,
                    "rot_base": m["rot"]["base"] if m.get("rot") is not None else 1.0,
                    "kv_projection": own,
                    "names": {"dq": f"{mp}.dq", "dq_norm": f"{mp}.dq.norm", "uq": f"{mp}.uq", "dkv": f"{mp}.dkv",
                              "dkv_norm": f"{mp}.dkv.norm", "uk": f"{mp}.uk", "uv": f"{mp}.uv", "sink": f"{mp}.sink",
                              "gate": f"{mp}.g", "o": f"{mp}.o"},
                }, mp)
                schedule.append(ScheduleStep(i, None if own else int(m["kv_from"])))
            if layer.get("mlp") is not None:
                parts["feed_forward_norm"] = PartSpec("rms_norm", dict(offset_norm, tensor=f"{p}.norm2"), f"{p}.norm2")
                parts["feed_forward"] = PartSpec("relu_squared", {
                    "hidden_size": self.width, "intermediate_size": layer["mlp"]["ff"],
                    "up": f"{p}.mlp.up", "down": f"{p}.mlp.down"}, f"{p}.mlp")
            if self.streams is None:
                layers.append(LayerSpec(block="pre_norm_residual", parts=parts))
            else:
                names = {f"{role}_{k}": f"{p}.hc{q}.{k}" for q, role in ((1, "mixer"), (2, "feed_forward"))
                         for k in ("in", "out", "mix")}
                layers.append(LayerSpec(block="hyper_connection", parts=parts,
                                        block_params={"streams": self.streams, "names": names}))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
            embedding_name="embed", layers=tuple(layers), schedule=tuple(schedule),
            final_norm=PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "offset": 1.0,
                                             "tensor": "final.norm"}, "final.norm"),
            head_name="head", tie_head_to_embedding=False, stop_token_ids=(),
            embedding_scale=self.embedding_scale, residual_streams=self.streams)
        spec.validate()
        return spec
