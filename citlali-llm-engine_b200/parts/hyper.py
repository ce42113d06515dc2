"""A layer around several residual streams (hyper-connections).

Instead of one residual x there are S copies X_1 .. X_S (float32, ``[S, rows, hidden]``).  For sub-layer q of a layer
(1: the mixer, 2: the feed-forward), with three small learned tensors ``in`` [S], ``out`` [S] and ``mix`` [S, S]
(indexed [from, to]):

    u = sum_s in[s] X_s;    y = sublayer(norm(u));    X_t <- sum_s mix[s, t] X_s + out[t] y   (all t from the old X).

With S = 1 and in = out = mix = 1 this is the pre-norm residual layer.  The mixture u, the norm and the write-back are
32-bit: one kernel reads the streams and leaves the normed rows in the compute dtype (``ops.hyper_read_norm``), one
updates all streams in place (``ops.hyper_write``); a write-back and the read that follows it, in this layer or the next,
are one pass over the streams (``ops.hyper_write_read_norm``; the last write-back of a layer is left in
``batch.stream_write`` for whoever comes next).  The sub-layer's parts are the ones any block uses: they add their
output into a float32 buffer, which here is a fresh one (a part that says ``can_overwrite`` is told to store instead of
add and spares the zero fill).  The norm must be an RMS norm (its sum of squares is taken inside the read kernel).

Parts by name: ``mixer_norm``, ``mixer``, ``feed_forward_norm``, ``feed_forward`` (either pair optional).  Block
parameters: ``streams``; ``names``: full tensor names ``mixer_in``, ``mixer_out``, ``mixer_mix``, ``feed_forward_in``,
``feed_forward_out``, ``feed_forward_mix``.
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import require
from ..weights.loader import TensorSpec
from .base import build_part, register_part
from .delta import bind_float32
from .norm import RMSNorm


class HyperConnectionBlock:
    takes_stream_write = True        # does the write-back the block ahead left in ``batch.stream_write``

    def __init__(self, layer_spec):
        has = layer_spec.parts.__contains__
        params = layer_spec.block_params
        self.residual_streams = int(params["streams"])
        require(1 <= self.residual_streams <= 8, f"a layer takes 1 to 8 residual streams, not {self.residual_streams}")
        names = dict(params.get("names") or {})
        self.subs = []                                   # (role, norm, part, names of in / out / mix)
        for role, norm_name in (("mixer", "mixer_norm"), ("feed_forward", "feed_forward_norm")):
            if not has(role):
                continue
            norm = build_part("norm", layer_spec.part(norm_name))
            require(isinstance(norm, RMSNorm), f"the norm in front of a {role} on several streams must be an RMS norm")
            part = build_part(role, layer_spec.part(role))
            for k in ("in", "out", "mix"):
                require(f"{role}_{k}" in names, f"a layer on several streams needs the tensor name '{role}_{k}'")
            self.subs.append((role, norm, part, tuple(str(names[f"{role}_{k}"]) for k in ("in", "out", "mix"))))
        self.mixer = next((p for r, _, p, _ in self.subs if r == "mixer"), None)
        self.weights = {}

    def parts(self):
        return [p for _, norm, part, _ in self.subs for p in (norm, part)]

    def tensor_specs(self):
        S = self.residual_streams
        specs = [t for p in self.parts() for t in p.tensor_specs()]
        for _, _, _, (w_in, w_out, w_mix) in self.subs:
            specs += [TensorSpec(w_in, (S,), "state"), TensorSpec(w_out, (S,), "state"), TensorSpec(w_mix, (S, S), "state")]
        return specs

    def cache_requirement(self):
        return self.mixer.cache_requirement() if self.mixer is not None else None

    def bind(self, weights, ctx):
        S = self.residual_streams
        for p in self.parts():
            p.bind(weights, ctx)
        for role, _, _, (w_in, w_out, w_mix) in self.subs:
            self.weights[role] = (bind_float32(weights, w_in, (S,), ctx), bind_float32(weights, w_out, (S,), ctx),
                                  bind_float32(weights, w_mix, (S, S), ctx))
        # the read kernel takes the gain in 32-bit
        self.gains = {role: norm.gain.to(torch.float32).contiguous() for role, norm, _, _ in self.subs}
        self.dtype = ctx.dtype

    def forward(self, X, batch, cache_view, write_cache=True):
        S, rows, hidden = X.shape
        require(S == self.residual_streams, f"the layer takes {self.residual_streams} streams, got {S}")
        pending, batch.stream_write = batch.stream_write, None        # (y, mix, out) of the sub-layer before, not yet applied
        for role, norm, part, _ in self.subs:
            w_in, w_out, w_mix = self.weights[role]
            h = torch.empty((rows, hidden), dtype=self.dtype, device=X.device)
            if pending is None:
                ops.hyper_read_norm(X, w_in, self.gains[role], norm.eps, h)
            else:
                ops.hyper_write_read_norm(X, pending[0], pending[1], pending[2], w_in, self.gains[role], norm.eps, h)
            fresh = bool(getattr(part, "can_overwrite", False))
            y = (torch.empty if fresh else torch.zeros)((rows, hidden), dtype=torch.float32, device=X.device)
            extra = {"overwrite": True} if fresh else {}
            if role == "mixer":
                part.forward(h, batch, cache_view, y, write_cache, **extra)
            else:
                part.forward(h, batch, y, **extra)
            pending = (y, w_mix, w_out)
        batch.stream_write = pending
        return X


register_part("block", "hyper_connection", HyperConnectionBlock)
