"""Routed experts: a feed-forward made of ``experts`` small gated feed-forwards of which every token uses ``top``.

Router logits z = W_router h in 32-bit; scores s = softmax(z) over all experts.  The experts form ``groups`` equal groups of
neighbours; a group's score is the largest score in it, and only experts of the ``keep_groups`` best groups can be chosen
(``groups`` None: no groups).  The ``top`` experts with the largest scores among those are chosen; their weights are their
scores, not renormalised.  An expert is  W_down (silu(W_gate h) * (W_up h)), without biases; the output is the weighted sum
of the chosen experts' outputs.

How it runs: the router is a product with a float32 result; one kernel turns a row's logits into a row of weights (zero
for an expert that was not chosen); the experts' gate and up matrices are ONE product for all experts (the gate in its
epilogue where the shape allows), a kernel multiplies every expert's activations by the row's weight for it, and the
experts' output matrices side by side are ONE product that sums over experts.  Nothing depends on counts known to the host
only, so a decoding step replays as a graph; the price is that every expert's matrices are applied to every row.

Parameters: hidden_size, experts, top, intermediate_size, groups, keep_groups; ``names``: {"router": name, "gate": [names],
"up": [names], "down": [names]} (default ``<prefix>.router`` and ``<prefix>.e<i>.{gate,up,down}``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..errors import require
from .base import register_part
from .linear import DenseLinear, ExpertDown, ExpertGateUp


class RoutedExperts:
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.E, self.top, self.ff = int(params["experts"]), int(params["top"]), int(params["intermediate_size"])
        self.groups = None if params.get("groups") is None else int(params["groups"])
        self.keep = int(params.get("keep_groups") or (self.groups or 1))
        require(1 <= self.top <= self.E, f"{prefix}: {self.top} of {self.E} experts cannot be chosen")
        require(self.E <= 512, f"{prefix}: {self.E} experts exceed the router kernel's 512")
        if self.groups is not None:
            require(self.groups >= 1 and self.E % self.groups == 0, f"{prefix}: {self.E} experts do not form {self.groups} equal groups")
            require(1 <= self.keep <= self.groups and self.keep * (self.E // self.groups) >= self.top,
                    f"{prefix}: {self.keep} groups of {self.E // self.groups} experts cannot give {self.top} experts")
        n = dict(params.get("names") or {})
        each = lambda role: list(n.get(role) or [f"{prefix}.e{i}.{role}" for i in range(self.E)])
        self.router = DenseLinear([str(n.get("router") or f"{prefix}.router")], [self.E], self.hidden)
        self.gate_up = ExpertGateUp(each("gate"), each("up"), self.ff, self.hidden)
        self.down = ExpertDown(each("down"), self.ff, self.hidden)
        self.prefix = prefix

    def tensor_specs(self):
        return self.router.tensor_specs() + self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, weights, ctx):
        self.router.bind(weights, ctx)
        self.gate_up.bind(weights, ctx)
        self.down.bind(weights, ctx)
        self.dtype = ctx.dtype

    def route(self, h):
        """The row's weights for every expert, float32 [rows, experts]: its score where chosen, zero elsewhere."""
        logits = self.router.forward(h, out_dtype=torch.float32)
        weights = torch.empty_like(logits)
        ops.moe_route(logits, weights, self.groups, self.keep, self.top)
        return weights

    def forward(self, h, batch, residual, overwrite=False):
        weights = self.route(h)
        act = self.gate_up.forward_gated(h, self.gate_up.run)
        if act is None:
            act = torch.empty((h.shape[0], self.E * self.ff), dtype=self.dtype, device=h.device)
            ops.swiglu(self.gate_up.forward(h), act, self.gate_up.run)
        ops.moe_scale(act, weights, self.ff)
        if overwrite:
            self.down.forward(act, out=residual)
        else:
            self.down.forward(act, accumulate_into=residual)
        return residual


register_part("feed_forward", "routed_experts", RoutedExperts)
