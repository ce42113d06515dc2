"""A recurrent block around a real-gated linear recurrent unit.

Two branches of ``width`` channels read the input h:  y = gelu_tanh(W_y h + b_y)  and  u = conv(W_x h + b_x), a short causal
convolution over time per channel with a bias and no activation.  u is cut into ``blocks`` equal parts; in part b, with
square matrices [out, in]:  r = sigmoid(Wa_b u_b + ba_b),  i = sigmoid(Wi_b u_b + bi_b).  Then per channel

    log a = -8 r softplus(lam);   a = exp(log a);   S <- a S + sqrt(1 - a^2) i u      (S = 0 before the first token)

and the block gives W_o (S * y).  The gates, the decay and the state are float32 in both paths (the gate matrices are kept
in float32, transposed for the kernel); the two branch projections are one product whose result stays float32.

A sequence keeps, in one float32 region: S, then the last ``conv - 1`` inputs of the convolution (bias included).

Parameters: hidden_size, width, blocks, conv (None: none); ``names``: full tensor names by role (y, y_bias, x, x_bias, conv,
conv_bias, gate_a, gate_a_bias, gate_i, gate_i_bias, lam, o).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import register_part
from .delta import bind_float32
from .linear import DenseLinear

_ROLES = ("y", "y_bias", "x", "x_bias", "conv", "conv_bias", "gate_a", "gate_a_bias", "gate_i", "gate_i_bias", "lam", "o")


class GatedRecurrentMixer:
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.blocks = int(params.get("blocks") or 1)
        self.has_conv = params.get("conv") is not None
        self.taps = int(params.get("conv") or 1)
        require(self.width % self.blocks == 0, f"{prefix}: a width of {self.width} does not split into {self.blocks} blocks")
        n = dict(params.get("names") or {})
        self.names = {r: str(n.get(r) or f"{prefix}.{r}") for r in _ROLES}
        self.prefix = prefix
        self.branches = DenseLinear([self.names["y"], self.names["x"]], [self.width, self.width], self.hidden)
        self.o = DenseLinear([self.names["o"]], [self.hidden], self.width)
        self.state_floats = self.width * self.taps

    def tensor_specs(self):
        nm, w, b = self.names, self.width, self.blocks
        bw = w // b
        conv = [TensorSpec(nm["conv"], (w, self.taps), "state"), TensorSpec(nm["conv_bias"], (w,), "state")] if self.has_conv else []
        return self.branches.tensor_specs() + self.o.tensor_specs() + conv + [
            TensorSpec(nm["y_bias"], (w,), "state"), TensorSpec(nm["x_bias"], (w,), "state"),
            TensorSpec(nm["gate_a"], (b, bw, bw), "state"), TensorSpec(nm["gate_a_bias"], (b, bw), "state"),
            TensorSpec(nm["gate_i"], (b, bw, bw), "state"), TensorSpec(nm["gate_i_bias"], (b, bw), "state"),
            TensorSpec(nm["lam"], (w,), "state")]

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def bind(self, weights, ctx):
        nm, w, b = self.names, self.width, self.blocks
        bw = w // b
        self.branches.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.has_conv:
            self.conv_w = bind_float32(weights, nm["conv"], (w, self.taps), ctx)
            self.conv_b = bind_float32(weights, nm["conv_bias"], (w,), ctx)
        else:
            self.conv_w = torch.ones((w, 1), dtype=torch.float32, device=ctx.device)
            self.conv_b = None
        self.y_b = bind_float32(weights, nm["y_bias"], (w,), ctx)
        self.x_b = bind_float32(weights, nm["x_bias"], (w,), ctx)
        # [block, out, in] as stored -> [block, in, out]: neighbouring threads (outputs) read neighbouring words
        self.wa_t = bind_float32(weights, nm["gate_a"], (b, bw, bw), ctx).transpose(1, 2).contiguous()
        self.wi_t = bind_float32(weights, nm["gate_i"], (b, bw, bw), ctx).transpose(1, 2).contiguous()
        self.ba = bind_float32(weights, nm["gate_a_bias"], (b, bw), ctx).reshape(w).contiguous()
        self.bi = bind_float32(weights, nm["gate_i_bias"], (b, bw), ctx).reshape(w).contiguous()
        self.lam = bind_float32(weights, nm["lam"], (w,), ctx)
        self.dtype = ctx.dtype

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(cache_view is not None and tuple(cache_view.requirement.shape) == (self.state_floats,),
                f"{self.prefix}: the recurrent block needs its state region of {self.state_floats} floats a sequence")
        require(write_cache, f"{self.prefix}: a recurrent mixer cannot run without carrying its state")
        state = cache_view.storage
        rows, w = batch.rows, self.width
        proj = self.branches.forward(h, out_dtype=torch.float32)           # [rows, y | x]
        u = torch.empty((rows, w), dtype=torch.float32, device=proj.device)
        ops.causal_conv(proj[:, w:], 2 * w, self.conv_w, state, w, batch, u, in_bias=self.x_b, bias=self.conv_b)
        a = torch.empty_like(u)
        coef = torch.empty_like(u)
        ops.lru_gates(u, self.wa_t, self.ba, self.wi_t, self.bi, self.lam, a, coef, self.blocks)
        out = torch.empty((rows, w), dtype=self.dtype, device=proj.device)
        ops.gated_scan(a, coef, proj, 2 * w, self.y_b, state, 0, batch, out)
        if overwrite:
            self.o.forward(out, out=residual)
        else:
            self.o.forward(out, accumulate_into=residual)
        return residual


register_part("mixer", "gated_recurrent", GatedRecurrentMixer)
