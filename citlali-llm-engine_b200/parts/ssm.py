"""A state-space mixer (the "state-space duality" form): a matrix of state per head that decays by one factor a token.

For a token with input h, one projection gives  z (inner) | x (inner) | B (G N) | C (G N) | dt (H), inner = H P.  x, B and
C together pass a short causal convolution over time per channel (with a bias) and SiLU; dt <- softplus(dt + dt_bias).
Head i (P channels of x; the B and C of group i // (H / G)) keeps S [N, P], zero at a sequence's start:

    S <- exp(-exp(A_log_i) dt) S + dt B x^T;    y = S^T C + D_i x.

y, all heads side by side, is multiplied by silu(z), divided by the root mean square of each of ``norm_groups`` equal parts
of the row (the gate comes before the norm), multiplied by a weight, and passes the output matrix.

The recurrence is the delta rule's without its correction term (keys B, queries C, values x, write strength dt) and runs
in that kernel; the preparation and the output stage are kernels of their own.  Everything behind the projection is
float32 in both paths.  A sequence keeps, in one float32 region: S of every head, then the last ``conv - 1`` inputs of
the convolved channels.

Parameters: hidden_size, heads, vdim, state, groups, norm_groups, conv (None: no convolution, no tap tensors), norm_eps;
``names``: full tensor names by role (in, conv, conv_bias, dt_bias, a_log, skip, norm, o).
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


class StateSpaceMixer:
    graph_safe = True
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.H, self.P, self.N = int(params["heads"]), int(params["vdim"]), int(params["state"])
        self.G = int(params.get("groups") or 1)
        self.NG = int(params.get("norm_groups") or 1)
        self.has_conv = params.get("conv") is not None
        self.taps = int(params.get("conv") or 1)
        self.eps = float(params["norm_eps"])
        self.inner = self.H * self.P
        require(self.H % self.G == 0, f"{prefix}: {self.H} heads are not a multiple of {self.G} groups")
        require(self.inner % self.NG == 0, f"{prefix}: {self.inner} channels do not split into {self.NG} norm groups")
        require(self.N <= 256, f"{prefix}: a state of {self.N} exceeds the recurrence kernel's 256")
        n = dict(params.get("names") or {})
        self.names = {r: str(n.get(r) or f"{prefix}.{r}") for r in
                      ("in", "conv", "conv_bias", "dt_bias", "a_log", "skip", "norm", "o")}
        self.prefix = prefix
        self.Cc = self.inner + 2 * self.G * self.N
        self.in_proj = DenseLinear([self.names["in"]], [self.inner + self.Cc + self.H], self.hidden)
        self.o = DenseLinear([self.names["o"]], [self.hidden], self.inner)
        self.state_floats = self.H * self.N * self.P + (self.taps - 1) * self.Cc

    def tensor_specs(self):
        nm = self.names
        conv = [TensorSpec(nm["conv"], (self.Cc, self.taps), "state"),
                TensorSpec(nm["conv_bias"], (self.Cc,), "state")] if self.has_conv else []
        return self.in_proj.tensor_specs() + self.o.tensor_specs() + conv + [
            TensorSpec(nm["dt_bias"], (self.H,), "state"), TensorSpec(nm["a_log"], (self.H,), "state"),
            TensorSpec(nm["skip"], (self.H,), "state"), TensorSpec(nm["norm"], (self.inner,), "gain")]

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def bind(self, weights, ctx):
        nm = self.names
        self.in_proj.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.has_conv:
            self.conv_w = bind_float32(weights, nm["conv"], (self.Cc, self.taps), ctx)
            self.conv_b = bind_float32(weights, nm["conv_bias"], (self.Cc,), ctx)
        else:
            self.conv_w = torch.ones((self.Cc, 1), dtype=torch.float32, device=ctx.device)
            self.conv_b = None
        self.dt_bias = bind_float32(weights, nm["dt_bias"], (self.H,), ctx)
        self.a_log = bind_float32(weights, nm["a_log"], (self.H,), ctx)
        self.skip = bind_float32(weights, nm["skip"], (self.H,), ctx)
        self.norm_w = bind_float32(weights, nm["norm"], (self.inner,), ctx)
        self.dtype = ctx.dtype

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(cache_view is not None and tuple(cache_view.requirement.shape) == (self.state_floats,),
                f"{self.prefix}: the state-space mixer needs its state region of {self.state_floats} floats a sequence")
        require(write_cache, f"{self.prefix}: a recurrent mixer cannot run without carrying its state")
        state = cache_view.storage
        rows, H, P, G, N = batch.rows, self.H, self.P, self.G, self.N
        proj = self.in_proj.forward(h, out_dtype=torch.float32)
        prep = torch.empty((rows, self.Cc + 2 * H), dtype=torch.float32, device=proj.device)
        ops.ssm_prepare(proj, self.conv_w, self.conv_b, state, H * N * P, batch, self.a_log, self.dt_bias, prep, H, P, G, N)
        o = torch.empty((rows, self.inner), dtype=torch.float32, device=proj.device)
        ops.delta_rule(prep, state, batch.seq_start, batch.seq_slot, batch.sequences, H, G, N, P, o,
                       mode=ops.DELTA_NO_CORRECTION)
        y = torch.empty((rows, self.inner), dtype=self.dtype, device=proj.device)
        ops.ssm_output(o, prep, 2 * G * N, proj, self.skip, self.norm_w, y, H, P, self.NG, self.eps)
        if overwrite:
            self.o.forward(y, out=residual)
        else:
            self.o.forward(y, accumulate_into=residual)
        return residual


register_part("mixer", "state_space", StateSpaceMixer)
