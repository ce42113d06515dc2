"""The gated delta rule: a mixer whose memory of a sequence is a matrix per head instead of keys and values.

For a token with input h: q, k (``kv_heads`` heads of ``dim``) and v (``heads`` heads of ``vdim``) are projections of
h that pass a short causal convolution over time per channel (``conv`` taps, no bias, zeros before the sequence's
start) and SiLU; q and k heads are made unit vectors (x / sqrt(sum x^2 + 1e-6)), q is also multiplied by dim^-1/2;
head i reads q/k head i // (heads / kv_heads).  With beta = sigmoid(W_b h) and g = exp(-exp(A_log) softplus(W_a h +
dt_bias)) per head, the state S [dim, vdim] of a head goes

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

and the head's output is o / sqrt(mean(o^2) + eps) times a weight [vdim] shared by the heads, times SiLU(W_g h); the
heads side by side pass the output matrix.  Everything behind the projections is float32 in both paths; the six
projections are one product whose result is kept in float32.

What a sequence keeps between steps (one float32 region per slot, zero at its start): S for every head, then the
last ``conv - 1`` inputs of the convolved channels.

Options.  ``decay`` "channel": one decay per head and key channel instead of one per head, g [heads, dim] acting on the
rows of S that belong to key channels (``dt_bias`` is then [heads * dim], ``A_log`` stays [heads]).  ``decay_rank`` r: the
decay's projection is two matrices, W_a2 [.., r] (W_a1 [r, hidden] h).  ``gate_rank`` r: likewise the output gate,
W_g2 (W_g1 h).  ``gate_act`` "sigmoid" instead of "silu".  With a rank given, q, k, v and b are one product, the first halves
of the low-rank maps a second, and their second halves a third (block-diagonal); without, all six are one product.

Parameters: hidden_size, heads, kv_heads, dim, vdim, conv (None: no convolution and no tap tensors), norm_eps, decay
("head"), decay_rank (None), gate_rank (None), gate_act ("silu"); ``names``: the tensors' full names by role
(q, k, v, gate, b, a, q_conv, k_conv, v_conv, a_log, dt_bias, norm, o; with ranks: a1, a2, g1, g2 in place of a, gate).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateRequirement
from ..errors import require
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import BlockDiagonalLinear, DenseLinear

_UNIT_EPS = 1e-6


def bind_float32(weights, name: str, shape, ctx) -> torch.Tensor:
    """A small parameter that enters 32-bit arithmetic: on the device in float32 whatever it was stored in."""
    h = weights[name]
    require(tuple(h.shape) == tuple(shape),
            f"unexpected tensor shape for {name}: got {list(h.shape)}, expected {list(shape)}")
    return h.tensor.to(device=ctx.device, dtype=torch.float32).contiguous()


class GatedDeltaMixer:
    graph_safe = True        # slots and row ranges are read on the device; the launches depend on the counts alone
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.hidden = int(params["hidden_size"])
        self.H = int(params["heads"])
        self.KH = int(params.get("kv_heads") or self.H)
        self.D = int(params["dim"])
        self.V = int(params["vdim"])
        self.has_conv = params.get("conv") is not None       # no taps given: the channels pass straight to SiLU, no tensors
        self.taps = int(params.get("conv") or 1)
        self.eps = float(params["norm_eps"])
        require(self.H % self.KH == 0, f"{prefix}: {self.H} heads are not a multiple of {self.KH} query/key heads")
        require(self.D <= 256, f"{prefix}: a head size of {self.D} exceeds the recurrence kernel's 256")
        require(self.taps >= 1, f"{prefix}: the convolution needs at least one tap")
        self.channel_decay = str(params.get("decay") or "head") == "channel"
        require(str(params.get("decay") or "head") in ("head", "channel"), f"{prefix}: decay is 'head' or 'channel'")
        self.decay_rank = None if params.get("decay_rank") is None else int(params["decay_rank"])
        self.gate_rank = None if params.get("gate_rank") is None else int(params["gate_rank"])
        self.gate_act = str(params.get("gate_act") or "silu")
        require(self.gate_act in ("silu", "sigmoid"), f"{prefix}: gate_act is 'silu' or 'sigmoid'")
        require((self.decay_rank is None) == (self.gate_rank is None),
                f"{prefix}: the decay and the gate are either both low-rank or both full projections")
        require(not self.channel_decay or self.decay_rank is not None,
                f"{prefix}: a decay per key channel is built with a low-rank projection (decay_rank)")
        n = dict(params.get("names") or {})
        self.names = {r: str(n.get(r) or f"{prefix}.{r}") for r in
                      ("q", "k", "v", "gate", "b", "a", "a1", "a2", "g1", "g2", "q_conv", "k_conv", "v_conv", "a_log",
                       "dt_bias", "norm", "o")}
        self.prefix = prefix
        qk, hv = self.KH * self.D, self.H * self.V
        self.C = 2 * qk + hv                                  # convolved channels
        self.GD = self.D if self.channel_decay else 1         # decays a head
        nm = self.names
        if self.decay_rank is None:
            self.proj = DenseLinear([nm["q"], nm["k"], nm["v"], nm["gate"], nm["b"], nm["a"]],
                                    [qk, qk, hv, hv, self.H, self.H], self.hidden)
            self.low1 = self.low2 = None
        else:
            self.proj = DenseLinear([nm["q"], nm["k"], nm["v"], nm["b"]], [qk, qk, hv, self.H], self.hidden)
            self.low1 = DenseLinear([nm["a1"], nm["g1"]], [self.decay_rank, self.gate_rank], self.hidden)
            self.low2 = BlockDiagonalLinear([nm["a2"], nm["g2"]], [(self.H * self.GD, self.decay_rank), (hv, self.gate_rank)])
        self.o = DenseLinear([nm["o"]], [self.hidden], hv)
        self.state_floats = self.H * self.D * self.V + (self.taps - 1) * self.C

    def tensor_specs(self):
        nm, qk, hv = self.names, self.KH * self.D, self.H * self.V
        conv = [TensorSpec(nm["q_conv"], (qk, self.taps), "state"), TensorSpec(nm["k_conv"], (qk, self.taps), "state"),
                TensorSpec(nm["v_conv"], (hv, self.taps), "state")] if self.has_conv else []
        low = [] if self.low1 is None else self.low1.tensor_specs() + self.low2.tensor_specs()
        return self.proj.tensor_specs() + low + self.o.tensor_specs() + conv + [
            TensorSpec(nm["a_log"], (self.H,), "state"), TensorSpec(nm["dt_bias"], (self.H * self.GD,), "state"),
            TensorSpec(nm["norm"], (self.V,), "gain")]

    def cache_requirement(self):
        return StateRequirement((self.state_floats,), torch.float32)

    def bind(self, weights, ctx):
        nm, qk, hv = self.names, self.KH * self.D, self.H * self.V
        self.proj.bind(weights, ctx)
        self.o.bind(weights, ctx)
        if self.low1 is not None:
            self.low1.bind(weights, ctx)
            self.low2.bind(weights, ctx)
        if self.has_conv:
            self.conv_w = torch.cat([bind_float32(weights, nm["q_conv"], (qk, self.taps), ctx),
                                     bind_float32(weights, nm["k_conv"], (qk, self.taps), ctx),
                                     bind_float32(weights, nm["v_conv"], (hv, self.taps), ctx)], 0).contiguous()
        else:
            self.conv_w = torch.ones((self.C, 1), dtype=torch.float32, device=ctx.device)
        self.a_log = bind_float32(weights, nm["a_log"], (self.H,), ctx)
        self.dt_bias = bind_float32(weights, nm["dt_bias"], (self.H * self.GD,), ctx)
        self.norm_w = bind_float32(weights, nm["norm"], (self.V,), ctx)
        self.dtype = ctx.dtype

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(cache_view is not None and tuple(cache_view.requirement.shape) == (self.state_floats,),
                f"{self.prefix}: the delta rule needs its state region of {self.state_floats} floats a sequence")
        require(write_cache, f"{self.prefix}: a recurrent mixer cannot run without carrying its state")
        state = cache_view.storage                                  # [slots, state_floats]
        rows, hv = batch.rows, self.H * self.V
        proj = self.proj.forward(h, out_dtype=torch.float32)
        few = self.dtype == torch.bfloat16 and rows < 64
        prep = torch.empty((rows, self.C + self.H + self.H * self.GD), dtype=torch.float32, device=proj.device)
        if self.low1 is None:
            gate, gate_stride = proj[:, self.C:], proj.shape[1]
            ops.delta_prepare(proj, self.conv_w, state, self.H * self.D * self.V, batch.row_slot, batch.seq_start,
                              batch.seq_slot, batch.sequences, self.a_log, self.dt_bias, prep, self.H, self.KH, self.D,
                              self.V, _UNIT_EPS, block_a_segment=few)
        else:
            # the low-rank maps: [a1 h | g1 h] in the compute dtype, then both second halves in one block-diagonal product
            low = self.low2.forward(self.low1.forward(h), out_dtype=torch.float32)      # [rows, H GD | H V]
            gate, gate_stride = low[:, self.H * self.GD:], low.shape[1]
            ops.delta_prepare(proj, self.conv_w, state, self.H * self.D * self.V, batch.row_slot, batch.seq_start,
                              batch.seq_slot, batch.sequences, self.a_log, self.dt_bias, prep, self.H, self.KH, self.D,
                              self.V, _UNIT_EPS, block_a_segment=few, beta_col=self.C,
                              decay_in=low[:, :self.H * self.GD], channel_decay=self.channel_decay)
        o = torch.empty((rows, hv), dtype=torch.float32, device=proj.device)
        # bfloat16 steps take a sequence's rows two at a time; the 32-bit path keeps one order of operations for every cut
        ops.delta_rule(prep, state, batch.seq_start, batch.seq_slot, batch.sequences, self.H, self.KH, self.D, self.V, o,
                       pairs=self.dtype == torch.bfloat16,
                       mode=ops.DELTA_CHANNEL_DECAY if self.channel_decay else ops.DELTA_HEAD_DECAY)
        y = torch.empty((rows, hv), dtype=self.dtype, device=proj.device)
        ops.delta_output(o, gate, gate_stride, self.norm_w, y, self.H, self.V, self.eps, gate_act=self.gate_act)
        if overwrite:
            self.o.forward(y, out=residual)
        else:
            self.o.forward(y, accumulate_into=residual)
        return residual


register_part("mixer", "gated_delta", GatedDeltaMixer)
