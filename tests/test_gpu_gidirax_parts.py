"""Each new mechanism alone, built through the registries at sizes no model uses, against the plain implementation: the
norm on a sub-layer's output; the state-space mixer; the delta rule with a decay per key channel (and its other forms: a
decay per head behind low-rank maps); the gated linear recurrent unit; attention over a window with kept first tokens,
with one key made to stand out just inside and just outside every edge, in prompts, in decoding and over page borders;
the parallel pair; the router (groups, ties, top = experts) and the routed feed-forward.  Every mixer is run whole, token by
token and in portions through one state region or cache, so that what a sequence keeps between steps is tested alone."""
import math

import pytest
import torch

import citlali_b200 as cb
import plain_gidirax as plain
from citlali_b200 import ops
from citlali_b200.config.spec import PartSpec
from citlali_b200.engine.step import StepEntry, pack_step
from citlali_b200.parts.base import BuildContext, build_part
from citlali_b200.weights.loader import WeightHandle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def ctx_for(dtype):
    return BuildContext(torch.device(DEV), dtype, torch.zeros(4, dtype=torch.int32, device=DEV))


def handles(weights):
    return {n: WeightHandle(n, t.dtype, tuple(t.shape), tensor=t) for n, t in weights.items()}


def draw(specs, seed, scale=None):
    """Random bfloat16 weights for a part's tensors, sized so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in specs:
        r = torch.randn(tuple(s.shape), generator=g)
        n = s.name
        if s.role == "gain":
            t = 1.0 + 0.3 * r
        elif n.endswith(("conv", "q_conv", "k_conv", "v_conv")):
            t = 0.6 * r
        elif n.endswith("a_log"):
            t = -1.0 + 0.7 * r
        elif n.endswith("lam"):
            t = -1.5 + r
        elif n.endswith(("bias", "skip")) or len(s.shape) == 1:
            t = 0.5 * r + (1.0 if n.endswith("skip") else 0.0)
        else:
            t = r / s.shape[-1] ** 0.5
        out[n] = t.to(torch.bfloat16)
    return out


class Harness:
    """One mixer with a cache of its own: feeds a sequence in the given portions and returns the mixer's output rows."""

    def __init__(self, kind, params, dtype, weights=None, seed=1, slots=3, capacity=1024, max_seq=1024):
        self.part = build_part("mixer", PartSpec(kind, params, "m"))
        self.weights = weights if weights is not None else draw(self.part.tensor_specs(), seed)
        self.ctx = ctx_for(dtype)
        self.part.bind(handles(self.weights), self.ctx)
        self.cache = cb.SequenceCache([self.part.cache_requirement()], slots, capacity, max_seq, dtype, DEV)
        self.hidden = params["hidden_size"]
        self.dtype = dtype

    def run(self, sequences, portions):
        """``sequences``: {slot name: h [T, hidden] float64}; ``portions``: a list of steps, each {name: n new tokens}."""
        slots, done, out = {}, {}, {n: [] for n in sequences}
        for step in portions:
            names = [n for n in step if step[n] > 0]
            for n in names:
                if n not in slots:
                    slots[n] = self.cache.acquire()
                    done[n] = 0
            entries = [StepEntry(slots[n], [0] * step[n], []) for n in names]
            past = [done[n] for n in names]
            batch = pack_step(entries, past, 1, DEV)
            for n in names:
                self.cache.reserve(slots[n], done[n] + step[n])
            h = torch.cat([sequences[n][done[n]:done[n] + step[n]] for n in names]).to(DEV).to(self.dtype).contiguous()
            y = torch.empty((h.shape[0], self.hidden), dtype=torch.float32, device=DEV)
            self.part.forward(h, batch, self.cache.view(0), y, True, overwrite=True)
            at = 0
            for n in names:
                out[n].append(y[at:at + step[n]].double().cpu())
                at += step[n]
                done[n] += step[n]
                self.cache.commit(slots[n], done[n])
        for n in list(slots):
            self.cache.release(slots.pop(n))
        assert not any(self.ctx.error_flag.tolist())
        return {n: torch.cat(v) for n, v in out.items()}


def inputs(T, hidden, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, hidden, generator=g).to(torch.bfloat16).double()       # what both paths read exactly


def close(got, want, dtype, what):
    scale = float(want.abs().max())
    err = float((got - want).abs().max())
    assert err <= TOL[dtype] * scale, f"{what}: |diff| {err:.3e} of {scale:.3e}"


def cuts(T):
    """Ways of feeding T tokens of sequence 'a': whole, one by one, portions of two (and a last odd one), mixed."""
    two = [{"a": 2}] * (T // 2) + ([{"a": 1}] if T % 2 else [])
    mixed, left = [], T
    for n in (3, 1, 7, 2, 64, 5, 1, 1, 40):
        if left <= 0:
            break
        mixed.append({"a": min(n, left)})
        left -= min(n, left)
    if left:
        mixed.append({"a": left})
    return {"whole": [{"a": T}], "one by one": [{"a": 1}] * T, "twos": two, "mixed": mixed}


def run_all_cuts(kind, params, plain_fn, dtype, T=90, seed=3):
    h = inputs(T, params["hidden_size"], seed)
    hs = Harness(kind, params, dtype, seed=seed)
    want = plain_fn(h, hs.weights)
    results = {}
    for what, portions in cuts(T).items():
        results[what] = hs.run({"a": h}, portions)["a"]
        close(results[what], want, dtype, f"{kind} {dtype} {what}")
    if dtype == torch.float32:
        for what in results:
            assert torch.equal(results[what], results["whole"]), f"{kind}: '{what}' gives other bits than 'whole'"
    # two unequal sequences in one batch, a third that takes a slot which was given back
    other = inputs(37, params["hidden_size"], seed + 1)
    both = hs.run({"a": h, "b": other}, [{"a": 50, "b": 20}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": T - 52, "b": 15}])
    close(both["a"], want, dtype, f"{kind} {dtype} batched a")
    close(both["b"], plain_fn(other, hs.weights), dtype, f"{kind} {dtype} batched b")
    again = hs.run({"c": other}, [{"c": 37}])["c"]                  # the slot's state region and pages were used before
    close(again, plain_fn(other, hs.weights), dtype, f"{kind} {dtype} reused slot")


# ---- the norm on a sub-layer's output -------------------------------------------------------------------------------

@pytest.mark.parametrize("hidden", [60, 256, 1000])
def test_layer_norm_add_and_rows(hidden):
    g = torch.Generator().manual_seed(hidden)
    y = (3.0 * torch.randn(7, hidden, generator=g) + 2.0).to(DEV)
    x = torch.randn(7, hidden, generator=g).to(DEV)
    w = (1.0 + 0.3 * torch.randn(hidden, generator=g)).to(DEV)
    want = x.double().cpu() + plain.layer_norm(y.double().cpu(), w.cpu(), 1e-5)
    emit = torch.empty((7, hidden), dtype=torch.bfloat16, device=DEV)
    x2 = x.clone()
    ops.layer_norm_add(y, w, 1e-5, x2, emit)
    assert float((x2.double().cpu() - want).abs().max()) < 1e-5
    assert torch.equal(emit, x2.to(torch.bfloat16))
    idx = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out = torch.empty((3, hidden), dtype=torch.float32, device=DEV)
    ops.layer_norm_rows(y, w, 1e-5, out, idx)
    assert float((out.double().cpu() - plain.layer_norm(y.double().cpu()[[5, 0, 5]], w.cpu(), 1e-5)).abs().max()) < 1e-5


# ---- mixers with a state ----------------------------------------------------------------------------------------------

SSM = [dict(hidden_size=40, heads=3, vdim=12, state=20, groups=1, norm_groups=1, conv=4, norm_eps=1e-5),
       dict(hidden_size=64, heads=4, vdim=40, state=72, groups=2, norm_groups=4, conv=2, norm_eps=1e-6),
       dict(hidden_size=32, heads=2, vdim=8, state=130, groups=2, norm_groups=2, conv=None, norm_eps=1e-5)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", SSM)
def test_state_space_mixer(params, dtype):
    m = {k: params[k] for k in ("heads", "vdim", "state", "groups", "norm_groups", "conv")}
    names = {"m.in": "p.in", "m.conv": "p.conv", "m.conv_bias": "p.conv.b", "m.dt_bias": "p.dt_bias", "m.a_log": "p.A_log",
             "m.skip": "p.D", "m.norm": "p.norm", "m.o": "p.o"}
    fn = lambda h, w: plain.mamba2_mixer(h, {names[k]: v for k, v in w.items()}, "p", m, params["norm_eps"])
    run_all_cuts("state_space", params, fn, dtype)


DELTA = [dict(hidden_size=48, heads=4, kv_heads=2, dim=20, vdim=12, conv=3, norm_eps=1e-5, decay="channel", decay_rank=8,
              gate_rank=16, gate_act="sigmoid"),
         dict(hidden_size=40, heads=2, kv_heads=2, dim=72, vdim=40, conv=None, norm_eps=1e-6, decay="channel", decay_rank=4,
              gate_rank=4, gate_act="sigmoid"),
         dict(hidden_size=32, heads=3, kv_heads=1, dim=136, vdim=8, conv=2, norm_eps=1e-5, decay="channel", decay_rank=8,
              gate_rank=8, gate_act="sigmoid")]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", DELTA)
def test_delta_rule_with_channel_decay(params, dtype):
    m = {k: params[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
    names = {"m.q": "p.q", "m.k": "p.k", "m.v": "p.v", "m.b": "p.b", "m.a1": "p.a1", "m.a2": "p.a2", "m.g1": "p.g1",
             "m.g2": "p.g2", "m.q_conv": "p.q.conv", "m.k_conv": "p.k.conv", "m.v_conv": "p.v.conv", "m.a_log": "p.A_log",
             "m.dt_bias": "p.dt_bias", "m.norm": "p.norm", "m.o": "p.o"}
    fn = lambda h, w: plain.channel_delta_mixer(h, {names[k]: v for k, v in w.items()}, "p", m, params["norm_eps"])
    run_all_cuts("gated_delta", params, fn, dtype)


def test_delta_rule_remembers_a_far_write():
    """One write far back, read 500 tokens later: keys orthogonal to it in between, decays close to one.  The read-out must
    be the written value times the product of the key channel's decays; a state lost or reset on the way shows as zero."""
    H, D, V, T = 1, 32, 16, 520
    C = 2 * D + V
    prep = torch.zeros(T, C + H + H * D, dtype=torch.float32)
    g = torch.Generator().manual_seed(5)
    decay = 1.0 - 0.002 * torch.rand(T, D, generator=g)
    prep[:, C + H:] = decay
    prep[:, C] = 1.0                                        # beta
    e = torch.eye(D)
    prep[:, D:2 * D] = e[1 + torch.arange(T) % (D - 1)]     # keys: unit vectors that never touch channel 0 ...
    prep[7, D:2 * D] = e[0]                                 # ... except the write at token 7
    value = torch.randn(V, generator=g)
    prep[7, 2 * D:2 * D + V] = value
    prep[T - 1, :D] = e[0]                                  # the last token asks for channel 0
    want = value.double() * decay[8:, 0].double().prod()
    state = torch.zeros(1, H * D * V, dtype=torch.float32, device=DEV)
    for cut in ([T], [300, T - 300], [T - 1, 1]):
        state.zero_()
        outs, at = [], 0
        for n in cut:
            o = torch.empty(n, H * V, dtype=torch.float32, device=DEV)
            ops.delta_rule(prep[at:at + n].contiguous().to(DEV), state, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                           torch.zeros(1, dtype=torch.int32, device=DEV), 1, H, 1, D, V, o, mode=ops.DELTA_CHANNEL_DECAY)
            outs.append(o)
            at += n
        got = torch.cat(outs)[-1].double().cpu()
        assert float((got - want).abs().max()) < 1e-5 * float(want.abs().max()), cut


LRU = [dict(hidden_size=40, width=48, blocks=3, conv=4), dict(hidden_size=64, width=80, blocks=1, conv=None),
       dict(hidden_size=32, width=264, blocks=2, conv=2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", LRU)
def test_gated_recurrent_mixer(params, dtype):
    m = {k: params[k] for k in ("width", "blocks", "conv")}
    names = {"m.y": "p.y", "m.y_bias": "p.y.b", "m.x": "p.x", "m.x_bias": "p.x.b", "m.conv": "p.conv", "m.conv_bias": "p.conv.b",
             "m.gate_a": "p.ra", "m.gate_a_bias": "p.ra.b", "m.gate_i": "p.ri", "m.gate_i_bias": "p.ri.b", "m.lam": "p.lam",
             "m.o": "p.o"}
    fn = lambda h, w: plain.recurrent_block_mixer(h, {names[k]: v for k, v in w.items()}, "p", m, 0.0)
    run_all_cuts("gated_recurrent", params, fn, dtype)


# ---- attention over a window with kept first tokens -----------------------------------------------------------------

ATT = [dict(hidden_size=48, heads=4, kv_heads=2, dim=16, vdim=24, conv=3, qk_norm_eps=1e-5, rot_dims=8, rot_base=1e4,
            scale=0.25, window=9, keep_first=2),
       dict(hidden_size=40, heads=3, kv_heads=3, dim=80, vdim=12, conv=None, qk_norm_eps=1e-6, rot_dims=80, rot_base=5e5,
            scale=0.11, window=65, keep_first=5),
       dict(hidden_size=32, heads=2, kv_heads=1, dim=24, vdim=40, conv=4, qk_norm_eps=1e-5, rot_dims=0, rot_base=1.0,
            scale=0.2, window=None, keep_first=0),
       dict(hidden_size=32, heads=2, kv_heads=2, dim=8, vdim=8, conv=2, qk_norm_eps=1e-5, rot_dims=4, rot_base=1e2,
            scale=0.35, window=1, keep_first=70),
       # keys and values of one size that the tensor-core kernel for runs of tokens takes (bfloat16)
       dict(hidden_size=48, heads=4, kv_heads=2, dim=32, vdim=32, conv=2, qk_norm_eps=1e-5, rot_dims=16, rot_base=1e4,
            scale=0.18, window=70, keep_first=3),
       dict(hidden_size=32, heads=2, kv_heads=1, dim=16, vdim=16, conv=None, qk_norm_eps=1e-5, rot_dims=16, rot_base=1e3,
            scale=0.25, window=9, keep_first=130),
       dict(hidden_size=64, heads=2, kv_heads=2, dim=64, vdim=64, conv=3, qk_norm_eps=1e-6, rot_dims=32, rot_base=1e4,
            scale=0.125, window=None, keep_first=0)]


def attention_plain(params):
    m = {"heads": params["heads"], "kv_heads": params["kv_heads"], "dim": params["dim"], "vdim": params["vdim"],
         "conv": params["conv"], "scale": params["scale"]}
    if params["window"] is not None:
        m["mask"] = {"size": params["window"], "keep_first": params["keep_first"]}
    if params["rot_dims"]:
        m["rot"] = {"dims": params["rot_dims"], "base": params["rot_base"]}
    names = {"m.q": "p.q", "m.k": "p.k", "m.v": "p.v", "m.q_conv": "p.q.conv", "m.k_conv": "p.k.conv", "m.v_conv": "p.v.conv",
             "m.q_norm": "p.q.norm", "m.k_norm": "p.k.norm", "m.o": "p.o"}
    return lambda h, w: plain.window_attention_mixer(h, {names[k]: v for k, v in w.items()}, "p", m, params["qk_norm_eps"])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("params", ATT)
def test_window_attention_mixer(params, dtype):
    run_all_cuts("window_attention", params, attention_plain(params), dtype, T=150)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode_from", [None, 40])
@pytest.mark.parametrize("window,keep_first", [(9, 2), (64, 4), (65, 1), (130, 0), (1, 3), (20, 70)])
def test_window_edges_with_one_key_that_stands_out(window, keep_first, decode_from, dtype):
    """Queries and keys are the inputs themselves (identity projections, no norm, no rotation, one tap); one key is made
    twenty times longer than the rest and every later query points along it, so a row's output is that key's value exactly
    when the key is visible: just inside and just outside the window, at the kept tokens' edge, over page borders."""
    d, T = 16, 210
    params = dict(hidden_size=d, heads=1, kv_heads=1, dim=d, vdim=d, conv=None, qk_norm_eps=None, rot_dims=0, scale=1.0,
                  window=window, keep_first=keep_first)
    eye = torch.eye(d).to(torch.bfloat16)
    weights = {"m.q": eye, "m.k": eye, "m.v": eye, "m.o": eye}
    # (in bfloat16 a prompt of this head size runs the tensor-core kernel for runs of tokens)
    for special in (0, keep_first - 1, keep_first, 63, 64, 100):
        if special < 0:
            continue
        g = torch.Generator().manual_seed(special)
        h = (0.1 * torch.randn(T, d, generator=g))
        h[:, 0] = 1.0                                       # every query has a part along the first axis ...
        h[special, 0] = 20.0                                # ... and one key is long along it
        h = h.to(torch.bfloat16).double()
        hs = Harness("window_attention", params, dtype, weights=weights)
        portions = [{"a": T}] if decode_from is None else [{"a": decode_from}] + [{"a": 1}] * (T - decode_from)
        got = hs.run({"a": h}, portions)["a"]
        see = plain.visible(T, window, keep_first)
        for i in range(T):
            s = (h[i] @ h[:i + 1].T).masked_fill(~see[i, :i + 1], -math.inf)
            ref = torch.softmax(s, -1) @ h[:i + 1]
            assert float((got[i] - ref).abs().max()) < (1e-4 if dtype == torch.float32 else 0.15), (window, keep_first, special, i)
            if i > special:                                 # the test's point: the special key decides the row
                visible_now = bool(see[i, special])
                assert (float(got[i][0]) > 10.0) == visible_now, (window, keep_first, special, i)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,keep_first", [(None, 0), (40, 6)])
def test_a_far_key_among_hundreds(window, keep_first, dtype):
    """One long key at position 3 among 900 ordinary ones, over fourteen pages: every later row must find it (without a
    window, or as one of the kept first tokens) whether it comes in the prompt, in a later portion or token by token."""
    d, T = 32, 900
    params = dict(hidden_size=d, heads=2, kv_heads=1, dim=d // 2, vdim=d // 2, conv=None, qk_norm_eps=None, rot_dims=0,
                  scale=1.0, window=window, keep_first=keep_first)
    eye = torch.eye(d).to(torch.bfloat16)
    weights = {"m.q": eye, "m.k": eye[:d // 2], "m.v": eye[d // 2:], "m.o": eye}
    g = torch.Generator().manual_seed(11)
    h = 0.1 * torch.randn(T, d, generator=g)
    h[:, 0] = 1.0
    h[:, d // 2] = 1.0                                       # both query heads look along the first key axis
    h[3, 0] = 20.0
    h[3, d // 2:] = 7.0                                      # the far token's value
    h = h.to(torch.bfloat16).double()
    hs = Harness("window_attention", params, dtype, weights=weights, capacity=1024)
    for portions in ([{"a": T}], [{"a": 500}, {"a": 300}] + [{"a": 1}] * 100, [{"a": 2}] * 450):
        got = hs.run({"a": h}, portions)["a"]
        assert float((got[10:] - 7.0).abs().max()) < (1e-3 if dtype == torch.float32 else 0.1), len(portions)


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_pair(dtype):
    left = dict(ATT[0])
    right = dict(LRU[0], hidden_size=48)
    params = {"hidden_size": 48, "left": {"kind": "window_attention", "params": left, "prefix": "m.left"},
              "right": {"kind": "gated_recurrent", "params": right, "prefix": "m.right"}, "left_scale": 1.3, "right_scale": 0.6}
    lp, rp = attention_plain(left), None
    names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b", "gate_a": "ra",
             "gate_a_bias": "ra.b", "gate_i": "ri", "gate_i_bias": "ri.b", "lam": "lam", "o": "o"}

    def fn(h, w):
        lw = {"m." + k[len("m.left."):]: v for k, v in w.items() if k.startswith("m.left.")}
        rw = {"p." + names[k[len("m.right."):]]: v for k, v in w.items() if k.startswith("m.right.")}
        r = plain.recurrent_block_mixer(h, rw, "p", {"width": right["width"], "blocks": right["blocks"], "conv": right["conv"]}, 0.0)
        return 1.3 * lp(h, lw) + 0.6 * r
    run_all_cuts("parallel", params, fn, dtype)


# ---- routed experts ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("E,top,count,keep", [(16, 4, 4, 3), (8, 2, None, None), (6, 6, 3, 3), (12, 3, 12, 5), (40, 5, 5, 1),
                                              (64, 8, 8, 4), (5, 1, 1, 1)])
def test_router_against_plain(E, top, count, keep):
    g = torch.Generator().manual_seed(E * 7 + top)
    logits = 2.0 * torch.randn(300, E, generator=g)
    weights = torch.empty(300, E, device=DEV)
    chosen = torch.empty(300, top, dtype=torch.int32, device=DEV)
    ops.moe_route(logits.to(DEV), weights, count, keep, top, chosen)
    s = torch.softmax(logits.double(), -1)
    want = plain.route(s, top, count, keep if keep is not None else 1)
    for r in range(300):
        assert sorted(chosen[r].tolist()) == sorted(want[r].tolist()), r
        row = weights[r].double().cpu()
        assert int((row != 0).sum()) == top
        assert float((row[want[r]] - s[r, want[r]]).abs().max()) < 1e-6


def test_router_ties_go_to_the_lower_index():
    logits = torch.zeros(2, 8, device=DEV)
    weights = torch.empty(2, 8, device=DEV)
    chosen = torch.empty(2, 3, dtype=torch.int32, device=DEV)
    ops.moe_route(logits, weights, 4, 2, 3, chosen)
    assert chosen.tolist() == [[0, 1, 2], [0, 1, 2]]
    assert torch.allclose(weights[0].cpu(), torch.tensor([0.125] * 3 + [0.0] * 5))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,count,keep,hidden", [(8, 2, 32, 4, 2, 64), (5, 2, 24, None, None, 60), (4, 4, 16, 4, 4, 32),
                                                        (16, 4, 48, 4, 3, 128)])
def test_routed_feed_forward(E, top, ff, count, keep, hidden, dtype):
    params = {"hidden_size": hidden, "experts": E, "top": top, "intermediate_size": ff, "groups": count, "keep_groups": keep}
    part = build_part("feed_forward", PartSpec("routed_experts", params, "f"))
    w = draw(part.tensor_specs(), E)
    w["f.router"] = (3.0 * w["f.router"].float()).to(torch.bfloat16)
    part.bind(handles(w), ctx_for(dtype))
    h = inputs(70, hidden, 9)
    mlp = {"expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    if count is not None:
        mlp["router"]["groups"] = {"count": count, "keep": keep}
    want = plain.moe_feed_forward(h, {k.replace("f.", "p.", 1): v for k, v in w.items()}, "p", mlp)
    y = torch.empty((70, hidden), dtype=torch.float32, device=DEV)
    part.forward(h.to(DEV).to(dtype), None, y, overwrite=True)
    close(y.double().cpu(), want, dtype, f"routed experts {dtype}")
    y2 = torch.ones_like(y)
    part.forward(h.to(DEV).to(dtype), None, y2)                       # the adding form
    close(y2.double().cpu() - 1.0, want, dtype, "routed experts, added")
