"""The mechanisms of the Lanizen decoder one at a time: parts built through the registries and kernels called alone,
at sizes no model here uses, against the plain implementation's function for the mechanism.  Where random numbers
would hide a fault, the inputs are made so that it shows: one key far back whose score stands out, keys just inside
and just outside a window in shuffled pages, a sink that takes all or none of the weight, a memory written once and
read hundreds of tokens later."""
import math

import pytest
import torch

import citlali_b200 as cb
import plain_lanizen as plain
from citlali_b200 import ops
from citlali_b200.cache import KVRequirement, SequenceCache
from citlali_b200.engine.step import StepEntry, pack_step
from citlali_b200.parts import BuildContext, part_class
from citlali_b200.weights.loader import WeightHandle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def ctx_for(dtype):
    return BuildContext(DEV, dtype, torch.zeros(4, dtype=torch.int32, device=DEV))


def weights_for(part, seed, special=None):
    """bfloat16-representable values for every tensor the part names: matrices of unit-scale rows, the rest by name."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for spec in part.tensor_specs():
        r = torch.randn(tuple(spec.shape), generator=g)
        if special and any(spec.name.endswith(k) for k in special):
            t = next(f for k, f in special.items() if spec.name.endswith(k))(r)
        elif spec.role == "matrix":
            t = r / spec.shape[1] ** 0.5
        else:
            t = 0.5 * r
        w[spec.name] = t.to(torch.bfloat16).float()
    return w


def handles(w, dtype):
    return {n: WeightHandle(n, dtype, tuple(t.shape), t.to(dtype)) for n, t in w.items()}


def close(got, want, dtype, f32=2e-5, bf16=3e-2):
    scale = float(want.abs().max())
    err = float((got.double().cpu() - want).abs().max())
    assert err <= (f32 if dtype == torch.float32 else bf16) * scale, f"|diff| {err:.3e} against scale {scale:.3e}"


def run_steps(mixer, cache, hidden, steps, dtype):
    """``steps``: lists of (slot, rows [n, hidden]).  Returns {slot: every output row so far}."""
    out = {}
    for step in steps:
        entries = [StepEntry(slot, [0] * x.shape[0]) for slot, x in step]
        past = [cache.length(slot) for slot, _ in step]
        batch = pack_step(entries, past, 10, DEV)
        for (slot, x), p in zip(step, past):
            cache.reserve(slot, p + x.shape[0])
        h = torch.cat([x for _, x in step]).to(DEV, dtype)
        y = torch.zeros((h.shape[0], hidden), dtype=torch.float32, device=DEV)
        mixer.forward(h, batch, cache.view(0), y, True)
        at = 0
        for (slot, x), p in zip(step, past):
            cache.commit(slot, p + x.shape[0])
            out.setdefault(slot, []).append(y[at:at + x.shape[0]].cpu())
            at += x.shape[0]
    return {slot: torch.cat(rows) for slot, rows in out.items()}


# ---- norm, feed-forward, streams ----------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_with_offset_and_named_tensor(dtype):
    norm = part_class("norm", "rms_norm")({"size": 70, "eps": 1e-4, "offset": 1.0, "tensor": "blk.n1"}, "ignored")
    assert [t.name for t in norm.tensor_specs()] == ["blk.n1"]
    w = {"blk.n1": (0.01 * torch.randn(70)).to(torch.bfloat16).float()}       # 1 + w would lose w in bfloat16
    norm.bind(handles(w, torch.bfloat16), ctx_for(dtype))
    assert norm.gain.dtype == torch.float32
    x = torch.randn(5, 70) * 3
    close(norm.forward(x.to(DEV)), plain.offset_norm(x.double(), w["blk.n1"], 1e-4), dtype, bf16=5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [48, 50])
def test_squared_relu_feed_forward(dtype, inter):
    ff = part_class("feed_forward", "relu_squared")({"hidden_size": 40, "intermediate_size": inter,
                                                     "up": "f.up", "down": "f.down"}, "f")
    w = weights_for(ff, 3)
    ff.bind(handles(w, dtype), ctx_for(dtype))
    x = torch.randn(7, 40).to(torch.bfloat16).float()
    want = plain.dense_feed_forward(x.double(), w, "f")
    res = torch.randn(7, 40)
    close(ff.forward(x.to(DEV, dtype), None, res.to(DEV).clone()), res.double() + want, dtype)
    junk = torch.full((7, 40), 1e9, device=DEV)
    close(ff.forward(x.to(DEV, dtype), None, junk, overwrite=True), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S, width", [(1, 64), (3, 70), (8, 33)])
def test_stream_kernels(dtype, S, width):
    rows = 9
    X = torch.randn(S, rows, width)
    w_in, w_out, w_mix, gain = torch.randn(S), torch.randn(S), torch.randn(S, S), 1 + 0.3 * torch.randn(width)
    h = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.hyper_read_norm(X.to(DEV), w_in.to(DEV), gain.to(DEV), 1e-5, h)
    close(h, plain.rms_normalise(plain.hyper_read(X.double(), w_in), 1e-5) * gain.double(), dtype, bf16=5e-3)
    y = torch.randn(rows, width)
    Xd = X.to(DEV).clone()
    ops.hyper_write(Xd, y.to(DEV), w_mix.to(DEV), w_out.to(DEV))
    close(Xd, plain.hyper_write(X.double(), y.double(), w_mix, w_out), torch.float32)
    # the write-back and the next read in one pass: the same bits as the two kernels one after the other
    w_in2 = torch.randn(S)
    Xf, h2, h2f = X.to(DEV).clone(), torch.empty_like(h), torch.empty_like(h)
    ops.hyper_write_read_norm(Xf, y.to(DEV), w_mix.to(DEV), w_out.to(DEV), w_in2.to(DEV), gain.to(DEV), 1e-5, h2f)
    ops.hyper_read_norm(Xd, w_in2.to(DEV), gain.to(DEV), 1e-5, h2)
    assert torch.equal(Xf, Xd) and torch.equal(h2f, h2)
    idx = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(3, width, device=DEV)
    ops.stream_sum(X.to(DEV), out, idx)
    close(out, X.double().sum(0)[[8, 0, 3]], torch.float32)
    with pytest.raises(cb.CitlaliError, match="streams"):
        ops.hyper_write(torch.zeros(9, 2, 4, device=DEV), torch.zeros(2, 4, device=DEV), torch.zeros(9, 9, device=DEV),
                        torch.zeros(9, device=DEV))


# ---- the delta rule ------------------------------------------------------------------------------------------------

DELTA_SIZES = [dict(heads=6, kv_heads=2, dim=40, vdim=36, conv=3), dict(heads=2, kv_heads=2, dim=130, vdim=8, conv=1),
               dict(heads=4, kv_heads=1, dim=16, vdim=64, conv=5)]


def delta_part(sizes, hidden=48):
    params = dict(sizes, hidden_size=hidden, norm_eps=1e-5)
    return part_class("mixer", "gated_delta")(params, "m")


def delta_plain(h, w, sizes):
    names = {"m.q": "m.q", "m.k": "m.k", "m.v": "m.v", "m.g": "m.gate", "m.b": "m.b", "m.a": "m.a", "m.q.conv": "m.q_conv",
             "m.k.conv": "m.k_conv", "m.v.conv": "m.v_conv", "m.A_log": "m.a_log", "m.dt_bias": "m.dt_bias",
             "m.norm": "m.norm", "m.o": "m.o"}
    return plain.delta_mixer(h.double(), {k: w[v] for k, v in names.items()}, "m", sizes, 1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", DELTA_SIZES)
def test_delta_mixer_whole_in_portions_and_batched(dtype, sizes):
    hidden = 48
    mixer = delta_part(sizes, hidden)
    w = weights_for(mixer, 7, {"a_log": lambda r: -1 + 0.5 * r, "m.b": lambda r: r / 3, "m.a": lambda r: r / 3,
                               "_conv": lambda r: 0.6 * r, "m.norm": lambda r: 1 + 0.3 * r})
    mixer.bind(handles(w, dtype), ctx_for(dtype))
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (37, 1, 12)]
    want = [delta_plain(x, w, sizes) for x in xs]
    cache = SequenceCache([mixer.cache_requirement()], 4, 256, 256, dtype, DEV)
    # whole, one sequence a step
    slots = [cache.acquire() for _ in xs]
    whole = run_steps(mixer, cache, hidden, [[(s, x)] for s, x in zip(slots, xs)], dtype)
    for s, ref in zip(slots, want):
        close(whole[s], ref, dtype)
        cache.release(s)
    # the same slots again (state regions are zeroed on acquire): all three in one step, then cut into portions
    slots = [cache.acquire() for _ in xs]
    first = [(s, x[:max(1, x.shape[0] // 3)]) for s, x in zip(slots, xs)]
    steps = [first]
    at = {s: f.shape[0] for s, f in first}
    sizes_of_portions = [1, 2, 5, 1, 3, 40]
    for n in sizes_of_portions:
        step = [(s, x[at[s]:at[s] + n]) for s, x in zip(slots, xs) if at[s] < x.shape[0]]
        for s, piece in step:
            at[s] += piece.shape[0]
        if step:
            steps.append(step)
    cut = run_steps(mixer, cache, hidden, steps, dtype)
    for s, ref, x in zip(slots, want, xs):
        close(cut[s], ref, dtype)
        if dtype == torch.float32:
            assert torch.equal(cut[s], whole[s]), "the recurrence depends on how the sequence was cut"


def test_delta_rule_keeps_a_memory_for_hundreds_of_tokens():
    """One key/value written at the first token with beta = 1; 600 tokens follow whose keys are orthogonal to it, without
    decay; a query along the first key then reads the first value back, and a query along another direction does not."""
    H, D, V, T = 2, 32, 40, 602
    C = 2 * H * D + H * V
    prep = torch.zeros(T, C + 2 * H)
    k0 = torch.zeros(D); k0[3] = 1.0
    v0 = torch.randn(H, V)
    others = torch.nn.functional.normalize(torch.randn(T, D), dim=-1)
    others[:, 3] = 0.0
    others = torch.nn.functional.normalize(others, dim=-1)
    for h in range(H):
        prep[:, (H + h) * D:(H + h + 1) * D] = others
        prep[0, (H + h) * D:(H + h + 1) * D] = k0
        prep[T - 1, h * D:(h + 1) * D] = k0                       # the last token asks for the first key
        prep[T - 2, h * D:(h + 1) * D] = others[5]
    prep[:, 2 * H * D:C] = torch.randn(T, H * V)
    prep[0, 2 * H * D:C] = v0.flatten()
    prep[:, C:C + H] = 0.5                                         # beta
    prep[0, C:C + H] = 1.0
    prep[:, C + H:] = 1.0                                          # no decay
    prep[T - 1, C:C + H] = 0.0                                     # the reading token writes nothing
    state = torch.zeros(3, H * D * V, device=DEV)
    out = torch.empty(T, H * V, device=DEV)
    seq_start = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([2], dtype=torch.int32, device=DEV)
    ops.delta_rule(prep.to(DEV), state, seq_start, seq_slot, 1, H, H, D, V, out)
    assert torch.allclose(out[T - 1].cpu(), v0.flatten(), atol=1e-4)
    assert not torch.allclose(out[T - 2].cpu(), v0.flatten(), atol=1e-1)
    assert float(state[:2].abs().max()) == 0.0 and float(state[2].abs().max()) > 0.0
    for h in range(H):
        ref = plain.delta_rule(prep[:, h * D:(h + 1) * D].double(), prep[:, (H + h) * D:(H + h + 1) * D].double(),
                               prep[:, 2 * H * D + h * V:2 * H * D + (h + 1) * V].double(), prep[:, C + H + h].double(),
                               prep[:, C + h].double())
        close(out[:, h * V:(h + 1) * V], ref, torch.float32)


# ---- attention through the latent ---------------------------------------------------------------------------------

LATENT_SIZES = [
    dict(heads=5, dim=24, rot_dim=16, vdim=20, q_rank=40, kv_rank=56, scale=0.2, window=11, rot_dims=16, rot_base=1e4),
    dict(heads=2, dim=64, rot_dim=8, vdim=96, q_rank=16, kv_rank=200, scale=0.1, window=None, rot_dims=4, rot_base=5e5),
    dict(heads=3, dim=8, rot_dim=6, vdim=8, q_rank=8, kv_rank=10, scale=0.5, window=64, rot_dims=6, rot_base=100.0,
         sink=None),
]


def latent_part(sizes, hidden=56):
    params = dict(sizes, hidden_size=hidden, norm_eps=1e-5)
    if "sink" in sizes:
        params["names"] = {"sink": None}
    return part_class("mixer", "latent_attention")(params, "m")


def latent_plain(h, w, sizes):
    m = dict(sizes, mask=None if sizes["window"] is None else {"size": sizes["window"]},
             rot={"dims": sizes["rot_dims"], "base": sizes["rot_base"]})
    names = {"m.dq": "m.dq", "m.dq.norm": "m.dq_norm", "m.uq": "m.uq", "m.dkv": "m.dkv", "m.dkv.norm": "m.dkv_norm",
             "m.uk": "m.uk", "m.uv": "m.uv", "m.g": "m.gate", "m.o": "m.o"}
    ww = {k: w[v] for k, v in names.items()}
    if "m.sink" in w:
        ww["m.sink"] = w["m.sink"]
    pos = torch.arange(h.shape[0])
    return plain.latent_attention_mixer(h.double(), ww, "m", m, 1e-5, pos, plain.latent_of(h.double(), ww, "m", m, 1e-5, pos))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", LATENT_SIZES)
def test_latent_attention_whole_in_portions_and_token_by_token(dtype, sizes):
    hidden = 56
    mixer = latent_part(sizes, hidden)
    w = weights_for(mixer, 11, {"_norm": lambda r: 1 + 0.3 * r, "sink": lambda r: 2 * r})
    mixer.bind(handles(w, dtype), ctx_for(dtype))
    x = torch.randn(150, hidden).to(torch.bfloat16).float()
    want = latent_plain(x, w, sizes)
    cache = SequenceCache([mixer.cache_requirement()], 3, 1024, 512, dtype, DEV)
    assert cache.kv_groups[0].values.numel() == 0
    a, b, c = cache.acquire(), cache.acquire(), cache.acquire()
    got = run_steps(mixer, cache, hidden, [[(a, x)], [(b, x[:70]), (c, x[:3])], [(b, x[70:72]), (c, x[3:40])],
                                           [(b, x[72:150]), (c, x[40:41])]] + [[(c, x[i:i + 1])] for i in range(41, 150)],
                    dtype)
    for s in (a, b, c):
        close(got[s], want, dtype)
    if dtype == torch.float32:
        assert torch.equal(got[a], got[b]) and torch.equal(got[a], got[c])


def _latent_walk(q, keys, table_rows, positions, sink, H, R, E, window, scale, page=64, dtype=torch.float32):
    """The walk alone: ``keys`` [T, E] of one sequence are laid into the pages ``table_rows`` names."""
    pages = max(table_rows) + 1
    pool = torch.full((pages + 1, page, E), 1e4, dtype=dtype)              # junk where nothing was written
    for t in range(keys.shape[0]):
        pool[table_rows[t // page], t % page] = keys[t].to(dtype)
    table = torch.tensor([table_rows], dtype=torch.int32, device=DEV)
    rows = len(positions)
    out = torch.empty(rows, H * R, device=DEV)
    ops.latent_attention(q.to(DEV), pool.to(DEV), table, torch.zeros(rows, dtype=torch.int32, device=DEV),
                         torch.tensor(positions, dtype=torch.int32, device=DEV), None if sink is None else sink.to(DEV),
                         out, H, R, E, page, window, scale)
    return out.cpu()


def _walk_plain(q, keys, positions, sink, H, R, E, window, scale):
    out = torch.zeros(len(positions), H, R, dtype=torch.float64)
    for r, p in enumerate(positions):
        lo = 0 if not window else max(0, p - window + 1)
        ks = keys[lo:p + 1].double()
        for h in range(H):
            s = (ks @ q[r, h * E:(h + 1) * E].double()) * scale
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h].double())
            e = torch.exp(s - top)
            den = e.sum() + (0 if sink is None else torch.exp(sink[h].double() - top))
            out[r, h] = (e / den) @ ks[:, :R]
    return out.view(len(positions), H * R)


@pytest.mark.parametrize("dtype", DTYPES)
def test_walk_finds_one_key_far_back_in_shuffled_pages(dtype):
    H, R, E, T = 2, 40, 48, 900
    keys = (0.3 * torch.randn(T, E)).to(torch.bfloat16).float()
    far = 17
    keys[far, R:] = 0.0
    keys[far, R + 1] = 6.0                                    # one key answers the direction the query asks for
    q = 0.3 * torch.randn(3, H * E)
    q[:, R + 1] = 8.0                                          # head 0 of every row asks for it; head 1 does not
    order = torch.randperm((T + 63) // 64).tolist()
    positions = [T - 1, 500, 16]                               # the last row cannot see position 17 yet
    got = _latent_walk(q, keys, order, positions, None, H, R, E, 0, 1.0, dtype=dtype)
    want = _walk_plain(q, keys, positions, None, H, R, E, 0, 1.0)
    close(got, want, dtype, bf16=1e-2)
    for r in (0, 1):
        assert torch.allclose(got[r, :R], keys[far, :R], atol=2e-2), "the far key does not dominate head 0"
    assert not torch.allclose(got[2, :R], keys[far, :R], atol=2e-2)


@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 200])
def test_walk_window_edges(window):
    """A key that takes all the weight when it is seen: the row at distance window - 1 sees it, the row at distance
    window does not, in a prompt's rows and over a page's border."""
    H, R, E, T = 1, 8, 12, 420
    keys = (0.1 * torch.randn(T, E)).to(torch.bfloat16).float()
    q = torch.zeros(2, E); q[:, R] = 1.0
    for marked in (0, 63, 64, 130):
        ks = keys.clone()
        ks[marked, R] = 60.0
        positions = [marked + window - 1, marked + window]
        got = _latent_walk(q, ks, list(range(7))[::-1], positions, None, H, R, E, window, 1.0)
        close(got, _walk_plain(q, ks, positions, None, H, R, E, window, 1.0), torch.float32)
        assert torch.allclose(got[0], ks[marked, :R], atol=1e-5)
        assert not torch.allclose(got[1], ks[marked, :R], atol=1e-2)


def test_walk_sink_takes_weight_without_a_value():
    H, R, E, T = 3, 16, 16, 50
    keys = torch.randn(T, E).to(torch.bfloat16).float()
    q = torch.randn(1, H * E)
    sink = torch.tensor([-1e4, 0.7, 60.0])                    # none, some, nearly all of the weight
    got = _latent_walk(q, keys, [0], [T - 1], sink, H, R, E, 0, 0.3)
    want = _walk_plain(q, keys, [T - 1], sink, H, R, E, 0, 0.3)
    close(got, want, torch.float32)
    plain_softmax = _walk_plain(q, keys, [T - 1], None, H, R, E, 0, 0.3)
    assert torch.allclose(got[0, :R].double(), plain_softmax[0, :R], atol=1e-5)
    assert not torch.allclose(got[0, R:2 * R].double(), plain_softmax[0, R:2 * R], atol=1e-3)
    assert float(got[0, 2 * R:].abs().max()) < 1e-6
    # the sink is not scaled and counts once: a single key with score 0 and a sink of 0 share the weight evenly
    one = _latent_walk(torch.zeros(1, E), keys[:1], [0], [0], torch.zeros(1), 1, R, E, 0, 5.0)
    assert torch.allclose(one[0], 0.5 * keys[0, :R], atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_heads_product_both_orientations(dtype):
    rows, H, K, N, tail = 11, 3, 20, 70, 6
    x = torch.randn(rows, H * (K + tail)).to(torch.bfloat16).float()      # the tensor-core form rounds x to bfloat16
    M = torch.randn(H * K, N).to(torch.bfloat16).float()                      # [h, k, n] as stored
    inv = torch.tensor([1.0, 0.1], dtype=torch.float32)
    pos = torch.arange(100, 100 + rows, dtype=torch.int32)
    y = torch.empty(rows, H * (N + tail), device=DEV)
    ops.heads_product(x.to(DEV), H * (K + tail), K + tail, M.to(DEV, dtype), K * N, N, 1, y, H * (N + tail), N + tail,
                      rows, H, K, N, tail=tail, inv_freq=inv.to(DEV), rot_dims=4, row_pos=pos.to(DEV))
    xv = x.view(rows, H, K + tail).double()
    want = torch.cat([torch.einsum("rhk,hkn->rhn", xv[..., :K], M.view(H, K, N).double()),
                      plain.rotate_interleaved(xv[..., K:], pos, 4, 100.0)], -1)
    close(y.view(rows, H, N + tail), want, torch.float32)
    Mt = torch.randn(H * N, K).to(torch.bfloat16).float()                     # [h, n, k] as stored: y = x . M_h^T
    gate = torch.randn(rows, 5 + H * N)
    out = torch.empty(rows, H * N, dtype=dtype, device=DEV)
    x2 = torch.randn(rows, H * K).to(torch.bfloat16).float()
    gd = gate.to(DEV)
    ops.heads_product(x2.to(DEV), H * K, K, Mt.to(DEV, dtype), N * K, 1, K, out, H * N, N, rows, H, K, N,
                      gate=gd[:, 5:], gate_stride=gd.shape[1])
    want = torch.einsum("rhk,hnk->rhn", x2.view(rows, H, K).double(), Mt.view(H, N, K).double()).reshape(rows, H * N)
    close(out, want * torch.sigmoid(gate[:, 5:].double()), dtype, bf16=1e-2)


# ---- the walk on the tensor cores (bfloat16 caches whose sizes it takes) -------------------------------------------

@pytest.mark.parametrize("H, R, E, T", [(5, 64, 80, 200), (20, 128, 192, 150), (16, 512, 576, 130), (33, 192, 208, 70)])
def test_walk_on_tensor_cores_against_plain(H, R, E, T):
    keys = (0.5 * torch.randn(T, E)).to(torch.bfloat16).float()
    positions = [T - 1, 0, 63, 64, 65, T // 2]
    q = torch.randn(len(positions), H * E).to(torch.bfloat16).float()
    sink = torch.randn(H)
    order = torch.randperm((T + 63) // 64).tolist()
    for window in (0, 70):
        for sk in (None, sink):
            got = _latent_walk(q, keys, order, positions, sk, H, R, E, window, 0.1, dtype=torch.bfloat16)
            close(got, _walk_plain(q, keys, positions, sk, H, R, E, window, 0.1), torch.bfloat16, bf16=1e-2)


@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 130])
def test_tensor_core_walk_window_edges_and_far_key(window):
    H, R, E, T = 3, 64, 80, 460
    keys = (0.1 * torch.randn(T, E)).to(torch.bfloat16).float()
    q = torch.zeros(2, H * E)
    q[:, R] = 1.0                                              # head 0 asks for the marked direction
    for marked in (0, 63, 64, 200):
        ks = keys.clone()
        ks[marked, R] = 60.0
        positions = [marked + window - 1, marked + window]
        got = _latent_walk(q, ks, list(range(8))[::-1], positions, None, H, R, E, window, 1.0, dtype=torch.bfloat16)
        close(got, _walk_plain(q, ks, positions, None, H, R, E, window, 1.0), torch.bfloat16, bf16=1e-2)
        assert torch.allclose(got[0, :R], ks[marked, :R], atol=1e-3)
        assert not torch.allclose(got[1, :R], ks[marked, :R], atol=1e-2)
    # without a window the first key still reaches the last row
    ks = keys.clone()
    ks[0, R] = 60.0
    got = _latent_walk(q[:1], ks, list(range(8)), [T - 1], None, H, R, E, 0, 1.0, dtype=torch.bfloat16)
    assert torch.allclose(got[0, :R], ks[0, :R], atol=1e-3)


def test_tensor_core_walk_does_not_depend_on_the_batch():
    """A row's result is the same bits among other rows in any order, whatever pages it lies in and whatever the other
    rows are; in a step of another size (whose rows' keys are dealt to blocks in other runs) it differs by rounding."""
    H, R, E, T = 8, 64, 80, 300
    keys = torch.randn(T, E).to(torch.bfloat16).float()
    q = torch.randn(4, H * E)
    sink = torch.randn(H)
    a = _latent_walk(q, keys, list(range(5)), [299, 10, 150, 64], sink, H, R, E, 100, 0.2, dtype=torch.bfloat16)
    b = _latent_walk(q[[2, 0, 0, 1]], keys, [4, 2, 0, 1, 3], [150, 299, 7, 40], sink, H, R, E, 100, 0.2, dtype=torch.bfloat16)
    assert torch.equal(a[2], b[0]) and torch.equal(a[0], b[1])
    alone = _latent_walk(q[:1], keys, [3, 1, 4, 0, 2], [299], sink, H, R, E, 100, 0.2, dtype=torch.bfloat16)
    assert torch.allclose(alone[0], a[0], atol=2e-3)
    want = _walk_plain(q, keys, [299, 10, 150, 64], sink, H, R, E, 100, 0.2)
    close(a, want, torch.bfloat16, bf16=1e-2)


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
def test_tensor_core_walk_in_runs(splits):
    """The keys of a row dealt to several blocks and merged: every number of runs, also more runs than tiles."""
    H, R, E, T = 20, 128, 192, 330
    keys = (0.5 * torch.randn(T, E)).to(torch.bfloat16).float()
    positions = [T - 1, 0, 64, 200]
    q = torch.randn(len(positions), H * E)
    sink = torch.randn(H)
    pool = torch.zeros(7, 64, E, dtype=torch.bfloat16)
    order = [5, 0, 3, 1, 6, 2]
    for t_ in range(T):
        pool[order[t_ // 64], t_ % 64] = keys[t_].to(torch.bfloat16)
    for window in (0, 150):
        out = torch.empty(len(positions), H * R, device=DEV)
        ops.latent_attention(q.to(DEV), pool.to(DEV), torch.tensor([order], dtype=torch.int32, device=DEV),
                             torch.zeros(len(positions), dtype=torch.int32, device=DEV),
                             torch.tensor(positions, dtype=torch.int32, device=DEV), sink.to(DEV), out, H, R, E, 64, window,
                             0.1, splits=splits)
        close(out, _walk_plain(q, keys, positions, sink, H, R, E, window, 0.1), torch.bfloat16, bf16=1e-2)


@pytest.mark.parametrize("D, V", [(32, 40), (128, 24), (80, 8)])
def test_delta_rule_two_tokens_at_a_time(D, V):
    """The form that takes a sequence's rows in pairs against the plain recurrence: even and odd lengths, a single row,
    three sequences in one launch, states carried over from a launch before."""
    H, KH = 4, 2
    C = 2 * KH * D + H * V
    lengths = [7, 1, 64]
    T = sum(lengths)
    g = torch.Generator().manual_seed(D + V)
    prep = torch.zeros(T, C + 2 * H)
    prep[:, :2 * KH * D] = torch.nn.functional.normalize(torch.randn(T, 2 * KH, D, generator=g), dim=-1).view(T, -1)
    prep[:, :KH * D] *= D ** -0.5
    prep[:, 2 * KH * D:C] = torch.randn(T, H * V, generator=g)
    prep[:, C:C + H] = torch.rand(T, H, generator=g)
    prep[:, C + H:] = 0.9 + 0.1 * torch.rand(T, H, generator=g)
    seq_start = torch.tensor([0, 7, 8, T], dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([2, 0, 1], dtype=torch.int32, device=DEV)
    outs = {}
    for pairs in (False, True):
        state = torch.zeros(3, H * D * V, device=DEV)
        out = torch.empty(T, H * V, device=DEV)
        ops.delta_rule(prep.to(DEV), state, seq_start, seq_slot, 3, H, KH, D, V, out, pairs=pairs)
        again = torch.empty(T, H * V, device=DEV)                # the same rows once more, from the states just left
        ops.delta_rule(prep.to(DEV), state, seq_start, seq_slot, 3, H, KH, D, V, again, pairs=pairs)
        outs[pairs] = (out.cpu(), again.cpu(), state.cpu())
    for a, b in zip(outs[False], outs[True]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)
    at = 0
    for n in lengths:
        for h in range(H):
            kh = h // (H // KH)
            rows = slice(at, at + n)
            ref = plain.delta_rule(prep[rows, kh * D:(kh + 1) * D].double(), prep[rows, (KH + kh) * D:(KH + kh + 1) * D].double(),
                                   prep[rows, 2 * KH * D + h * V:2 * KH * D + (h + 1) * V].double(),
                                   prep[rows, C + H + h].double(), prep[rows, C + h].double())
            close(outs[True][0][rows, h * V:(h + 1) * V], ref, torch.float32, f32=1e-4)
        at += n
