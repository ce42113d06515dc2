"""The Lanizen decoder through the session, the cache and the step function, against the plain implementation:
whole prompts; prompts with their tails decoded token by token; every token alone from the first; portions of 2 to
40 tokens; batches of unequal requests over few slots and few pages (slots and pages are used again); requests that
join a running batch; long decoding past every window and over several pages; bin/trace_run; greedy generation
through ``generate`` (whose decode steps are replayed CUDA graphs).  In 32-bit the ways of cutting a sequence must
agree to rounding with the exact evaluation; in bfloat16 within the rounding of 8-bit mantissas."""
import json
import os
import subprocess
import sys

import pytest
import torch

import citlali_b200 as cb
import plain_lanizen as plain
import replay
from helpers import random_tokens
from lanizen_models import CONFIGS, write_model

pytestmark = pytest.mark.gpu

LENGTHS = {"P": [1, 2, 5, 9, 10, 21, 64, 65, 150], "Q": [3, 40, 129, 7, 70], "R": [64, 65, 66, 131, 200, 1, 33],
           "S": [1, 6, 30]}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("lanizen")
    out = {}
    for i, name in enumerate(CONFIGS):
        path = str(root / name)
        cfg, w = write_model(path, name, seed=50 + i)
        out[name] = (path, cfg.to_dict(), w)
    return out


def requests_for(name):
    return [(f"r{i}", random_tokens(CONFIGS[name]["vocab"], n, 31 * i + n)) for i, n in enumerate(LENGTHS[name])]


_plain = {}


def plain_rows(models, name):
    if name not in _plain:
        _, cfg, w = models[name]
        _plain[name] = {rid: plain.forward(cfg, w, toks) for rid, toks in requests_for(name)}
    return _plain[name]


def session_for(models, name, dtype, max_batch=8, max_tokens=None, graphs=True):
    s = cb.InferenceSession()
    s.use_graphs = graphs
    return s.load_model(models[name][0], max_context=1024, dtype=dtype, max_batch=max_batch, max_tokens=max_tokens)


def check(got, want_rows, dtype, what):
    worst = 0.0
    for (rid, pos), row in got.items():
        ref = want_rows[rid][pos]
        scale = float(ref.abs().max())
        err = float((row.double() - ref).abs().max())
        worst = max(worst, err / scale)
        assert err <= TOL[dtype] * scale, f"{what}: request {rid} position {pos}: |diff| {err:.3e} of {scale:.3e}"
    print(f"[{what}] worst |diff| / max|logit| = {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_way_of_cutting_agrees_with_plain(models, name, dtype):
    want = plain_rows(models, name)
    reqs = requests_for(name)
    s = session_for(models, name, dtype, max_batch=3, max_tokens=512)
    ways = {
        "whole": replay.whole(reqs),
        "tail": replay.tail(reqs, last=32),
        "token by token": replay.tail(reqs, last=10 ** 6),
        "portions": replay.chunked(reqs, 3, seed=5, low=2, high=40),
        "portions of two": replay.chunked(reqs, 2, seed=6, low=2, high=2),
        "batched": replay.batched(reqs, [max(1, len(t) * 2 // 3) for _, t in reqs], 3),
        "joining": replay.joining(reqs[:3], [max(1, len(t) // 2) for _, t in reqs[:3]], every=2),
    }
    results = {}
    for what, steps in ways.items():
        results[what] = replay.run_in_process(s, steps)
        check(results[what], want, dtype, f"{name} {dtype} {what}")
        assert s.cache.pages_held() == 0 and s.cache.slots.held == []
    # one order of operations for every cut: in 32-bit the recurrent layers and the walk over the cache give the same
    # bits; the products' summation order is the same too
    if dtype == "float32":
        base = results["whole"]
        for what in ("tail", "token by token", "portions", "portions of two"):
            for key, row in results[what].items():
                assert torch.equal(row, base[key]), f"{name}: '{what}' differs from 'whole' at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(models, dtype):
    """A short prompt, then 300 tokens one by one: the windows (9, 20; 65, 130, 1) pass over decoded tokens only, pages
    fill up, are given back behind the window and taken again."""
    for name in ("P", "R"):
        _, cfg, w = models[name]
        toks = random_tokens(CONFIGS[name]["vocab"], 305, 77)
        want = {"x": plain.forward(cfg, w, toks)}
        s = session_for(models, name, dtype, max_batch=1, max_tokens=256)    # four pages: fewer than the sequence needs
        got = replay.run_in_process(s, replay.tail([("x", toks)], last=300))
        check(got, want, dtype, f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, dtype):
    name = "P"
    reqs = requests_for(name)[2:7]
    steps = replay.batched(reqs, [max(1, len(t) - 3) for _, t in reqs], 3)
    got = replay.run_trace_run(models[name][0], dtype, steps, CONFIGS[name]["vocab"])
    check(got, plain_rows(models, name), dtype, f"trace_run {dtype}")


def test_trace_run_counts_tokens_without_page_padding(models):
    """--max-tokens is the number of tokens live requests hold, not whole pages: twelve requests of 1 to 12 tokens live
    at once need twelve pages although they hold 78 tokens."""
    name = "S"
    _, cfg, w = models[name]
    reqs = [(f"q{i}", random_tokens(CONFIGS[name]["vocab"], i + 1, 900 + i)) for i in range(12)]
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks, "want": [len(toks) - 1]} for rid, toks in reqs],
              "end": [rid for rid, _ in reqs]}]
    got = replay.run_trace_run(models[name][0], "float32", steps, CONFIGS[name]["vocab"],
                               max_tokens=sum(len(t) for _, t in reqs))
    want = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs}
    check(got, want, "float32", "trace_run with many short requests")


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_follows_plain(models, name, graphs):
    """``generate`` with temperature 0 in 32-bit: every generated token is the plain implementation's choice on the same
    prefix, unless its margin there is within rounding.  Five prompts over two slots: slots and state regions are used
    again, and the decode steps are replayed graphs (or plain launches)."""
    _, cfg, w = models[name]
    s = session_for(models, name, "float32", max_batch=2, graphs=graphs)
    assert (s.runner is not None) == graphs
    prompts = [random_tokens(CONFIGS[name]["vocab"], n, 9 * n) for n in (3, 17, 1, 66, 30)]
    results = s.generate(prompts, cb.GenerationOptions(max_new_tokens=24, temperature=0.0))
    compared = 0
    for prompt, res in zip(prompts, results):
        assert len(res.tokens) == 24
        logits = plain.forward(cfg, w, list(prompt) + list(res.tokens))
        for i, tok in enumerate(res.tokens):
            row = logits[len(prompt) - 1 + i]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) > 1e-4 * float(row.abs().max()):
                assert int(row.argmax()) == tok, f"{name}: token {i} of a prompt of {len(prompt)}"
                compared += 1
    assert compared >= 100


def test_command_line(models):
    """bin/citlali_cli on a Lanizen folder: the same tokens as ``generate``, and --info from the configuration alone."""
    cli = os.path.join(replay.ROOT, "bin", "citlali_cli")
    path = models["R"][0]
    out = subprocess.run([sys.executable, cli, "--model", path, "--prompt-ids", "1,2,3,4,5", "--prompt-ids", "9,8,7",
                          "--max-new-tokens", "6", "--ctx", "64", "--dtype", "float32", "--json"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    data = json.loads(out.stdout)
    session = cb.InferenceSession().load_model(path, max_context=64, dtype="float32", max_batch=8)
    want = session.generate([[1, 2, 3, 4, 5], [9, 8, 7]], cb.GenerationOptions(max_new_tokens=6, max_context=64))
    assert [r["tokens"] for r in data["results"]] == [r.tokens for r in want]
    info = subprocess.run([sys.executable, cli, "--model", path, "--info"], capture_output=True, text=True, timeout=120)
    assert info.returncode == 0 and "architecture: Lanizen" in info.stdout and "streams: 4" in info.stdout
    assert "cache bytes per token (bfloat16): %d" % (2 * (96 + 32) + 2 * (12 + 4)) in info.stdout
    assert "state bytes per sequence: %d" % (4 * (8 * 80 * 40 + 3 * (2 * 2 * 80 + 8 * 40))) in info.stdout
