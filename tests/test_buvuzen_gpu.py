"""Buvuzen in the engine against the plain implementation (`plain_buvuzen.py`): whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal requests in one batch against each alone, pages that are
given back (by a window, by a request's end) and used again, long decoding, other sizes, and greedy generation through
the engine's own entry point and scheduler; in 32-bit (every value within 1e-4) and in bfloat16 (by what rounding
costs).  The cache pool is filled with NaN first."""
import numpy as np
import pytest

import plain_buvuzen as B
from buvuzen_helpers import CONFIGS, Oracle, compare, decided_tokens, lively_weights, write_model
from helpers import RoundingJudge, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("buvuzen")
    out = {}
    for name, cfg in CONFIGS.items():
        w = lively_weights(cfg, seed=23 + len(name))
        out[name] = (cfg, w, write_model(str(root / name), cfg, w))
    return out


def tokens_of(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def engine_for(folder, dtype, pool_tokens, slots=4, page_size=16, graphs=True):
    from velox_b200 import Engine, EngineConfig
    return Engine(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool_tokens,
                                       max_running_requests=slots, max_model_len=pool_tokens, cuda_graphs=graphs),
                  poison_cache=True)


def run(engine, steps):
    """steps: [[(request, tokens, want)], ...] with ("end", request) entries to give a request's cache back.
    Returns the logits of every step that wanted some."""
    from velox_b200.engine import StepEntry
    out = []
    for step in steps:
        entries = []
        for e in step:
            if e[0] == "end":
                continue
            if not engine.cache.has_request(e[0]):
                assert engine.cache.add_request(e[0]) is not None
            entries.append(StepEntry(e[0], e[1], e[2]))
        logits = engine.run_step(entries) if entries else None
        out.append(None if logits is None else logits.cpu().numpy())
        for e in step:
            if e[0] == "end":
                engine.cache.release(e[1])
    engine.cache.check()
    return out


def portions(tokens, sizes, name):
    """The sequence cut into portions of the given sizes (repeated), every position wanted."""
    steps, at, k = [], 0, 0
    while at < len(tokens):
        s = min(sizes[k % len(sizes)], len(tokens) - at)
        steps.append([(name, tokens[at:at + s], list(range(s)))])
        at += s
        k += 1
    return steps


def test_the_residual_stream_after_every_layer_run(models):
    """Layer by layer, in 32 bits, through the model's own blocks in an ordinary step: what the plain implementation has
    after every run of a layer (a layer that shares another's tensors counts each time)."""
    cfg, w, folder = models["odd"]
    toks = tokens_of(cfg, 21, 2)
    want = []
    B.forward(cfg, w, toks, layers_out=want)
    engine = engine_for(folder, "float32", 64, graphs=False)
    model, seen = engine.runner.model, []
    for block in set(model.blocks):
        def forward(residual, delta, ctx, cache, inner=block.forward):
            residual, delta = inner(residual, delta, ctx, cache)
            assert delta is None
            seen.append(residual.clone())
            return residual, delta
        block.forward = forward
    run(engine, [[("a", toks, [])]])
    assert len(seen) == len(cfg["layers"]) == len(want)
    for place, (got, exact) in enumerate(zip(seen, want)):
        got = got.cpu().numpy().astype(np.float64)
        assert np.abs(got - exact).max() <= 1e-4 * max(1.0, np.abs(exact).max()), "after layer run %d" % place


# In bfloat16 a router's close call may go the other way, and the other expert's output then reaches every later
# position through the keys; so long bfloat16 runs use the configuration whose routers have nothing to decide, and
# the routed ones run on sequences that have no close call.
@pytest.mark.parametrize("name,dtype,length", [("odd", "float32", 150), ("even", "float32", 150), ("all", "float32", 150),
                                               ("odd", "bfloat16", 40), ("all", "bfloat16", 150), ("even", "bfloat16", 24),
                                               ("mid", "float32", 100), ("mid", "bfloat16", 150)])
def test_whole_prompts_portions_and_decoding_agree_with_the_plain_implementation(models, name, dtype, length):
    cfg, w, folder = models[name]
    toks, oracle = decided_tokens(cfg, w, length, 1) if (name, dtype) in (("even", "bfloat16"), ("odd", "bfloat16")) else (tokens_of(cfg, length, 1), None)
    oracle = oracle or Oracle(cfg, w, toks)
    judge = RoundingJudge.of([oracle], "buvuzen %s %s" % (name, dtype))
    engine = engine_for(folder, dtype, 160 + 64)
    ways = {
        "whole": [[("a", toks, list(range(len(toks))))]],
        "prompt then one by one": [[("a", toks[:length * 3 // 5], list(range(length * 3 // 5)))]]
                                  + [[("a", [t], [0])] for t in toks[length * 3 // 5:]],
        "token by token from the start": [[("a", [t], [0])] for t in toks[:40]],
        "portions 2 3 64 5 1 16 2": portions(toks, [2, 3, 64, 5, 1, 16, 2], "a"),
        "portions 17 31": portions(toks, [17, 31], "a"),
        "portions 2": portions(toks[:48], [2], "a"),
    }
    for what, steps in ways.items():
        got = np.concatenate([g for g in run(engine, steps + [[("end", "a")]]) if g is not None])
        compare(got, [(oracle, 0, len(got))], dtype, "%s, %s" % (name, what), judge)
    if dtype != "float32":
        judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages(models, dtype):
    """Four live requests at most in a pool of 20 pages: requests of 1 to 130 tokens come, go on beside one another in
    portions and single tokens, are left out of steps, end, and their pages go to the next."""
    cfg, w, folder = models["even" if dtype == "float32" else "all"]
    lens = {"a": 130, "b": 37, "c": 1, "d": 64, "e": 90, "f": 2, "g": 70}
    toks = {k: tokens_of(cfg, n, 100 + i) for i, (k, n) in enumerate(lens.items())}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    judge = RoundingJudge.of(oracle.values(), "buvuzen mixed %s" % dtype)
    engine = engine_for(folder, dtype, 20 * 16, slots=4)
    at = {k: 0 for k in toks}

    def take(k, n):
        lo = at[k]
        hi = min(lo + n, len(toks[k]))
        at[k] = hi
        return (k, toks[k][lo:hi], list(range(hi - lo)), lo)

    plan = [
        [("a", 33), ("b", 7), ("c", 1)], [("end", "c")],
        [("a", 1), ("b", 30), ("d", 2)], [("end", "b")],
        [("a", 64), ("d", 1), ("f", 2)], [("end", "f")],
        [("d", 61), ("e", 17)], [("end", "d")],
        [("a", 2), ("e", 1), ("g", 48)],
        [("e", 72)], [("end", "e")],
        [("a", 30), ("g", 1)], [("end", "a")],
        [("g", 21)], [("end", "g")],
    ]
    for step in plan:
        if step[0][0] == "end":
            run(engine, [[step[0]]])
            continue
        entries = [take(k, n) for k, n in step]
        got = run(engine, [[(k, t, want) for k, t, want, _ in entries]])[0]
        compare(got, [(oracle[k], lo, lo + len(t)) for k, t, _, lo in entries], dtype, "step %s" % (step,), judge)
    assert all(at[k] == len(toks[k]) for k in toks)
    assert all(g.allocator.num_free == g.allocator.num_pages for g in engine.cache.groups)
    if dtype != "float32":
        judge.finish()


def test_a_window_gives_its_pages_back_as_it_passes(models):
    cfg, w, folder = models["even"]
    toks = tokens_of(cfg, 200, 5)
    oracle = Oracle(cfg, w, toks)
    engine = engine_for(folder, "float32", 208)
    got = np.concatenate(run(engine, portions(toks, [50, 1, 1, 30], "a")))
    assert_close(got, oracle.exact, "float32", "long prompt over many pages")
    tables = {g.spec.window: engine.cache.requests["a"].tables[i] for i, g in enumerate(engine.cache.groups)}
    assert sorted(tables) == [23, 40, 70]
    for window, table in tables.items():
        gone = (200 - window) // 16          # pages wholly before the last position's window
        assert all(p < 0 for p in table[:gone]) and all(p >= 0 for p in table[gone + 1:13])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_request_beside_short_ones_in_a_pool_made_for_what_is_live(models, dtype):
    """700 tokens in portions that end inside pages and windows, beside a request that decodes token by token, ends, and
    whose pages a third one takes; the pool holds what is live at any time (each request rounded up to 64 tokens) and
    no more, so the windows' pages that went back are used again."""
    cfg, w, folder = models["even" if dtype == "float32" else "all"]
    toks = {"a": tokens_of(cfg, 700, 71), "b": tokens_of(cfg, 40, 72), "c": tokens_of(cfg, 60, 73)}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    judge = RoundingJudge.of(oracle.values(), "buvuzen long request %s" % dtype)
    engine = engine_for(folder, dtype, 704 + 64)
    at = {k: 0 for k in toks}

    def take(k, n):
        lo = at[k]
        hi = min(lo + n, len(toks[k]))
        at[k] = hi
        return (k, toks[k][lo:hi], list(range(hi - lo)), lo)

    plan = [[("a", 128), ("b", 21)], [("a", 29), ("b", 1)], [("a", 2), ("b", 1)], [("a", 300), ("b", 1)]]
    plan += [[("a", 1), ("b", 1)] for _ in range(16)] + [[("end", "b")], [("a", 1), ("c", 33)], [("a", 224), ("c", 1)]]
    plan += [[("c", 2)], [("c", 24)], [("end", "a")], [("end", "c")]]
    for step in plan:
        if step[0][0] == "end":
            run(engine, [[step[0]]])
            continue
        entries = [take(k, n) for k, n in step]
        got = run(engine, [[(k, t, want) for k, t, want, _ in entries]])[0]
        compare(got, [(oracle[k], lo, lo + len(t)) for k, t, _, lo in entries], dtype, "step %s" % (step,), judge)
    assert all(at[k] == len(toks[k]) for k in toks)
    assert all(g.allocator.num_free == g.allocator.num_pages for g in engine.cache.groups)
    if dtype != "float32":
        judge.finish()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """360 tokens one by one after a short prompt: the windows pass over decoded tokens only, pages go back and are
    taken again, the captured step is replayed."""
    cfg, w, folder = models["even" if dtype == "float32" else "all"]
    toks = tokens_of(cfg, 380, 9)
    oracle = Oracle(cfg, w, toks)
    judge = RoundingJudge.of([oracle], "buvuzen long decoding %s" % dtype)
    engine = engine_for(folder, dtype, 384)
    steps = [[("a", toks[:20], list(range(20)))]] + [[("a", [t], [0])] for t in toks[20:]]
    got = np.concatenate(run(engine, steps))
    compare(got, [(oracle, 0, len(toks))], dtype, "long decoding", judge)
    if dtype != "float32":
        judge.finish()


def test_two_requests_decode_side_by_side_in_captured_steps(models):
    cfg, w, folder = models["odd"]
    ta, tb = tokens_of(cfg, 60, 21), tokens_of(cfg, 45, 22)
    oa, ob = Oracle(cfg, w, ta), Oracle(cfg, w, tb)
    engine = engine_for(folder, "float32", 128)
    run(engine, [[("a", ta[:30], []), ("b", tb[:15], [])]])
    for i in range(30):
        got = run(engine, [[("a", [ta[30 + i]], [0]), ("b", [tb[15 + i]], [0])]])[0]
        assert_close(got, np.stack([oa[30 + i], ob[15 + i]]), "float32", "decode step %d" % i)


def test_greedy_generation_through_the_engine(models):
    from velox_b200 import SamplingParams
    cfg, w, folder = models["odd"]
    engine = engine_for(folder, "float32", 256)
    prompts = [tokens_of(cfg, 19, 31), tokens_of(cfg, 3, 32), tokens_of(cfg, 40, 33)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, o in zip(prompts, outs):
        assert o == B.greedy_generate(cfg, w, p, 12)
    # a second round on the same engine: the pages of the first are used again
    outs2 = engine.generate(prompts[::-1], SamplingParams(max_tokens=5, temperature=0.0))
    assert outs2 == [o[:5] for o in outs[::-1]]


def test_generation_with_chunked_prompts_and_a_small_batch_budget(models):
    from velox_b200 import Engine, EngineConfig, SamplingParams
    cfg, w, folder = models["even"]
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=512, max_running_requests=3,
                                         max_model_len=256, max_batch_tokens=24, chunk_size=16))
    prompts = [tokens_of(cfg, n, 40 + n) for n in (50, 7, 33, 21)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for p, o in zip(prompts, outs):
        assert o == B.greedy_generate(cfg, w, p, 6)


def test_the_command_line_writes_and_runs_a_random_model(tmp_path):
    import json
    import subprocess
    import sys
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    (tmp_path / "c.json").write_text(json.dumps(CONFIGS["odd"]))
    out = subprocess.run([sys.executable, "-m", "velox_b200", "random-model", "--config", str(tmp_path / "c.json"),
                          "--model-dir", str(tmp_path / "m"), "--seed", "3"], cwd=root, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout.strip().splitlines()[-1])["architecture"] == "Buvuzen"
    gen = subprocess.run([sys.executable, "-m", "velox_b200", "generate", "--model-dir", str(tmp_path / "m"),
                          "--prompt-tokens", "5,6,7,8", "--max-tokens", "4", "--dtype", "float32"],
                         cwd=root, capture_output=True, text=True)
    assert gen.returncode == 0, gen.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_replays_requests_through_a_small_pool(models, tmp_path, dtype):
    """bin/trace_run as a user starts it (its own process, a pool of 24 pages): five requests, at most four of them
    live, portions beside single tokens, a request left out of steps, pages used again."""
    from helpers import run_trace
    cfg, w, folder = models["even" if dtype == "float32" else "all"]
    toks = {k: tokens_of(cfg, n, 60 + i) for i, (k, n) in enumerate({"p": 100, "q": 37, "r": 64, "s": 2, "t": 90}.items())}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    at = {k: 0 for k in toks}
    steps, expect = [], []

    def step(parts, end=()):
        entries, rows = [], []
        for k, n in parts:
            lo, hi = at[k], min(at[k] + n, len(toks[k]))
            at[k] = hi
            entries.append({"id": k, "tokens": toks[k][lo:hi], "want": list(range(hi - lo))})
            rows.append((oracle[k], lo, hi))
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})
        expect.append(rows)
    step([("p", 40), ("q", 36), ("r", 1)])
    step([("p", 1), ("q", 1), ("r", 63), ("s", 2)], end=["q", "r", "s"])
    step([("t", 33)])                          # ("p" is left out of this step)
    step([("p", 59), ("t", 1)], end=["p"])
    step([("t", 56)], end=["t"])
    got = run_trace(folder, dtype, steps, 24 * 16, str(tmp_path / "out"), vocab=cfg["vocab"])
    judge = RoundingJudge.of(oracle.values(), "buvuzen trace runner %s" % dtype)
    for n, rows in enumerate(expect):
        compare(got[n], rows, dtype, "step %d" % n, judge)
    if dtype != "float32":
        judge.finish()
