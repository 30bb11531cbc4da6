"""Dugulorn through the engine against the plain implementation (tests/plain_dugulorn.py): whole prompts, the last tokens
one by one, portions down to two tokens, the first tokens one by one, unequal requests in one batch with pools so small
that pages and state slots are used again, long decoding, the residual stream after every layer, greedy generation
through the public entry point and the replay command.  The weights are made telling (tests/dugulorn_models.py): a key
read from a wrong page or a state lost at a cut moves the logits by hundreds of tolerances."""
import numpy as np
import pytest
import torch

import dugulorn_models as dm
import plain_dugulorn as plain
from trace_util import TraceBuilder, needed_max_tokens, portions, rows_by_position, run_trace, run_trace_in_process, tail_one_by_one, whole

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 4e-2}        # of the largest logit


@pytest.fixture(scope="module")
def dg_dirs(tmp_path_factory):
    return dm.write_all(str(tmp_path_factory.mktemp("dugulorn")))


def make_runner(d, name, dtype, pages=24, **kw):
    from cppvllm_b200.engine.runner import ModelRunner
    args = dict(dtype=torch.float32 if dtype == "float32" else torch.bfloat16, page_size=dm.page_size(name), num_pages=pages,
                max_step_tokens=256, max_seqs=8, max_model_len=384)
    args.update(kw)
    return ModelRunner(d, **args)


def check(rows, refs, dtype):
    errs = []
    for (rid, pos), row in rows.items():
        ref = refs[rid.split("#")[0]]
        scale = max(1.0, float(ref.abs().max()))
        errs.append((float(np.abs(row - ref[pos].numpy()).max()) / scale, rid, pos))
    worst, rid, pos = max(errs)
    over = sum(1 for e in errs if e[0] > TOL[dtype])
    allowed = 0 if dtype == "float32" else max(1, len(errs) // 50)
    assert over <= allowed, f"{over} of {len(errs)} rows beyond {TOL[dtype]:.1e}; worst {worst:.3e} at request {rid} position {pos}"
    print(f"worst error {worst:.3e} of scale, {over} rows beyond the tolerance ({dtype})")
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["dg_a", "dg_b", "dg_c", "dg_d"])
def test_whole_tail_and_portions_match_the_plain_implementation(dg_dirs, name, dtype):
    d, vocab = dg_dirs[name], dm.config(name)["vocab"]
    toks = {"w": dm.random_tokens(vocab, 110, 1), "t": dm.random_tokens(vocab, 101, 2), "p": dm.random_tokens(vocab, 110, 1),
            "s": dm.random_tokens(vocab, 1, 3), "q": dm.random_tokens(vocab, 3, 4)}
    tb = TraceBuilder()
    whole(tb, "w", toks["w"])
    tail_one_by_one(tb, "t", toks["t"], tail=40)
    portions(tb, "p", toks["p"])
    whole(tb, "s", toks["s"])                          # the first token alone
    tb.add([("q", toks["q"][:1], [0])])                # the first tokens one by one
    tb.add([("q", toks["q"][1:2], [0])])
    tb.add([("q", toks["q"][2:3], [0])], end=["q"])
    runner = make_runner(d, name, dtype, pages=(128 // dm.page_size(name)), num_state_slots=1)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    assert len(rows) == 110 + 101 + 110 + 1 + 3
    refs = {k: plain.forward(d, v).float() for k, v in toks.items()}
    check(rows, refs, dtype)
    apart = sum(1 for pos in range(110)               # cut differently, equal beyond rounding
                if np.abs(rows[("w", pos)] - rows[("p", pos)]).max() > TOL[dtype] * max(1.0, np.abs(rows[("w", pos)]).max()))
    assert apart <= (0 if dtype == "float32" else 3)
    runner.cache.check_invariants()
    assert all(runner.cache.num_free_pages(g) == 128 // dm.page_size(name) for g in range(len(runner.group_specs)))


@pytest.mark.parametrize("seed", range(100, 110))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Layers of every kind in any order and size (tests/dugulorn_models.py: random_config): a whole prompt, a tail decoded
    token by token and portions down to two tokens, in float32, where nothing but the order of sums may differ."""
    import random
    cfg = dm.random_config(seed)
    d = dm.write_model(str(tmp_path / "m"), cfg, seed)
    toks = {"w": dm.random_tokens(cfg["vocab"], 90, 1), "t": dm.random_tokens(cfg["vocab"], 75, 2), "p": dm.random_tokens(cfg["vocab"], 90, 1)}
    tb = TraceBuilder()
    whole(tb, "w", toks["w"])
    tail_one_by_one(tb, "t", toks["t"], tail=20)
    portions(tb, "p", toks["p"])
    from cppvllm_b200.engine.runner import ModelRunner
    page = random.Random(seed).choice([16, 32, 64])
    runner = ModelRunner(d, dtype=torch.float32, page_size=page, num_pages=128 // page, max_step_tokens=128, max_seqs=4, max_model_len=128,
                         num_state_slots=2)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    check(rows, {k: plain.forward(d, v).float() for k, v in toks.items()}, "float32")


@pytest.mark.parametrize("dtype,eager", [("float32", False), ("bfloat16", False), ("float32", True)])
@pytest.mark.parametrize("name", ["dg_a", "dg_b", "dg_c"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dg_dirs, name, dtype, eager):
    """Up to four live requests: portions of some beside single tokens of others, in a pool of 384 tokens (the requests need
    704) and four state slots, so that every page and slot serves several requests; every logit is compared with the
    request run alone in the plain implementation."""
    d, vocab = dg_dirs[name], dm.config(name)["vocab"]
    lens = {"a": 97, "b": 64, "c": 33, "d": 120, "e": 2, "f": 71, "g": 65}
    toks = {k: dm.random_tokens(vocab, n, 30 + n) for k, n in lens.items()}
    cuts = {"a": [2, 31, 1, 1, 1, 29, 32], "b": [64], "c": [16, 15, 1, 1], "d": [3, 2, 59, 1, 1, 1, 53], "e": [1, 1],
            "f": [40, 2, 29], "g": [63, 1, 1]}
    waiting = ["a", "b", "c", "d", "e", "f", "g"]
    live, at, part = [], {k: 0 for k in lens}, {k: 0 for k in lens}
    tb = TraceBuilder()
    while waiting or live:
        while waiting and len(live) < 4 and sum((lens[k] + 63) // 64 * 64 for k in live + [waiting[0]]) <= 384:
            live.append(waiting.pop(0))
        entries, end = [], []
        for k in list(live):
            n = cuts[k][part[k]]
            entries.append((k, toks[k][at[k]:at[k] + n], range(n)))
            at[k] += n
            part[k] += 1
            if at[k] == lens[k]:
                end.append(k)
                live.remove(k)
        tb.add(entries, end=end)
    assert needed_max_tokens(tb.steps) <= 384 and max(len(st["entries"]) for st in tb.steps) == 4
    runner = make_runner(d, name, dtype, pages=384 // dm.page_size(name), num_state_slots=4, enforce_eager=eager)
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    assert len(rows) == sum(lens.values())
    check(rows, {k: plain.forward(d, v).float() for k, v in toks.items()}, dtype)
    runner.cache.check_invariants()
    # the same trace once more on the same runner: every page and slot has had another owner by now
    again = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    for key, row in rows.items():                      # the same steps, the same kernels: the same bits
        assert np.array_equal(again[key], row)


@pytest.mark.parametrize("use_ref_kernels", [False, True])
@pytest.mark.parametrize("name", ["dg_a", "dg_b"])
def test_residual_stream_after_every_layer(dg_dirs, name, use_ref_kernels):
    d = dg_dirs[name]
    toks = dm.random_tokens(dm.config(name)["vocab"], 37, 5)
    runner = make_runner(d, name, "float32", enforce_eager=True, use_ref_kernels=use_ref_kernels)
    seen = []
    for b in runner.model.blocks:
        def wrapped(h, pending, ctx, cache, state, f=b.forward):
            h2, p2 = f(h, pending, ctx, cache, state)
            assert p2 is None
            seen.append(h2.clone().cpu())
            return h2, p2
        b.forward = wrapped
    tb = TraceBuilder()
    whole(tb, "x", toks)
    run_trace_in_process(runner, tb.steps)
    _, runs = plain.forward(d, toks, return_layers=True)
    assert len(seen) == len(runs) == 4
    for got, ref in zip(seen, runs):
        assert float((got.double() - ref).abs().max()) <= 2e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["dg_a", "dg_c"])
def test_long_decoding(dg_dirs, name, dtype):
    """A prompt of 20 tokens and 300 tokens decoded one by one (through the captured graphs): the matrices of the recurrent
    mixers are read and written 300 times and the first keys stay visible."""
    d, vocab = dg_dirs[name], dm.config(name)["vocab"]
    toks = dm.random_tokens(vocab, 320, 9)
    tb = TraceBuilder()
    tb.add([("z", toks[:20], range(20))])
    for i in range(20, 320):
        tb.add([("z", toks[i:i + 1], [0])], end=["z"] if i == 319 else [])
    runner = make_runner(d, name, dtype, pages=320 // dm.page_size(name))
    rows = rows_by_position(tb.steps, run_trace_in_process(runner, tb.steps))
    check(rows, {"z": plain.forward(d, toks).float()}, dtype)
    assert runner.stats["graph_steps"] >= 299


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(dg_dirs, dtype):
    from cppvllm_b200 import LLM, SamplingParams
    d = dg_dirs["dg_b"]
    prompts = [dm.random_tokens(131, n, 70 + n) for n in (1, 6, 40, 75)]
    llm = LLM(d, dtype=dtype, block_size=32, num_kv_blocks=12, max_num_batched_tokens=48, max_num_seqs=4, max_chunk_tokens=20,
              max_model_len=200)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.prompt_ids == p and len(o.token_ids) == 10
        if dtype == "float32":
            assert o.token_ids == plain.greedy_generate(d, p, 10)
        else:
            ref = plain.forward(d, (p + o.token_ids)[:-1])
            for i, tok in enumerate(o.token_ids):
                row = ref[len(p) - 1 + i]
                assert row[tok] >= row.max() - 0.05 * max(1.0, float(row.abs().max()))
    llm.runner.check_errors()
    llm.runner.cache.check_invariants()


def test_generation_when_pages_run_out_and_requests_are_recomputed(dg_dirs):
    """A pool that cannot hold all running requests: some are preempted and recomputed from their first token, with a fresh
    state slot; the tokens are those of each request alone."""
    from cppvllm_b200 import LLM, SamplingParams
    d = dg_dirs["dg_a"]
    prompts = [dm.random_tokens(97, n, 90 + n) for n in (30, 45, 28, 50)]
    llm = LLM(d, dtype="float32", block_size=16, num_kv_blocks=9, max_num_batched_tokens=64, max_num_seqs=4, max_chunk_tokens=32,
              max_model_len=128)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy_generate(d, p, 24)
    llm.runner.cache.check_invariants()


def test_trace_replay_command_line(dg_dirs, tmp_path):
    d = dg_dirs["dg_c"]
    toks = dm.random_tokens(150, 70, 8)
    tb = TraceBuilder()
    portions(tb, "r", toks, sizes=(2, 5, 2, 31))
    out = run_trace(d, "float32", tb.steps, 128, str(tmp_path / "o"), ["--block-size", "16", "--state-slots", "1"])
    check(rows_by_position(tb.steps, out), {"r": plain.forward(d, toks).float()}, "float32")


def test_the_example_command_line_with_a_pool_sized_from_free_memory(dg_dirs):
    """`example <model_dir>`: the registry picks the design by config.json, the pool is sized from what the device has left
    after the weights and the per-request state, and the completion is the plain implementation's."""
    import ast
    import os
    import subprocess
    import sys
    d = dg_dirs["dg_a"]
    prompt = dm.random_tokens(97, 9, 77)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "example"), d, "--dtype", "float32", "--prompt", ",".join(map(str, prompt)),
                        "--temperature", "0", "--max-tokens", "5", "--ignore-eos", "--max-num-seqs", "4", "--max-model-len", "64",
                        "--max-num-batched-tokens", "64", "--block-size", "16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("Completion:")][0]
    assert ast.literal_eval(line[len("Completion:"):].strip()) == plain.greedy_generate(d, prompt, 5)
