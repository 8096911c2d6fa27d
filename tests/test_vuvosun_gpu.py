"""The Vuvosun design on the GPU against its plain restatement (`plain_vuvosun.py`):
whole models through the trace replayer in every way of cutting, and generation through
the entry point."""
import numpy as np
import pytest
import torch

import helpers
import plain_vuvosun as plain
import vuvosun_cases as cases
from helpers import TOLERANCE, Trace

pytestmark = pytest.mark.gpu

LENGTHS = {"vu-a": [5, 41, 97, 150], "vu-b": [1, 33, 70], "vu-c": [19, 64, 131]}


def _requests(name):
    vocab = cases.CASES[name]["config"]["vocab"]
    return {f"r{i}": helpers.random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name])}


def _reference(model_dir, requests):
    config, tensors = plain.read_folder(model_dir)
    return {rid: plain.forward(config, tensors, tokens).numpy() for rid, tokens in requests.items()}


def _replay(name, dtype, model_dir, trace, out_dir, max_tokens):
    engine = helpers.replay_in_process(model_dir, dtype, trace, out_dir, max_tokens,
                                       cases.CASES[name]["page_tokens"])
    vocab = cases.CASES[name]["config"]["vocab"]
    return engine, helpers.collect(trace, out_dir, vocab)


def _compare(name, dtype, got, ref):
    assert got, "the trace asked for nothing"
    for rid in sorted({k[0] for k in got}):
        for key in sorted(k for k in got if k[0] == rid):
            base = rid.split("#")[0]
            e = helpers.relative_error(got[key], ref[base][key[1]])
            assert e <= TOLERANCE[dtype], (f"{name} {dtype}: request {rid} first differs at position "
                                           f"{key[1]} (relative error {e:.3g})")


def _whole(requests):
    trace = Trace()
    for rid, tokens in requests.items():
        trace.step([(rid, tokens, list(range(len(tokens))))], end=[rid])
    return trace


def _decode(requests, tail):
    trace = Trace()
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        trace.step([(rid, tokens[:head], [head - 1])], end=[rid] if head == len(tokens) else [])
        for i in range(head, len(tokens)):
            trace.step([(rid, [tokens[i]], [0])], end=[rid] if i == len(tokens) - 1 else [])
    return trace


def _portions(requests, sizes):
    trace = Trace()
    for rid, tokens in requests.items():
        at, k = 0, 0
        while at < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            trace.step([(rid, tokens[at:at + n], list(range(n)))], end=[rid] if at + n == len(tokens) else [])
            at += n
    return trace


def _mixed(requests):
    """Up to four live requests; portions of some beside single tokens of others; a
    request that ends makes room for one that runs a second time in its slot and pages."""
    order = list(requests) + [rid + "#2" for rid in list(requests)[:2]]
    tokens_of = lambda rid: requests[rid.split("#")[0]]
    fed = {rid: 0 for rid in order}
    live, waiting = [], list(order)
    trace = Trace()
    sizes = [2, 13, 1, 29, 3, 1, 1, 16, 7]
    k = 0
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, end = [], []
        for j, rid in enumerate(list(live)):
            if (k + j) % 5 == 4 and len(live) > 1:
                continue                                  # left out of this step, goes on later
            tokens = tokens_of(rid)
            n = min(sizes[(k + 3 * j) % len(sizes)], len(tokens) - fed[rid])
            entries.append((rid, tokens[fed[rid]:fed[rid] + n], list(range(n))))
            fed[rid] += n
            if fed[rid] == len(tokens):
                end.append(rid)
                live.remove(rid)
        k += 1
        if entries:
            trace.step(entries, end=end)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_every_way_of_cutting_agrees_with_the_plain_model(tmp_path, name, dtype):
    model_dir = cases.make_folder(tmp_path, name)
    requests = _requests(name)
    ref = _reference(model_dir, requests)
    longest = -(-max(LENGTHS[name]) // 64) * 64
    results = {}
    for label, trace, room in [("whole", _whole(requests), longest),
                               ("decode", _decode(requests, 60), longest),
                               ("portions", _portions(requests, [2, 37, 3, 16, 5, 2, 64]), longest),
                               ("mixed", _mixed(requests), 4 * longest)]:
        engine, got = _replay(name, dtype, model_dir, trace, str(tmp_path / label), room)
        _compare(name, dtype, got, ref)
        results[label] = got
        if label == "mixed":
            assert engine.cache.slots.free_slots == 4           # everything was given back
    if dtype == "float32":
        # the same position, however the prompt was cut and whatever else was in the batch
        for label in ("decode", "portions", "mixed"):
            for key, row in results[label].items():
                base = (key[0].split("#")[0], key[1])
                if base in results["whole"]:
                    assert np.array_equal(row, results["whole"][base]), (name, label, key)


def test_steps_are_replayed_as_graphs(tmp_path):
    model_dir = cases.make_folder(tmp_path, "vu-a")
    requests = {"r0": helpers.random_tokens(300, 90, 1)}
    engine, got = _replay("vu-a", "bfloat16", model_dir, _decode(requests, 70), str(tmp_path / "o"), 128)
    assert not engine._graph_failed, engine._graph_error
    assert engine._graph_replays >= 60
    _compare("vu-a", "bfloat16", got, _reference(model_dir, requests))


def test_long_decoding_past_window_and_pages(tmp_path):
    """Two tokens of prompt, then 200 decoded ones: the window (24) passes over decoded
    tokens many times, pages of passed keys go back while the first tokens' page stays."""
    model_dir = cases.make_folder(tmp_path, "vu-a")
    requests = {"r0": helpers.random_tokens(300, 202, 7)}
    ref = _reference(model_dir, requests)
    for dtype in ("float32", "bfloat16"):
        engine, got = _replay("vu-a", dtype, model_dir, _decode(requests, 200), str(tmp_path / dtype), 256)
        _compare("vu-a", dtype, got, ref)


def test_decoding_with_a_long_window_deals_the_keys_to_several_blocks(tmp_path):
    """A window of 150 keys and two kept tokens: decoded tokens' key tiles are split over
    blocks and merged (bfloat16, keys and values of one size)."""
    import copy
    config = copy.deepcopy(cases.CASES["vu-c"]["config"])
    for layer in config["layers"]:
        layer["mixer"]["left"]["mask"] = {"size": 150, "keep_first": 2}
    model_dir = cases.make_folder(tmp_path, "vu-long", config=config, seed=6)
    requests = {"r0": helpers.random_tokens(400, 330, 3), "r1": helpers.random_tokens(400, 200, 4)}
    ref = _reference(model_dir, requests)
    for dtype in ("bfloat16", "float32"):
        trace = Trace()
        trace.step([("r0", requests["r0"][:250], [249]), ("r1", requests["r1"][:120], [119])])
        for i in range(80):
            trace.step([("r0", [requests["r0"][250 + i]], [0]), ("r1", [requests["r1"][120 + i]], [0])],
                       end=["r0", "r1"] if i == 79 else [])
        engine = helpers.replay_in_process(model_dir, dtype, trace, str(tmp_path / dtype), 640, 8)
        got = helpers.collect(trace, str(tmp_path / dtype), 400)
        _compare("vu-long", dtype, got, ref)


def test_window_pages_go_back_and_kept_first_pages_stay(tmp_path):
    from crucible_b200.engine.engine import Engine, EngineOptions, StepEntry
    model_dir = cases.make_folder(tmp_path, "vu-a")
    engine = Engine(model_dir, EngineOptions(dtype="float32", page_tokens=16, n_pages=20, max_requests=2))
    tokens = helpers.random_tokens(300, 150, 9)
    engine.step([StepEntry("a", tokens[:100], [])])
    engine.step([StepEntry("a", tokens[100:], [])])
    table = engine.cache.block_table("a", 0)
    assert table[0] >= 0                                  # holds the kept first tokens
    # the second step began at position 100, whose window (24) reaches back to 77
    assert table[1] == -1 and table[2] == -1 and table[3] == -1 and table[4] >= 0
    assert table[-1] >= 0 and table[-2] >= 0
    engine.cache.check_invariants()
    engine.finish("a")
    assert engine.cache.free_pages(0) == 20 and engine.cache.free_pages(1) == 20


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    from crucible_b200 import LLM, SamplingParams
    model_dir = cases.make_folder(tmp_path, name)
    config, tensors = plain.read_folder(model_dir)
    vocab = config["vocab"]
    prompts = [helpers.random_tokens(vocab, n, 50 + n) for n in (3, 45, 18)]
    want = [plain.greedy(config, tensors, p, 12) for p in prompts]
    llm = LLM(model_dir, dtype="float32", kv_pages=64, max_batch=4, prefill_token_budget=32,
              page_tokens=cases.CASES[name]["page_tokens"])
    got = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    assert got == want
    llm16 = LLM(model_dir, dtype="bfloat16", kv_pages=64, max_batch=4, prefill_token_budget=32,
                page_tokens=cases.CASES[name]["page_tokens"])
    got16 = llm16.generate(prompts, SamplingParams(max_tokens=4, temperature=0.0))
    # bfloat16 may part from the plain model where two logits are close; the first tokens
    # of most prompts agree
    assert sum(g[:1] == w[:1] for g, w in zip(got16, want)) >= 2


def test_config_values_that_another_model_makes_equal_or_absent(tmp_path):
    """No window and no rotation on the left, kv_heads == heads, one tap, odd sizes whose
    products cannot run on tensor cores, eight streams."""
    left = {"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.3, "rot": None, "mask": None}
    right = {"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 1}
    config = {"architecture": "Vuvosun", "vocab": 97, "width": 44, "streams": 8, "norm": {"eps": 1e-4},
              "layers": [{"type": "parallel", "mlp": {"kind": "dense", "ff": 52},
                          "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 1.0}}]}
    model_dir = cases.make_folder(tmp_path, "odd", config=config, seed=11)
    requests = {"r0": helpers.random_tokens(97, 70, 1), "r1": helpers.random_tokens(97, 9, 2)}
    ref = _reference(model_dir, requests)
    for dtype in ("float32", "bfloat16"):
        trace = _portions(requests, [2, 9, 1, 30])
        engine = helpers.replay_in_process(model_dir, dtype, trace, str(tmp_path / dtype), 128, 16)
        got = helpers.collect(trace, str(tmp_path / dtype), 97)
        for key, row in got.items():
            assert helpers.relative_error(row, ref[key[0]][key[1]]) <= TOLERANCE[dtype], (dtype, key)


def test_a_design_without_a_context_limit_is_bounded_by_the_engine(tmp_path):
    from crucible_b200.engine.engine import Engine, EngineOptions, StepEntry, StepError
    model_dir = cases.make_folder(tmp_path, "vu-b")
    engine = Engine(model_dir, EngineOptions(dtype="float32", page_tokens=32, n_pages=4, max_requests=2))
    assert engine.max_context == 128                      # what its pages hold
    tokens = helpers.random_tokens(211, 129, 1)
    with pytest.raises(StepError):
        engine.step([StepEntry("a", tokens, [])])
    assert not engine.has_request("a") and engine.cache.slots.free_slots == 2
    engine.step([StepEntry("a", tokens[:128], [127])])
    with pytest.raises(StepError):
        engine.step([StepEntry("a", tokens[128:], [0])])
    assert engine.held_tokens("a") == 128
    bounded = Engine(model_dir, EngineOptions(dtype="float32", page_tokens=32, n_pages=8, max_requests=2,
                                              max_context=40))
    assert bounded.max_context == 40
    with pytest.raises(StepError):
        bounded.step([StepEntry("a", tokens[:41], [])])
