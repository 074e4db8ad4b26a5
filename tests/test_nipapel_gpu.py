"""The Nipapel design on the GPU against its plain restatement (`plain_nipapel.py`): whole
models through the trace replayer in every way of cutting, and generation through the entry
point."""
import copy

import numpy as np
import pytest

import helpers
import nipapel_cases as cases
import plain_nipapel as plain
from helpers import TOLERANCE
from test_vuvosun_gpu import _decode, _mixed, _portions, _whole

pytestmark = pytest.mark.gpu

# longer than every window, so that rows lose sight of keys inside prompts and while decoding
LENGTHS = {"ni-a": [5, 41, 97, 150], "ni-b": [1, 33, 70], "ni-c": [19, 64, 171]}


def _requests(name):
    vocab = cases.CASES[name]["config"]["vocab"]
    return {f"r{i}": helpers.random_tokens(vocab, n, 700 + i) for i, n in enumerate(LENGTHS[name])}


def _reference(model_dir, requests):
    config, tensors = plain.read_folder(model_dir)
    return {rid: plain.forward(config, tensors, tokens).numpy() for rid, tokens in requests.items()}


def _replay(name, dtype, model_dir, trace, out_dir, max_tokens, page_tokens=None):
    engine = helpers.replay_in_process(model_dir, dtype, trace, out_dir, max_tokens,
                                       page_tokens or cases.CASES[name]["page_tokens"])
    return engine, helpers.collect(trace, out_dir, engine.config.vocab_size)


def _compare(name, dtype, got, ref):
    assert got, "the trace asked for nothing"
    for key in sorted(got):
        base = key[0].split("#")[0]
        e = helpers.relative_error(got[key], ref[base][key[1]])
        assert e <= TOLERANCE[dtype], (f"{name} {dtype}: request {key[0]} first differs at position "
                                       f"{key[1]} (relative error {e:.3g})")


def _folder(tmp_path, name, dtype):
    """The case's folder.  In bfloat16 the router reads rounded rows, so where two experts'
    logits are close a token goes to another expert than in the plain model and its logits
    differ by more than rounding.  The bfloat16 runs therefore route every token to all
    experts (`top` = `experts`: the weights are still the softmax of the logits); which
    experts are chosen is the float32 runs' matter and the router's own test's."""
    config = copy.deepcopy(cases.CASES[name]["config"])
    if dtype == "bfloat16":
        for layer in config["layers"]:
            if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cases.make_folder(tmp_path, name, config=config, seed=cases.CASES[name]["seed"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_every_way_of_cutting_agrees_with_the_plain_model(tmp_path, name, dtype):
    model_dir = _folder(tmp_path, name, dtype)
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
    model_dir = _folder(tmp_path, "ni-a", "bfloat16")
    requests = {"r0": helpers.random_tokens(300, 90, 1)}
    engine, got = _replay("ni-a", "bfloat16", model_dir, _decode(requests, 70), str(tmp_path / "o"), 128)
    assert not engine._graph_failed, engine._graph_error
    assert engine._graph_replays >= 60
    _compare("ni-a", "bfloat16", got, _reference(model_dir, requests))


def test_prompt_steps_with_experts_are_replayed_as_graphs(tmp_path):
    """Portions of a fixed size repeat their shape: from the second time on they are replayed,
    experts and all (nothing of the routing comes to the host)."""
    model_dir = _folder(tmp_path, "ni-c", "bfloat16")
    requests = {"r0": helpers.random_tokens(400, 6 * 160 + 3, 1)}
    engine, got = _replay("ni-c", "bfloat16", model_dir, _portions(requests, [160]), str(tmp_path / "o"), 1024)
    assert not engine._graph_failed, engine._graph_error
    assert engine._prompt_graph_replays >= 2
    _compare("ni-c", "bfloat16", got, _reference(model_dir, requests))


def test_long_decoding_past_every_window(tmp_path):
    """Two tokens of prompt, then 300 decoded ones: every window passes over decoded tokens many
    times, the pages behind it go back to the pool while the kept first tokens' pages stay."""
    requests = {"r0": helpers.random_tokens(300, 302, 7)}
    for dtype in ("float32", "bfloat16"):
        model_dir = _folder(tmp_path / dtype, "ni-a", dtype)
        ref = _reference(model_dir, requests)
        engine, got = _replay("ni-a", dtype, model_dir, _decode(requests, 300), str(tmp_path / dtype / "out"),
                              320, page_tokens=8)
        _compare("ni-a", dtype, got, ref)


def test_slots_and_pages_that_are_used_again_start_clean(tmp_path):
    """One request's worth of pages: every request runs where the one before it ran."""
    requests = {f"r{i}": helpers.random_tokens(300, n, 40 + i) for i, n in enumerate([60, 64, 7, 33])}
    for dtype in ("float32", "bfloat16"):
        model_dir = _folder(tmp_path / dtype, "ni-a", dtype)
        ref = _reference(model_dir, requests)
        trace = _portions(requests, [3, 30, 2])
        engine = helpers.replay_in_process(model_dir, dtype, trace, str(tmp_path / dtype / "out"), 64, 16)
        _compare("ni-a", dtype, helpers.collect(trace, str(tmp_path / dtype / "out"), 300), ref)
        assert engine.cache.slots.free_slots == 4


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
    """A window of one token; a window wider than any request; kept first tokens beyond the
    window's reach and more of them than a page; no rotation at all on one attention and the
    whole head turned on another; a value size unlike the key size on tensor-core sizes; a
    reader between two attentions; top == experts; every layer without a feed-forward but one."""
    config = {"architecture": "Nipapel", "vocab": 97, "width": 48, "norm": {"eps": 1e-4},
              "layers": [cases.latent(2, 8, 4, 8, 12, 8, 0.4, 77.0, 1, None),
                         cases.attention(2, 1, 16, 32, 0.3, 0, 1.0, 1000, 0, None),
                         cases.latent(1, 8, 4, 12, 12, 20, 0.4, 77.0, 1000, cases.moe(2, 2, 16, 0.7), kv_from=0),
                         cases.attention(4, 4, 16, 16, 0.3, 16, 3.0, 3, 11, None)]}
    model_dir = cases.make_folder(tmp_path, "odd", config=config, seed=11)
    requests = {"r0": helpers.random_tokens(97, 70, 1), "r1": helpers.random_tokens(97, 9, 2)}
    ref = _reference(model_dir, requests)
    for dtype in ("float32", "bfloat16"):
        trace = _portions(requests, [2, 9, 1, 30])
        helpers.replay_in_process(model_dir, dtype, trace, str(tmp_path / dtype), 128, 8)
        _compare("odd", dtype, helpers.collect(trace, str(tmp_path / dtype), 97), ref)


def test_command_line(tmp_path):
    import json
    import os
    import subprocess
    import sys
    folder = cases.make_folder(tmp_path, "ni-a")
    tool = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "bin", "llm-engine")
    proc = subprocess.run([sys.executable, tool, "generate", folder, "--prompt-ids", "5,17,3,200,5,17",
                           "--max-tokens", "6", "--temperature", "0", "--dtype", "float32", "--graph"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    config, tensors = plain.read_folder(folder)
    assert json.loads(proc.stdout.strip().splitlines()[0])["tokens"] == plain.greedy(config, tensors, [5, 17, 3, 200, 5, 17], 6)
    proc = subprocess.run([sys.executable, tool, "inspect", folder], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    for word in ("Nipapel", "sink_attention+moe", "latent_attention+glu_capped", "sink_attention+none",
                 "token_normed_streams", "cache groups   4"):
        assert word in proc.stdout, (word, proc.stdout)
