"""The Sebalorn design on the GPU against its plain restatement (`plain_sebalorn.py`): whole
models through the trace replayer in every way of cutting, and generation through the entry
point."""
import numpy as np
import pytest

import helpers
import plain_sebalorn as plain
import sebalorn_cases as cases
from helpers import TOLERANCE
from test_vuvosun_gpu import _decode, _mixed, _portions, _whole

pytestmark = pytest.mark.gpu

LENGTHS = {"se-a": [5, 41, 97, 150], "se-b": [1, 33, 70], "se-c": [19, 64, 171], "se-d": [2, 50, 83]}


def _requests(name):
    vocab = cases.CASES[name]["config"]["vocab"]
    return {f"r{i}": helpers.random_tokens(vocab, n, 900 + i) for i, n in enumerate(LENGTHS[name])}


def _reference(model_dir, requests):
    config, tensors = plain.load_folder(model_dir)
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


def test_every_pass_of_a_repeated_layer_has_keys_and_state_of_its_own(tmp_path):
    """Three passes over [latent attention, retention]: three slots in the latent rows' pages,
    three states; a model whose passes shared them would differ from the plain one, and the
    passes' vectors are what tells them apart."""
    from crucible_b200.config import load_config
    from crucible_b200.models.decoder import DecoderModel
    model_dir = cases.make_folder(tmp_path, "se-b")
    model = DecoderModel(load_config(model_dir))
    assert [(e.layer, e.copy) for e in model.config.run_order] == \
        [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, 0), (3, 0)]
    latent_group = model.bindings[0].group
    assert sorted(b.slot for b in model.bindings[0:6:2]) == [0, 1, 2]
    assert all(b.group == latent_group for b in model.bindings[0:6:2])
    offsets = [b.state_offset for b in model.bindings[1:6:2]]
    assert len(set(offsets)) == 3 and model.state_bytes >= 3 * model.bindings[1].state_bytes
    # the vectors matter: without them the logits move far beyond rounding
    config, tensors = plain.load_folder(model_dir)
    tokens = helpers.random_tokens(211, 40, 5)
    with_vectors = plain.forward(config, tensors, tokens)
    without = dict(tensors)
    without["loop.step"] = tensors["loop.step"] * 0
    assert helpers.relative_error(plain.forward(config, without, tokens).numpy(), with_vectors.numpy()) > 0.05


def test_steps_are_replayed_as_graphs(tmp_path):
    model_dir = cases.make_folder(tmp_path, "se-a")
    requests = {"r0": helpers.random_tokens(300, 90, 1)}
    engine, got = _replay("se-a", "bfloat16", model_dir, _decode(requests, 70), str(tmp_path / "o"), 128)
    assert not engine._graph_failed, engine._graph_error
    assert engine._graph_replays >= 60
    _compare("se-a", "bfloat16", got, _reference(model_dir, requests))


def test_prompt_steps_are_replayed_as_graphs(tmp_path):
    model_dir = cases.make_folder(tmp_path, "se-c")
    requests = {"r0": helpers.random_tokens(400, 6 * 160 + 3, 1)}
    engine, got = _replay("se-c", "bfloat16", model_dir, _portions(requests, [160]), str(tmp_path / "o"), 1024)
    assert not engine._graph_failed, engine._graph_error
    assert engine._prompt_graph_replays >= 2
    _compare("se-c", "bfloat16", got, _reference(model_dir, requests))


def test_long_decoding(tmp_path):
    """Two tokens of prompt, then 300 decoded ones over pages of 8: the retention's state is
    carried through 300 steps, the attentions' keys lie over 38 pages."""
    requests = {"r0": helpers.random_tokens(300, 302, 7)}
    for dtype in ("float32", "bfloat16"):
        model_dir = cases.make_folder(tmp_path / dtype, "se-a")
        ref = _reference(model_dir, requests)
        engine, got = _replay("se-a", dtype, model_dir, _decode(requests, 300), str(tmp_path / dtype / "out"),
                              320, page_tokens=8)
        _compare("se-a", dtype, got, ref)


def test_slots_and_pages_that_are_used_again_start_clean(tmp_path):
    """One request's worth of pages: every request runs where the one before it ran, and finds
    the retention's state at zero."""
    requests = {f"r{i}": helpers.random_tokens(300, n, 40 + i) for i, n in enumerate([60, 64, 7, 33])}
    for dtype in ("float32", "bfloat16"):
        model_dir = cases.make_folder(tmp_path / dtype, "se-a")
        ref = _reference(model_dir, requests)
        trace = _portions(requests, [3, 30, 2])
        engine = helpers.replay_in_process(model_dir, dtype, trace, str(tmp_path / dtype / "out"), 64, 16)
        _compare("se-a", dtype, helpers.collect(trace, str(tmp_path / dtype / "out"), 300), ref)
        assert engine.cache.slots.free_slots == 4


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    from crucible_b200 import LLM, SamplingParams
    model_dir = cases.make_folder(tmp_path, name)
    config, tensors = plain.load_folder(model_dir)
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
    """One pass of a "repeated" run; one head everywhere; a decay of exactly 1 and a small one (a
    head that forgets at once is the kernel tests' matter: its o = (k . q) v has the sign of one
    dot product, which the norm behind it turns into a whole sign where bfloat16 rounds it); the
    whole head turned and nothing turned; value sizes unlike key sizes on tensor-core sizes; no
    `kv_heads`; a scale of 1 and no cap; every layer without a feed-forward but one."""
    config = cases.model(97, 48, 1e-4, 1.0, None, [
        cases.retention(2, 16, 32, [1.0, 0.25], 16, 3.0, None),
        cases.latent(1, 8, 4, 12, 12, 20, 0.4, 77.0, None),
        cases.attention(1, None, 16, 32, 0.3, None, 1.0, cases.dense(16)),
        cases.attention(4, 4, 16, 16, 0.3, 16, 3.0, None)], (1, 3, 1))
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
    folder = cases.make_folder(tmp_path, "se-a")
    tool = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "bin", "llm-engine")
    proc = subprocess.run([sys.executable, tool, "generate", folder, "--prompt-ids", "5,17,3,200,5,17",
                           "--max-tokens", "6", "--temperature", "0", "--dtype", "float32", "--graph"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    config, tensors = plain.load_folder(folder)
    assert json.loads(proc.stdout.strip().splitlines()[0])["tokens"] == \
        plain.greedy(config, tensors, [5, 17, 3, 200, 5, 17], 6)
    proc = subprocess.run([sys.executable, tool, "inspect", folder], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    for word in ("Sebalorn", "retention+dense_act", "sink_attention+dense_act", "latent_attention+none"):
        assert word in proc.stdout, (word, proc.stdout)
