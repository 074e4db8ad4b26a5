"""The Sebalorn design without a GPU: its config reader and the errors it gives, the run order
of a repeated run of layers, tensor names and shapes, storage planning (a slot in the pages and
a state of its own for every pass), the random folder, and the plain model's own rules."""
import copy

import pytest
import torch

import plain_sebalorn as plain
import sebalorn_cases as cases
from crucible_b200.config.model_config import ConfigError, ModelConfig, RunEntry
from crucible_b200.config.registry import known_architectures, parse_config
from crucible_b200.models.decoder import DecoderModel


def _config(name="se-a"):
    return copy.deepcopy(cases.CASES[name]["config"])


def test_the_architecture_is_registered_and_parsed():
    assert "Sebalorn" in known_architectures()
    cfg = parse_config(_config())
    assert (cfg.vocab_size, cfg.hidden_size, cfg.tie_word_embeddings) == (300, 64, False)
    kinds = [(layer.arrangement, layer.mixer.kind, layer.feed_forward.kind) for layer in cfg.layers]
    assert kinds == [("parallel", "retention", "dense_act"), ("parallel", "sink_attention", "dense_act"),
                     ("parallel", "latent_attention", "none"), ("parallel", "retention", "dense_act"),
                     ("parallel", "sink_attention", "dense_act")]
    assert all([name for name, _ in layer.norms] == ["norm"] and layer.norms[0][1].kind == "rmsnorm_offset"
               for layer in cfg.layers)
    r = cfg.layers[0].mixer
    assert (r.n_heads, r.head_dim, r.option("value_dim"), r.option("decay")) == (4, 16, 24, (0.9, 0.99, 1.0, 0.5))
    assert (r.position.kind, r.position.rotary_dim, r.position.theta) == ("rope_halves", 8, 10000.0)
    a = cfg.layers[1].mixer
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.option("value_dim"), a.softmax_scale, a.window,
            a.option("sink"), a.option("gate"), a.option("qk_norm_eps"), a.option("qk_norm_whole")) == \
        (4, 2, 16, 24, 0.5, None, False, "head", 1e-6, True)
    assert cfg.layers[4].mixer.n_kv_heads == 2          # no `kv_heads`: as many as heads
    b = cfg.layers[2].mixer
    assert (b.n_heads, b.head_dim, b.option("rot_dim"), b.option("value_dim"), b.option("kv_rank"),
            b.option("q_rank"), b.window, b.option("gate"), b.option("sink")) == \
        (2, 24, 8, 16, 40, 24, None, "element", True)
    assert b.position.kind == "rope_interleaved"
    assert cfg.layers[0].feed_forward.option("activation") == "relu2"
    assert cfg.embedding.kind == "token_hashed_positions" and cfg.embedding.option("scale") == 8.0
    assert cfg.head.option("softcap") == 20.0
    # layers 1..3 twice: each pass a copy, the pass's vector before its first layer
    assert [(e.layer, e.copy, e.add) for e in cfg.run_order] == [
        (0, 0, None), (1, 0, ("loop_step", 0)), (2, 0, None), (3, 0, None),
        (1, 1, ("loop_step", 1)), (2, 1, None), (3, 1, None), (4, 0, None)]
    assert cfg.vectors == (("loop_step", 2),)


def test_a_model_without_a_repeated_run_and_without_a_cap():
    cfg = parse_config(_config("se-d"))
    assert [(e.layer, e.copy, e.add) for e in cfg.run_order] == [(0, 0, None), (1, 0, None), (2, 0, None)]
    assert cfg.vectors == ()
    assert parse_config(_config("se-b")).head.option("softcap") is None
    latent = cfg.layers[2].mixer
    assert latent.option("rot_dim") == 0 and latent.position is None
    # an empty run repeats nothing; its table of vectors is still one of the model's tensors
    empty = _config()
    empty["loop"].update(start=2, stop=2, times=3)
    cfg = parse_config(empty)
    assert [(e.layer, e.copy, e.add) for e in cfg.run_order] == [(i, 0, None) for i in range(5)]
    assert cfg.vectors == (("loop_step", 3),)


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5, 1.5, 0.1]), "decay"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda c: c["loop"].update(stop=9), "stop"),
    (lambda c: c["loop"].update(start=5), "start"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_config_errors_name_the_key(edit, word):
    config = _config()
    edit(config)
    with pytest.raises(ConfigError) as e:
        parse_config(config)
    assert word in str(e.value)


def test_tensor_names_shapes_and_storage():
    model = DecoderModel(parse_config(_config()))
    shapes = {r.checkpoint_name: tuple(r.decl.shape) for r in model.tensor_requests()}
    assert shapes["embed"] == (300, 64) and shapes["head"] == (300, 64) and shapes["final.norm"] == (64,)
    assert shapes["loop.step"] == (2, 64)
    assert shapes["l1.mix.q"] == (64, 64) and shapes["l1.mix.k"] == (32, 64) and shapes["l1.mix.v"] == (48, 64)
    assert shapes["l1.mix.q.norm"] == (64,) and shapes["l1.mix.k.norm"] == (32,)       # over all heads
    assert shapes["l1.mix.g"] == (4, 64) and shapes["l1.mix.o"] == (64, 96)              # a logit a head
    assert shapes["l2.mix.dq"] == (24, 64) and shapes["l2.mix.uq"] == (2 * 32, 24)
    assert shapes["l2.mix.dkv"] == (48, 64) and shapes["l2.mix.dkv.norm"] == (40,)
    assert shapes["l2.mix.uk"] == (48, 40) and shapes["l2.mix.uv"] == (32, 40) and shapes["l2.mix.sink"] == (2,)
    assert shapes["l2.mix.g"] == (32, 64) and "l2.mlp.up" not in shapes
    assert shapes["l3.mix.q"] == (48, 64) and shapes["l3.mix.v"] == (16, 64) and shapes["l3.mix.g"] == (16, 64)
    assert shapes["l0.mlp.up"] == (96, 64) and shapes["l0.mlp.down"] == (64, 96)
    assert "l0.mix.norm" not in shapes and "l3.mix.decay" not in shapes       # the decays are numbers of the config
    # the repeated layers have a slot for every pass; the retention layers a state for every run
    by_need = {g.need.head_dim: g.layers for g in model.cache_groups}
    assert by_need[16] == (1, 1) and by_need[48] == (2, 2) and by_need[32] == (4,)
    runs = list(zip(model.config.run_order, model.bindings))
    slots = {(e.layer, e.copy): (b.group, b.slot) for e, b in runs if b.group is not None}
    assert len(set(slots.values())) == len(slots) == 5
    states = [(e.layer, e.copy, b.state_offset, b.state_bytes) for e, b in runs if b.state_bytes]
    assert [(l, c) for l, c, _, _ in states] == [(0, 0), (3, 0), (3, 1)]
    ends = sorted((off, off + n) for _, _, off, n in states)
    assert all(a[1] <= b[0] for a, b in zip(ends, ends[1:])) and ends[-1][1] <= model.state_bytes
    assert states[0][3] == 4 * 4 * 16 * 24 and states[1][3] == 4 * 2 * 24 * 8


def test_run_order_rules_of_the_generic_model():
    """A layer that runs twice writes its own cache twice unless its entries name copies; an
    added vector must be one the model holds."""
    cfg = parse_config(_config())
    twice = ModelConfig(**{**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__},
                           "run_order": (RunEntry(0), RunEntry(1), RunEntry(1))})
    with pytest.raises(ConfigError) as e:
        DecoderModel(twice.validate())
    assert "second" in str(e.value)
    state_twice = ModelConfig(**{**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__},
                                 "run_order": (RunEntry(0), RunEntry(0))})
    with pytest.raises(ConfigError) as e:
        DecoderModel(state_twice.validate())
    assert "same state" in str(e.value)
    bad = ModelConfig(**{**{f: getattr(cfg, f) for f in cfg.__dataclass_fields__},
                         "run_order": (RunEntry(0, add=("loop_step", 2)),)})
    with pytest.raises(ConfigError) as e:
        bad.validate()
    assert "loop_step" in str(e.value)


def test_the_random_folder_is_read_back_by_the_plain_model(tmp_path):
    for name in sorted(cases.CASES):
        folder = cases.make_folder(tmp_path, name)
        config, tensors = plain.load_folder(folder)
        assert config["architecture"] == "Sebalorn"
        model = DecoderModel(parse_config(config))
        assert {r.checkpoint_name: tuple(r.decl.shape) for r in model.tensor_requests()} == \
            {k: tuple(v.shape) for k, v in tensors.items()}
        logits = plain.forward(config, tensors, [1, 2, 3, 4, 5])
        assert tuple(logits.shape) == (5, config["vocab"]) and bool(torch.isfinite(logits).all())
        cap = config.get("logit_softcap")
        if cap:
            assert float(logits.abs().max()) < cap


def test_plain_rules():
    # the run list of a repeated run
    config = {"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 3}}
    assert plain.run_list(config) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False),
                                      (1, 2, True), (2, 2, False), (3, None, False)]
    # both pairings turn a vector without changing its length, and differ
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    pos = torch.arange(5) + 3
    a, b = plain.turn_halves(x, pos, 8, 100.0), plain.turn_neighbours(x, pos, 8, 100.0)
    assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1)) and torch.allclose(b.norm(dim=-1), x.norm(dim=-1))
    assert torch.equal(a[..., 8:], x[..., 8:]) and not torch.allclose(a, b)
    # pair (0, 4) of the split halves at position 3 turns by 3 radians (frequency 1)
    u, v = x[0, 0, 0], x[0, 0, 4]
    c, s = torch.cos(torch.tensor(3.0, dtype=torch.float64)), torch.sin(torch.tensor(3.0, dtype=torch.float64))
    assert torch.allclose(a[0, 0, 0], u * c - v * s) and torch.allclose(a[0, 0, 4], v * c + u * s)
    assert torch.allclose(b[0, 0, 0], x[0, 0, 0] * c - x[0, 0, 1] * s)
    # a row's weights and the sink's share add up to one
    scores = torch.randn(2, 6, 6, dtype=torch.float64)
    sink = torch.tensor([0.3, -2.0], dtype=torch.float64)
    p = plain.causal_weights(scores, sink)
    top = torch.maximum(scores.masked_fill(~torch.ones(6, 6, dtype=torch.bool).tril(), -1e30).max(-1).values, sink[:, None])
    rest = torch.exp(sink[:, None] - top) / (torch.exp(scores - top[..., None]).tril().sum(-1) + torch.exp(sink[:, None] - top))
    assert torch.allclose(p.sum(-1) + rest, torch.ones(2, 6, dtype=torch.float64))
    assert float(p[0, 2, 3:].abs().max()) == 0.0
    # the retention's recurrence equals the sum over earlier tokens with powers of the decay
    t, H, D, E = 7, 2, 4, 3
    m = {"heads": H, "dim": D, "vdim": E, "decay": [0.5, 0.9], "rot": None}
    g = torch.Generator().manual_seed(0)
    w = {"q": torch.randn(H * D, 6, generator=g, dtype=torch.float64), "k": torch.randn(H * D, 6, generator=g, dtype=torch.float64),
         "v": torch.randn(H * E, 6, generator=g, dtype=torch.float64), "g": torch.randn(H * E, 6, generator=g, dtype=torch.float64),
         "o": torch.eye(H * E, dtype=torch.float64)}
    h = torch.randn(t, 6, generator=g, dtype=torch.float64)
    got = plain.retention(h, w, m, 1e-6, "")
    q, k, v = (h @ w["q"].T).view(t, H, D), (h @ w["k"].T).view(t, H, D) * D ** -0.5, (h @ w["v"].T).view(t, H, E)
    decay = torch.tensor(m["decay"], dtype=torch.float64)
    o = torch.zeros(t, H, E, dtype=torch.float64)
    for i in range(t):
        for j in range(i + 1):
            o[i] += decay[:, None] ** (i - j) * (q[i] * k[j]).sum(-1, keepdim=True) * v[j]
    z = h @ w["g"].T
    assert torch.allclose(got, plain.unit_rms(o, 1e-6).reshape(t, H * E) * z * plain.sigmoid(z))
