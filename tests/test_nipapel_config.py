"""The Nipapel design without a GPU: its config reader and the errors it gives, tensor names
and shapes, storage planning (who owns pages, who reads them, for which window they are
kept), the random folder, and the plain model's own rules."""
import copy

import pytest
import torch

import nipapel_cases as cases
import plain_nipapel as plain
from crucible_b200.config.model_config import ConfigError
from crucible_b200.config.registry import known_architectures, parse_config
from crucible_b200.models.decoder import DecoderModel


def _config(name="ni-a"):
    return copy.deepcopy(cases.CASES[name]["config"])


def test_the_architecture_is_registered_and_parsed():
    assert "Nipapel" in known_architectures()
    cfg = parse_config(_config())
    assert (cfg.vocab_size, cfg.hidden_size, cfg.tie_word_embeddings) == (300, 64, False)
    kinds = [(layer.arrangement, layer.mixer.kind, layer.feed_forward.kind) for layer in cfg.layers]
    assert kinds == [("parallel", "sink_attention", "moe"), ("parallel", "latent_attention", "glu_capped"),
                     ("parallel", "latent_attention", "moe"), ("parallel", "sink_attention", "none"),
                     ("parallel", "latent_attention", "glu_capped")]
    assert all([name for name, _ in layer.norms] == ["norm"] and layer.norms[0][1].kind == "rmsnorm_offset"
               for layer in cfg.layers)
    a = cfg.layers[0].mixer
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.option("value_dim"), a.softmax_scale, a.window,
            a.option("keep_first"), a.option("sink"), a.option("gate"), a.option("qk_norm_eps")) == \
        (4, 2, 16, 24, 0.3, 20, 3, False, False, 1e-6)
    assert (a.position.kind, a.position.rotary_dim, a.position.theta) == ("rope_halves", 8, 10000.0)
    assert cfg.layers[3].mixer.n_kv_heads == 2 and cfg.layers[3].mixer.option("keep_first") == 0
    b = cfg.layers[1].mixer
    assert (b.n_heads, b.head_dim, b.option("rot_dim"), b.option("value_dim"), b.option("kv_rank"),
            b.option("q_rank"), b.window, b.option("gate"), b.option("reads_other")) == \
        (2, 24, 8, 16, 40, 24, 33, "element", False)
    assert b.position.kind == "rope_interleaved"
    # the reader's window is wider than its owner's: the pages are kept for the wider one
    assert cfg.layers[2].mixer.option("reads_other") and cfg.layers[2].mixer.window == 50
    assert b.option("cache_window") == 50 and cfg.layers[2].mixer.option("cache_window") == 50
    assert [(e.layer, e.cache_of) for e in cfg.run_order] == [(0, None), (1, None), (2, 1), (3, None), (4, None)]
    moe = cfg.layers[0].feed_forward
    assert (moe.option("experts"), moe.option("top"), moe.intermediate, moe.option("router_bias"),
            moe.option("pair")) == (6, 2, 40, True, (1.5, 1.702, 1.0))
    assert cfg.layers[1].feed_forward.option("limit") == 0.8
    assert cfg.embedding.kind == "token_normed_streams" and cfg.embedding.option("gain_offset") == 1.0


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),          # itself
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),          # not a latent layer
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),          # a reader, not an owner
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=48), "kv_rank"),         # differs from its owner's
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
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
    assert shapes["embed"] == (300, 64) and shapes["embed.norm"] == (64,) and shapes["head"] == (300, 64)
    assert shapes["final.norm"] == (64,) and shapes["l0.norm1"] == (64,) and "l0.norm2" not in shapes
    assert shapes["l0.mix.q"] == (64, 64) and shapes["l0.mix.k"] == (32, 64) and shapes["l0.mix.v"] == (48, 64)
    assert shapes["l0.mix.q.norm"] == (16,) and shapes["l0.mix.k.norm"] == (16,) and shapes["l0.mix.o"] == (64, 96)
    assert "l0.mix.sink" not in shapes and "l0.mix.g" not in shapes
    assert shapes["l1.mix.dq"] == (24, 64) and shapes["l1.mix.dq.norm"] == (24,) and shapes["l1.mix.uq"] == (64, 24)
    assert shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.dkv.norm"] == (40,)
    assert shapes["l1.mix.uk"] == (48, 40) and shapes["l1.mix.uv"] == (32, 40) and shapes["l1.mix.g"] == (32, 64)
    assert "l2.mix.dkv" not in shapes and "l2.mix.dkv.norm" not in shapes and shapes["l2.mix.uk"] == (72, 40)
    assert shapes["l0.mlp.router"] == (6, 64) and shapes["l0.mlp.router.b"] == (6,)
    assert shapes["l0.mlp.e5.down"] == (64, 40) and shapes["l1.mlp.gate"] == (96, 64)
    assert not any(name.startswith("l3.mlp") for name in shapes)
    # pages: the two attentions differ in everything; layers 1 and 4 cache rows of other sizes;
    # layer 2 owns nothing and reads layer 1's slot
    needs = [(g.need.kv_heads, g.need.head_dim, g.need.window, g.need.keep_first, g.need.value_dim,
              g.need.values_are_keys, g.layers) for g in model.cache_groups]
    assert needs == [(2, 16, 20, 3, 24, False, (0,)), (1, 48, 50, 0, None, True, (1,)),
                     (2, 32, 9, 0, None, False, (3,)), (1, 64, 12, 0, None, True, (4,))]
    b = model.bindings
    assert (b[1].group, b[1].slot, b[1].write) == (1, 0, True) and (b[2].group, b[2].slot, b[2].write) == (1, 0, False)
    assert model.state_bytes == 0


def test_owners_with_equal_rows_share_pages_and_a_reader_without_a_window_keeps_everything():
    config = _config("ni-c")
    config["layers"].append(copy.deepcopy(config["layers"][0]))          # a second owner, same sizes
    model = DecoderModel(parse_config(config))
    latent = [g for g in model.cache_groups if g.need.values_are_keys]
    assert len(latent) == 1 and latent[0].layers == (0, 3)
    config["layers"][2]["mixer"]["mask"] = None
    cfg = parse_config(config)
    assert cfg.layers[2].mixer.window is None and cfg.layers[0].mixer.window == 70
    assert cfg.layers[0].mixer.option("cache_window", "absent") is None
    assert cfg.layers[3].mixer.option("cache_window", "absent") == "absent"


def test_the_random_folder_is_read_back_by_the_plain_model(tmp_path):
    folder = cases.make_folder(tmp_path, "ni-b")
    config, tensors = plain.read_folder(folder)
    assert config["architecture"] == "Nipapel" and tensors["l0.mix.dkv"].shape == (27, 44)
    assert float(tensors["l0.norm1"].abs().max()) < 1.0                  # weights around zero, not one
    assert float((tensors["l2.mix.q.norm"] - 1.0).abs().max()) < 1.0     # plain weights around one
    logits = plain.forward(config, tensors, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, 211) and torch.isfinite(logits).all()


def test_plain_rules():
    pos = torch.arange(12)
    seen = plain.visible(pos, 4, 2)
    assert seen[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]
    assert plain.visible(pos, 4)[9].nonzero().flatten().tolist() == [6, 7, 8, 9]
    assert plain.visible(pos, None)[5].sum() == 6
    x = torch.arange(8, dtype=torch.float64).view(1, 1, 8) + 1.0
    one = torch.tensor([1])
    halves = plain.turn_split_halves(x, one, 4, 100.0)
    pairs = plain.turn_neighbours(x, one, 4, 100.0)
    f = plain.frequencies(4, 100.0, torch.float64)
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    c, s = torch.cos(f), torch.sin(f)
    assert torch.allclose(halves[0, 0, :4], torch.stack([1 * c[0] - 3 * s[0], 2 * c[1] - 4 * s[1],
                                                         3 * c[0] + 1 * s[0], 4 * c[1] + 2 * s[1]]))
    assert torch.allclose(pairs[0, 0, :4], torch.stack([1 * c[0] - 2 * s[0], 2 * c[0] + 1 * s[0],
                                                        3 * c[1] - 4 * s[1], 4 * c[1] + 3 * s[1]]))
    assert torch.equal(halves[0, 0, 4:], x[0, 0, 4:]) and torch.equal(pairs[0, 0, 4:], x[0, 0, 4:])
    # the capped pair: the gate is capped from above only, the linear half on both sides
    h = torch.eye(3, dtype=torch.float64)
    gate = torch.tensor([[5.0, -5.0, 0.5]], dtype=torch.float64).T
    up = torch.tensor([[5.0, -5.0, 0.25]], dtype=torch.float64).T
    y = plain.capped_glu(h, gate.T.reshape(1, 3), up.T.reshape(1, 3), torch.ones(1, 1, dtype=torch.float64), 2.0)
    sig = lambda z: 1.0 / (1.0 + torch.exp(torch.tensor(-1.702 * z, dtype=torch.float64)))
    want = torch.stack([2.0 * sig(2.0) * 3.0, -5.0 * sig(-5.0) * -1.0, 0.5 * sig(0.5) * 1.25])
    assert torch.allclose(y[:, 0], want)
    # the router: the chosen logits alone are normalised, the bias moves the choice
    idx, w = plain.route(torch.eye(2, dtype=torch.float64), torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.9, 0.9]], dtype=torch.float64),
                         torch.tensor([0.0, 0.0, 0.5], dtype=torch.float64), 2)
    assert idx.tolist() == [[2, 0], [2, 1]] and torch.allclose(w.sum(-1), torch.ones(2, dtype=torch.float64))
