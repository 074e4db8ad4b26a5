"""Each mechanism of the Sebalorn design alone: its part, driven over hand-made steps, against
the one-mechanism functions of `plain_sebalorn.py`.  Inputs are made so that a fault shows: the
softmax is made sharp, so that a row's result is the value of its best key wherever that lies
(far back, across page borders, the row itself); sinks are large on one head and negligible on
another; decays of exactly 1 keep the first token in the state for ever."""
import pytest
import torch

import plain_sebalorn as plain
from test_futepel_kernels_gpu import DEV, TOL, Steps, _bind, _binding, _i32, rel
from test_nipapel_kernels_gpu import StepsWithValues, _cuts, _run_part

pytestmark = pytest.mark.gpu


def _beside(cuts, slot, length, each):
    """Steps of slot 0's portions `cuts`, with `each` tokens of another request beside every
    one of them until its `length` tokens are through (alone, if slot 0 is done first)."""
    schedule, left = [], length
    for n in cuts:
        entry = [(0, n)]
        if left:
            m = min(left, each)
            entry.append((slot, m))
            left -= m
        schedule.append(entry)
    while left:
        m = min(left, each)
        schedule.append([(slot, m)])
        left -= m
    return schedule


def _position(kind, dims, base):
    from crucible_b200.config.model_config import PositionSpec
    return PositionSpec(kind=kind, rotary_dim=dims, theta=base, max_positions=0) if dims else None


# ---------------------------------------------------------------------------
# the small things: a vector on every row, the cap of the logits, the scaled embedding
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("rows,width", [(1, 40), (77, 320), (300, 1100)])
def test_vector_added_to_every_row(rows, width):
    from crucible_b200 import ops
    x, v = torch.randn(rows, width), torch.randn(width)
    got = x.to(DEV)
    ops.add_vector(got, v.to(DEV))
    assert torch.equal(got.cpu(), x + v)


@pytest.mark.parametrize("cap", [5.0, 30.0])
def test_soft_cap_of_the_logits(cap):
    from crucible_b200.config.model_config import EndSpec
    from crucible_b200.parts import HEADS
    for dtype in (torch.float32, torch.bfloat16):
        head = HEADS.build("linear", EndSpec("linear", (("softcap", cap),)), 130, 48, False)
        w = (torch.randn(130, 48) * 2.0).to(torch.bfloat16).float()
        head.bind({"weight": w.to(dtype).to(DEV)}, dtype, torch.device(DEV))
        rows = torch.randn(7, 48).to(torch.bfloat16).float()
        got = head.forward(Steps(dtype).ctx([(0, 7)], None), rows.to(dtype).to(DEV))
        z = rows.double() @ w.double().T
        assert float(z.abs().max()) > cap          # the cap bites
        assert rel(got, cap * torch.tanh(z / cap)) < (2e-6 if dtype == torch.float32 else 1e-2)
        assert float(got.abs().max()) <= cap


def test_embedding_rows_are_scaled():
    from crucible_b200.config.model_config import EndSpec
    from crucible_b200.parts import EMBEDDINGS
    spec = EndSpec("token_hashed_positions", (("scale", 13.25), ("bigram", None), ("max_positions", None)))
    for dtype in (torch.float32, torch.bfloat16):
        emb = EMBEDDINGS.build(spec.kind, spec, 50, 72)
        assert emb.state_bytes() == 0
        table = (torch.randn(50, 72) * 0.2).to(torch.bfloat16).float()
        emb.bind({"table": table.to(dtype).to(DEV)}, dtype, torch.device(DEV))
        ids = [3, 49, 0, 3, 17]
        x = emb.forward(Steps(dtype).ctx([(0, 5)], None), _i32(ids))
        assert x.dtype == torch.float32 and torch.equal(x.cpu(), table[ids] * 13.25)


# ---------------------------------------------------------------------------
# grouped attention: a norm over the whole projection, split-half rotation, a gate per head
# ---------------------------------------------------------------------------

def _attention_spec(H, G, D, E, R, width, scale, whole=True, gate="head"):
    from crucible_b200.config.model_config import MixerSpec
    return MixerSpec(kind="sink_attention", width=width, n_heads=H, n_kv_heads=G, head_dim=D, softmax_scale=scale,
                     window=None, position=_position("rope_halves", R, 700.0),
                     extra=(("value_dim", E), ("keep_first", 0), ("sink", False), ("gate", gate),
                            ("value_norm_eps", None), ("qk_norm_eps", 1e-5), ("qk_norm_whole", whole)))


def _attention_cfg(H, G, D, E, R, scale):
    return {"heads": H, "kv_heads": G, "dim": D, "vdim": E, "scale": scale,
            "rot": {"dims": R, "base": 700.0} if R else None}


@pytest.mark.parametrize("dtype,H,G,D,E,R,page", [
    (torch.float32, 4, 2, 16, 24, 8, 8), (torch.bfloat16, 4, 2, 16, 24, 8, 8),      # CUDA cores (E != D)
    (torch.float32, 3, 1, 20, 20, 20, 16), (torch.bfloat16, 3, 1, 20, 20, 20, 16),  # a head that is no multiple of 16
    (torch.bfloat16, 6, 2, 32, 32, 12, 16), (torch.bfloat16, 4, 4, 64, 64, 64, 16),  # mma.sync tiles
    (torch.bfloat16, 2, 1, 128, 128, 32, 32), (torch.float32, 2, 2, 64, 64, 0, 16)])
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
def test_grouped_attention_finds_its_best_key_anywhere(dtype, H, G, D, E, R, page, how):
    from crucible_b200.parts import MIXERS
    width, T, scale = 48, 330, 4.0 * D ** -0.5     # unit-rms q and k: scores of spread 4, up to about +-12
    part = MIXERS.build("sink_attention", _attention_spec(H, G, D, E, R, width, scale))
    w = _bind(part, dtype, 5, std=0.4)
    steps = StepsWithValues(dtype, part.cache_need(), page, 2, 512, seed=3)
    h_of = {0: torch.randn(T, width).to(torch.bfloat16).float(), 1: torch.randn(90, width).to(torch.bfloat16).float()}
    binding = _binding(part, group=0)
    got = _run_part(part, steps, _beside(_cuts(T, how), 1, 90, 7), h_of, width, binding)
    cfg = _attention_cfg(H, G, D, E, R, scale)
    for slot, h in h_of.items():
        ref = plain.grouped_attention(h.double(), w, cfg, 1e-5, "")
        # (a sharp softmax multiplies the rounding of bfloat16 scores: exp(12 * 2^-8) is 5 %)
        assert rel(got[slot], ref) < (TOL[dtype] if dtype == torch.float32 else 5e-2), (slot, how)
    # the softmax is sharp: many rows give a large share of their weight to one key, and those
    # keys lie all over the context (so a key that is lost anywhere shows above)
    q = plain.norm_plain(h_of[0].double() @ w["q"].T, w["q.norm"], 1e-5).view(T, H, D)
    k = plain.norm_plain(h_of[0].double() @ w["k"].T, w["k.norm"], 1e-5).view(T, G, D)
    if R:
        q, k = (plain.turn_halves(x, torch.arange(T), R, 700.0) for x in (q, k))
    p = plain.causal_weights(torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(H // G, 1)) * scale)
    best = p[:, 200:].max(-1)
    assert float((best.values > 0.25).double().mean()) > 0.3
    far = (200 + torch.arange(T - 200)[None] - best.indices > 150) & (best.values > 0.25)
    assert int(far.sum()) > 5                                                           # far keys among them


def test_the_whole_projections_norm_and_the_gate_per_head_matter():
    """The same tensors through a norm per head, or through no gate, give another result."""
    h = torch.randn(40, 48).to(torch.bfloat16).double()
    cfg = _attention_cfg(4, 2, 16, 16, 8, 0.7)
    g = torch.Generator().manual_seed(1)
    w = {"q": torch.randn(64, 48, generator=g).double() * 0.4, "k": torch.randn(32, 48, generator=g).double() * 0.4,
         "v": torch.randn(32, 48, generator=g).double() * 0.4, "g": torch.randn(4, 48, generator=g).double(),
         "o": torch.randn(48, 64, generator=g).double() * 0.4,
         "q.norm": 1 + 0.3 * torch.randn(64, generator=g).double(), "k.norm": 1 + 0.3 * torch.randn(32, generator=g).double()}
    ref = plain.grouped_attention(h, w, cfg, 1e-5, "")
    per_head = dict(w)
    t = 40
    q = (h @ w["q"].T).view(t, 4, 16)
    # a norm per head would divide every head by its own root mean square
    q = (plain.unit_rms(q, 1e-5) * w["q.norm"].view(4, 16)).reshape(t, 64)
    assert rel(q, plain.norm_plain(h @ w["q"].T, w["q.norm"], 1e-5)) > 0.05
    no_gate = dict(w)
    no_gate["g"] = torch.zeros(4, 48).double()       # sigmoid(0) = 1/2 for every head
    assert rel(2 * plain.grouped_attention(h, no_gate, cfg, 1e-5, ""), ref) > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_the_whole_projection_in_the_preparation_kernel(dtype):
    """The kernel alone: rows [q | k | v], one root mean square over all of q, one over all of k,
    gains over all heads' features, then the rotation of split halves; k and v land in the pages."""
    from crucible_b200.ops import sink_attention as kernels
    from crucible_b200.parts import CacheNeed, LayerBinding
    H, G, D, E, R, T = 5, 1, 24, 8, 10, 37
    steps = StepsWithValues(dtype, CacheNeed(kv_heads=G, head_dim=D, value_dim=E), 8, 1, 64, seed=1)
    ctx = steps.ctx([(0, T)], None)
    rows = (torch.randn(T, (H + G) * D + G * E) * 2).to(torch.bfloat16).float()
    qg = (1 + 0.3 * torch.randn(H * D)).float()
    kg = (1 + 0.3 * torch.randn(G * D)).float()
    freq = (50.0 ** (-2.0 * torch.arange(R // 2, dtype=torch.float64) / R)).float()
    proj = rows.to(dtype).to(DEV).contiguous()
    binding = LayerBinding(group=0, slot=0, write=True)
    kernels.norm_rotate_append(proj, qg.to(DEV), kg.to(DEV), 1e-5, freq.to(DEV), R, True, H, G, D, E, None, ctx,
                               steps.storage, binding, whole_norm=True)
    pos = torch.arange(T)
    q = plain.turn_halves(plain.norm_plain(rows[:, :H * D].double(), qg.double(), 1e-5).view(T, H, D), pos, R, 50.0)
    k = plain.turn_halves(plain.norm_plain(rows[:, H * D:(H + G) * D].double(), kg.double(), 1e-5).view(T, G, D), pos, R, 50.0)
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    assert rel(proj[:, :H * D], q.reshape(T, H * D)) < tol
    table = steps.tables[0].to(DEV).long()
    keys = steps.storage.keys(0)[table[pos.to(DEV) // 8], :, pos.to(DEV) % 8]       # [T, G, D]
    values = steps.storage.values(0)[table[pos.to(DEV) // 8], :, pos.to(DEV) % 8]
    assert rel(keys, k) < tol
    assert torch.equal(values.float().cpu().view(T, G * E), rows[:, (H + G) * D:])


# ---------------------------------------------------------------------------
# latent attention with a sink
# ---------------------------------------------------------------------------

def _latent_spec(H, D, R, E, C, Q, width, scale, sink=True):
    from crucible_b200.config.model_config import MixerSpec
    return MixerSpec(kind="latent_attention", width=width, n_heads=H, n_kv_heads=1, head_dim=D, softmax_scale=scale,
                     window=None, position=_position("rope_interleaved", R, 900.0),
                     extra=(("rot_dim", R), ("value_dim", E), ("kv_rank", C), ("norm_eps", 1e-5),
                            ("gate", "element"), ("q_rank", Q), ("sink", sink)))


def _latent_cfg(H, D, R, E, C, Q, scale):
    return {"heads": H, "dim": D, "rot_dim": R, "vdim": E, "kv_rank": C, "q_rank": Q, "scale": scale,
            "rot": {"dims": R, "base": 900.0} if R else None}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,E,C,Q,width,page", [
    (3, 16, 8, 24, 24, 16, 48, 8),        # a row of 32: tensor cores in bfloat16
    (2, 12, 6, 10, 21, 9, 44, 16),        # a row of 27: CUDA cores
    (4, 32, 32, 32, 96, 64, 128, 16),     # a row of 128
    (2, 16, 16, 16, 304, 32, 64, 16),     # a row of 320: the wide form of the plain kernel
    (2, 8, 0, 8, 16, 8, 40, 8)])          # no rotated part at all
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
def test_latent_attention_with_a_sink(dtype, H, D, R, E, C, Q, width, page, how):
    from crucible_b200.parts import MIXERS
    T, std = 200, 0.3
    scale = 2.5 / (std * std * (C * Q * D) ** 0.5)        # scores of spread 2.5 whatever the sizes
    part = MIXERS.build("latent_attention", _latent_spec(H, D, R, E, C, Q, width, scale))

    def edit(t):
        # a sink that takes most of the weight on the first head, one that is negligible on the last
        t["sink"] = torch.linspace(6.0, -6.0, H) if H > 1 else torch.tensor([3.0])
    w = _bind(part, dtype, 9, std=std, edit=edit)
    steps = StepsWithValues(dtype, part.cache_need(), page, 2, 256, seed=4)
    h_of = {0: torch.randn(T, width).to(torch.bfloat16).float(), 1: torch.randn(33, width).to(torch.bfloat16).float()}
    binding = _binding(part, group=0)
    got = _run_part(part, steps, _beside(_cuts(T, how), 1, 33, 5), h_of, width, binding)
    cfg = _latent_cfg(H, D, R, E, C, Q, scale)
    for slot, h in h_of.items():
        ref = plain.latent_attention(h.double(), w, cfg, 1e-5, "")
        assert rel(got[slot], ref) < TOL[dtype], (slot, how)
    # without the sink the result is another one, by far
    gone = dict(w)
    gone["sink"] = torch.full((H,), -60.0).double()
    ref = plain.latent_attention(h_of[0].double(), w, cfg, 1e-5, "")
    assert rel(plain.latent_attention(h_of[0].double(), gone, cfg, 1e-5, ""), ref) > 0.2


def test_the_sink_counts_once_and_is_not_scaled():
    """One key, score s: the weight is exp(s * scale) / (exp(s * scale) + exp(sink))."""
    import math
    scores = torch.tensor([[[2.0]]]).double()
    p = plain.causal_weights(scores * 0.5, sink=torch.tensor([1.5]).double())
    assert abs(float(p) - math.exp(1.0) / (math.exp(1.0) + math.exp(1.5))) < 1e-12


# ---------------------------------------------------------------------------
# retention
# ---------------------------------------------------------------------------

def _retention_spec(H, D, E, decay, R, width):
    from crucible_b200.config.model_config import MixerSpec
    return MixerSpec(kind="retention", width=width, n_heads=H, n_kv_heads=H, head_dim=D,
                     position=_position("rope_halves", R, 400.0),
                     extra=(("value_dim", E), ("norm_eps", 1e-5), ("decay", tuple(decay))))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,E,decay,R,width", [
    (4, 16, 24, [0.9, 0.99, 1.0, 0.5], 8, 48),
    (1, 40, 12, [0.97], 40, 44),                   # a key size that is no multiple of 16, the whole head turned
    (3, 10, 6, [0.8, 1.0, 0.0], 0, 40),            # no rotation; a head that forgets at once
    (2, 64, 64, [0.999, 0.9999], 16, 128),
    (2, 128, 32, [0.95, 0.99], 64, 64)])
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
def test_retention_carries_its_state(dtype, H, D, E, decay, R, width, how):
    from crucible_b200.parts import MIXERS
    T = 260
    part = MIXERS.build("retention", _retention_spec(H, D, E, decay, R, width))
    w = _bind(part, dtype, 2, std=0.3)
    steps = Steps(dtype, part.state_bytes(), None, 8, 3, 512)
    h_of = {0: torch.randn(T, width).to(torch.bfloat16).float(), 2: torch.randn(41, width).to(torch.bfloat16).float()}
    binding = _binding(part)
    got = _run_part(part, steps, _beside(_cuts(T, how), 2, 41, 3), h_of, width, binding)
    cfg = {"heads": H, "dim": D, "vdim": E, "decay": decay, "rot": {"dims": R, "base": 400.0} if R else None}
    for slot, h in h_of.items():
        assert rel(got[slot], plain.retention(h.double(), w, cfg, 1e-5, "")) < TOL[dtype], (slot, how)
    # a slot that is given back and used again starts from zero
    steps.free(0)
    again = _run_part(part, steps, [[(0, 41)]], {0: h_of[2]}, width, binding)
    assert rel(again[0], plain.retention(h_of[2].double(), w, cfg, 1e-5, "")) < TOL[dtype]


def test_retention_remembers_the_first_token_with_a_decay_of_one():
    """The plain rule: with decay 1 and orthogonal keys the state holds every token's value for
    ever; with a decay below 1 a token d steps back counts decay^d."""
    H, D, E, T = 1, 8, 4, 6
    k = torch.eye(D, dtype=torch.float64)[:T]
    v = torch.randn(T, E, dtype=torch.float64)
    for decay in (1.0, 0.5):
        state = torch.zeros(D, E, dtype=torch.float64)
        for i in range(T):
            state = decay * state + k[i][:, None] * v[i][None, :]
        out = state.T @ k[0]
        assert torch.allclose(out, v[0] * decay ** (T - 1))


# ---------------------------------------------------------------------------
# the dense feed-forward: the square of relu on the first product's way out
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,rows", [(40, 72, 19), (128, 256, 150), (44, 52, 1), (64, 96, 8), (256, 704, 300)])
def test_dense_feed_forward_with_the_square_of_relu(dtype, width, ff, rows, monkeypatch):
    from crucible_b200 import ops
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    part = FEED_FORWARDS.build("dense_act", FeedForwardSpec(kind="dense_act", width=width, intermediate=ff,
                                                            extra=(("activation", "relu2"),)))
    w = _bind(part, dtype, 3, std=0.2)
    h = torch.randn(rows, width).to(torch.bfloat16).float()
    ref = plain.dense_feed_forward(h.double(), w, "")
    results = []
    for fused in (True, False):
        monkeypatch.setattr(ops, "FUSE_ACTIVATION", fused)
        res = torch.zeros(rows, width, device=DEV)
        part.forward(Steps(dtype).ctx([(0, rows)], None), h.to(dtype).to(DEV), res)
        assert rel(res, ref) < TOL[dtype], fused
        results.append(res.clone())
    if dtype == torch.bfloat16:
        # the two forms differ by one rounding of the first product, no more
        assert rel(results[0], results[1]) < 1e-2
