"""Each mechanism of the Nipapel design alone: its part, driven over hand-made steps, against
the one-mechanism functions of `plain_nipapel.py`.  Inputs are made so that a fault shows: a
few keys' scores stand far out (far back, at page borders, just inside and just outside the
window, the last kept token and the first that is not), gates and caps are driven to both
sides."""
from types import SimpleNamespace

import pytest
import torch

import plain_nipapel as plain
from test_futepel_kernels_gpu import DEV, TOL, Steps, _bind, _check_mixer, _i32, rel

pytestmark = pytest.mark.gpu


class StepsWithValues(Steps):
    """`Steps` whose pages may hold values of a size of their own."""

    def __init__(self, dtype, cache_need, page, n_slots, max_tokens, seed=0):
        super().__init__(dtype, 0, cache_need, page, n_slots, max_tokens, seed)
        from crucible_b200.engine.context import CacheStorage
        self.storage = CacheStorage(1, self.storage.n_pages, page, cache_need.kv_heads, cache_need.head_dim, dtype,
                                    DEV, value_dim=cache_need.value_dim, values_are_keys=cache_need.values_are_keys)


# ---------------------------------------------------------------------------
# norms whose weight is kept around zero; the embedding that goes through one
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 256, 1100])
def test_norm_with_a_weight_around_zero(dtype, width):
    from crucible_b200.config.model_config import NormSpec
    from crucible_b200.parts import NORMS
    norm = NORMS.build("rmsnorm_offset", NormSpec(kind="rmsnorm_offset", width=width, eps=1e-5))
    w = (torch.randn(width) * 0.3).to(torch.bfloat16).float()
    norm.bind({"gain": w.to(DEV)}, dtype, torch.device(DEV))
    x = torch.randn(9, width) * 3.0
    out = norm.forward(Steps(dtype).ctx([(0, 9)], None), x.to(DEV))
    assert out.dtype == dtype
    assert rel(out, plain.norm_around_zero(x.double(), w.double(), 1e-5)) < (2e-6 if dtype == torch.float32 else 6e-3)
    # the offset is what makes the difference
    assert rel(plain.norm_plain(x.double(), w.double(), 1e-5), plain.norm_around_zero(x.double(), w.double(), 1e-5)) > 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_rows_pass_the_norm(dtype):
    from crucible_b200.config.model_config import EndSpec
    from crucible_b200.parts import EMBEDDINGS
    emb = EMBEDDINGS.build("token_normed_streams", EndSpec("token_normed_streams", (("eps", 1e-5), ("streams", None),
                                                                                  ("gain_offset", 1.0))), 50, 72)
    table = (torch.randn(50, 72) * 0.2).to(torch.bfloat16).float()
    w = (torch.randn(72) * 0.2).to(torch.bfloat16).float()
    emb.bind({"table": table.to(dtype).to(DEV), "norm_gain": w.to(DEV)}, dtype, torch.device(DEV))
    ids = [3, 49, 0, 3, 17]
    x = emb.forward(Steps(dtype).ctx([(0, 5)], None), _i32(ids))
    assert x.dtype == torch.float32 and tuple(x.shape) == (5, 72)
    assert rel(x, plain.norm_around_zero(table.double()[ids], w.double(), 1e-5)) < 2e-6


# ---------------------------------------------------------------------------
# feed-forwards: the capped pair, alone, dense, and in experts behind a router with a bias
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capped_pair(dtype):
    from crucible_b200 import ops
    g = torch.Generator().manual_seed(1)
    both = (torch.randn(13, 2 * 37, generator=g) * 3.0).to(dtype)          # well beyond a limit of 1.5 on both sides
    out = torch.empty(13, 37, device=DEV, dtype=dtype)
    ops.glu(both.to(DEV), out, 1.5, 1.702, 1.0)
    b = both.double()
    gate, up = torch.clamp(b[:, :37], max=1.5), torch.clamp(b[:, 37:], -1.5, 1.5)
    ref = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert rel(out, ref) < (2e-6 if dtype == torch.float32 else 6e-3)
    assert float((b[:, :37] > 1.5).float().mean()) > 0.1 and float((b[:, :37] < -1.5).float().mean()) > 0.1
    # the gate is not capped from below: a gate capped on both sides would differ
    both_sides = torch.clamp(b[:, :37], -1.5, 1.5)
    assert rel(both_sides * torch.sigmoid(1.702 * both_sides) * (up + 1.0), ref) > 1e-3
    ops.glu(both.to(DEV), out)                                               # without a limit: silu(g) * u
    assert rel(out, b[:, :37] * torch.sigmoid(b[:, :37]) * b[:, 37:]) < (2e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff,rows,limit", [(40, 72, 19, 0.5), (128, 256, 150, 2.0), (44, 52, 1, 1.0)])
def test_dense_feed_forward(dtype, width, ff, rows, limit):
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    part = FEED_FORWARDS.build("glu_capped", FeedForwardSpec(kind="glu_capped", width=width, intermediate=ff,
                                                             extra=(("limit", limit),)))
    w = _bind(part, dtype, seed=6)
    h = torch.randn(rows, width, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).float()
    res = torch.zeros(rows, width, device=DEV)
    part.forward(Steps(dtype).ctx([(0, rows)], None), h.to(dtype).to(DEV), res)
    assert rel(res, plain.capped_glu(h.double(), w["gate"], w["up"], w["down"], limit)) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,width,rows,limit", [(6, 2, 40, 48, 77, 1.5), (4, 1, 20, 24, 5, 0.5),
                                                             (8, 8, 64, 128, 200, 2.0), (40, 5, 12, 36, 300, 1.0),
                                                             (1, 1, 16, 32, 3, 1.0)])
def test_experts_behind_a_router_with_a_bias(dtype, experts, top, ff, width, rows, limit):
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    spec = FeedForwardSpec(kind="moe", width=width, intermediate=ff,
                           extra=(("experts", experts), ("top", top), ("shared_intermediate", None),
                                  ("router_bias", True), ("pair", (limit, 1.702, 1.0))))
    part = FEED_FORWARDS.build("moe", spec)

    def edit(t):
        # a bias as large as the logits: leaving it out sends most tokens elsewhere.  In bfloat16
        # the logits lie far apart, so that the rounding of the rows decides no choice
        t["router.b"] = torch.linspace(-2.0, 2.0, experts).flip(0).contiguous()
        if dtype == torch.bfloat16:
            t["router"] *= 0.02
    w = _bind(part, dtype, seed=4, edit=edit)
    cfg = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    h = torch.randn(rows, width, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).float()
    ref = plain.experts(h.double(), w, cfg)
    res = torch.zeros(rows, width, device=DEV)
    part.forward(Steps(dtype).ctx([(0, rows)], None), h.to(dtype).to(DEV), res)
    assert rel(res, ref) < TOL[dtype]
    if experts > top:
        unbiased = dict(w)
        unbiased["router.b"] = torch.zeros(experts, dtype=torch.float64)
        assert rel(plain.experts(h.double(), unbiased, cfg), ref) > 0.05
    # a token's result does not depend on what else is in the step
    few = [0, rows // 2, rows - 1]
    alone = torch.zeros(len(few), width, device=DEV)
    part.forward(Steps(dtype).ctx([(0, len(few))], None), h[few].to(dtype).to(DEV), alone)
    if dtype == torch.float32:
        assert torch.equal(alone, res[few])
    else:
        assert rel(alone, ref[few]) < TOL[dtype]


# ---------------------------------------------------------------------------
# attention: q and k norms, split halves, the window's edges, the kept first tokens, pages
# ---------------------------------------------------------------------------

def _attention_spec(H, G, D, E, R, window, keep, width, scale):
    from crucible_b200.config.model_config import MixerSpec, PositionSpec
    position = PositionSpec(kind="rope_halves", rotary_dim=R, theta=700.0, max_positions=0) if R else None
    return MixerSpec(kind="sink_attention", width=width, n_heads=H, n_kv_heads=G, head_dim=D, softmax_scale=scale,
                     window=window, position=position,
                     extra=(("value_dim", E), ("keep_first", keep), ("sink", False), ("gate", False),
                            ("value_norm_eps", None), ("qk_norm_eps", 1e-5)))


def _run_part(part, steps, schedule, h_of, width, binding):
    out = {}
    for entries in schedule:
        ctx = steps.ctx(entries, binding)
        h = torch.cat([h_of[slot][steps.fed[slot] - n:steps.fed[slot]] for slot, n in entries], 0).to(steps.dtype).to(DEV)
        res = torch.zeros(h.shape[0], width, device=DEV)
        part.forward(ctx, h.contiguous(), res, binding)
        at = 0
        for slot, n in entries:
            out.setdefault(slot, []).append(res[at:at + n].clone())
            at += n
    torch.cuda.synchronize()
    return {slot: torch.cat(chunks, 0) for slot, chunks in out.items()}


def _cuts(T, how):
    if how == "prompt":
        return [T]
    if how == "decode":
        return [5] + [1] * (T - 5)
    sizes, out = [2, 7, 2, 1, 37, 2, 64, 3], []
    while sum(out) < T:
        out.append(min(sizes[len(out) % len(sizes)], T - sum(out)))
    return out


@pytest.mark.parametrize("dtype,D,E,tensor_cores", [(torch.float32, 16, 24, False), (torch.bfloat16, 16, 24, False),
                                                    (torch.bfloat16, 32, 32, False), (torch.bfloat16, 32, 32, True),
                                                    # heads of 64 and 128: portions of 32 tokens and more on the tcgen05 tiles
                                                    (torch.bfloat16, 64, 64, True), (torch.bfloat16, 128, 128, True)])
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
@pytest.mark.parametrize("window,keep,T", [(10, 3, 90), (70, 5, 300), (33, 0, 120), (40, 130, 420)])
def test_attention_sees_exactly_its_keys(dtype, D, E, tensor_cores, how, window, keep, T, monkeypatch):
    """Feature 0 of the input is 1 for every token and feature 1 is large for a few marked
    tokens.  A channel that is not turned reads feature 0 in every query head and feature 1
    in every key head, with weights so large that it is all the head's norm leaves: a row's
    softmax is then held by the marked keys it may see."""
    from crucible_b200.ops import sink_attention as k
    from crucible_b200.parts import MIXERS, LayerBinding
    monkeypatch.setattr(k, "TENSOR_CORES", tensor_cores)
    H, G, R, width, page, scale = 4, 2, 8, 48, 8, 6.0 / D       # a marked key's score is D * scale
    marked = sorted({max(keep - 1, 0), keep, 7, 8, 40} | ({63, 64, 130} if T > 200 else set()))

    def edit(t):
        for name, heads, feature in (("q", H, 0), ("k", G, 1)):
            m = t[name].view(heads, D, width)
            m[:, :, feature] = 0.0
            m[:, D - 1, :] = 0.0
            m[:, D - 1, feature] = 40.0

    def h_edit(h):
        h[:, 0] = 1.0
        h[:, 1] = 0.0
        for j in marked:
            h[j, 1] = 1.0

    spec = _attention_spec(H, G, D, E, R, window, keep, width, scale)
    part = MIXERS.build(spec.kind, spec)
    w = _bind(part, dtype, seed=5, std=0.1, edit=edit)
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(9))
    h_edit(h)
    h = h.to(torch.bfloat16).float()
    cfg = {"heads": H, "kv_heads": G, "dim": D, "vdim": E, "scale": scale, "rot": {"base": 700.0, "dims": R},
           "mask": {"size": window, "keep_first": keep}}
    ref = plain.attention(h.double(), w, cfg, 1e-5, torch.arange(T))
    steps = StepsWithValues(dtype, part.cache_need(), page, 3, T + page)
    binding = LayerBinding(group=0, slot=0, write=True)
    got = _run_part(part, steps, [[(2, n)] for n in _cuts(T, how)], {2: h}, width, binding)[2]
    for j in marked:
        for i in (j, j + window - 1, j + window, T - 1):
            if i < T:
                assert rel(got[i], ref[i]) < TOL[dtype], (how, "key", j, "row", i)
    assert rel(got, ref) < TOL[dtype]
    # a window that is one token off would show: the plain result itself changes where a marked key leaves
    j = marked[-1]
    if j + window < T:
        assert rel(ref[j + window], ref[j + window - 1]) > 0.05


def test_attention_norm_and_pairing_matter():
    """The plain functions tell the norms' weights and the two pairings apart."""
    g = torch.Generator().manual_seed(3)
    w = {"q": torch.randn(32, 24, generator=g), "k": torch.randn(16, 24, generator=g), "v": torch.randn(16, 24, generator=g),
         "o": torch.randn(24, 32, generator=g), "q.norm": torch.rand(16, generator=g) + 0.5, "k.norm": torch.rand(16, generator=g) + 0.5}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(30, 24, generator=g).double()
    cfg = {"heads": 2, "kv_heads": 1, "dim": 16, "scale": 0.4, "rot": {"base": 50.0, "dims": 8}, "mask": {"size": 12, "keep_first": 2}}
    ref = plain.attention(h, w, cfg, 1e-5, torch.arange(30))
    flat = dict(w); flat["q.norm"] = torch.ones(16, dtype=torch.float64)
    assert rel(plain.attention(h, flat, cfg, 1e-5, torch.arange(30)), ref) > 0.02
    x = torch.randn(5, 2, 16, generator=g).double()
    assert rel(plain.turn_neighbours(x, torch.arange(5), 8, 50.0), plain.turn_split_halves(x, torch.arange(5), 8, 50.0)) > 0.1


# ---------------------------------------------------------------------------
# latent attention: a latent for the queries, neighbouring pairs, a window, a gate per feature,
# and a layer that reads another layer's rows
# ---------------------------------------------------------------------------

def _latent_spec(H, D, R, E, C, Q, width, window, reads_other=False, cache_window=None):
    from crucible_b200.config.model_config import MixerSpec, PositionSpec
    position = PositionSpec(kind="rope_interleaved", rotary_dim=R, theta=1000.0, max_positions=0)
    extra = (("rot_dim", R), ("value_dim", E), ("kv_rank", C), ("norm_eps", 1e-5), ("gate", "element"), ("q_rank", Q),
             ("reads_other", reads_other))
    if cache_window is not None:
        extra += (("cache_window", cache_window),)
    return MixerSpec(kind="latent_attention", width=width, n_heads=H, n_kv_heads=1, head_dim=D, softmax_scale=0.25,
                     window=window, position=position, extra=extra)


def _latent_cfg(H, D, R, E, C, Q, window):
    return {"heads": H, "dim": D, "rot_dim": R, "vdim": E, "kv_rank": C, "q_rank": Q, "scale": 0.25,
            "rot": {"base": 1000.0, "dims": R}, "mask": {"size": window}}


def _mark_latent(H, D, R, C, Q, width):
    """Latent channel 0 reads feature 1 alone; every head's key channel 0 reads latent channel 0;
    the queries' latent channel 0 reads feature 0 alone and every head's query channel 0 reads it."""
    def edit(t):
        if "dkv" in t:
            t["dkv"][0] = 0.0
            t["dkv"][0, 1] = 1.0
            t["dkv"][1:, 1] = 0.0
        t["uk"].view(H, D, C)[:, 0, :] = 0.0
        t["uk"].view(H, D, C)[:, 0, 0] = 2.0
        t["dq"][0] = 0.0
        t["dq"][0, 0] = 1.0
        t["dq"][1:, 0] = 0.0
        t["uq"].view(H, D + R, Q)[:, 0, :] = 0.0
        t["uq"].view(H, D + R, Q)[:, 0, 0] = 3.0
    return edit


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,E,C,Q,width,page,window",
                         [(2, 24, 8, 16, 40, 24, 48, 8, 21),
                          (4, 32, 32, 32, 96, 64, 64, 16, 70),          # rows of 128: tensor cores in bfloat16
                          (2, 16, 16, 16, 48, 8, 32, 8, 300),           # rows of 64; a window wider than the requests
                          (4, 64, 64, 64, 192, 96, 128, 16, 130),       # rows of 256: decoded tokens' keys in chunks of 64
                          (3, 10, 6, 14, 21, 9, 40, 4, 5)])
def test_latent_attention_finds_marked_keys(dtype, H, D, R, E, C, Q, width, page, window):
    marked = [2, page - 1, page, 3 * page - 1, 3 * page, 150, 263]

    def h_edit(h):
        h[:, 0] = 1.0
        h[:, 1] = 0.0
        for j in marked:
            if j < h.shape[0]:
                h[j, 1] = 4.0

    cfg = _latent_cfg(H, D, R, E, C, Q, window)

    def ref(h, w):
        pos = torch.arange(h.shape[0])
        return plain.latent_attention(h, w, cfg, 1e-5, pos, plain.latent_rows(h, w, cfg, 1e-5, pos))
    _check_mixer(_latent_spec(H, D, R, E, C, Q, width, window), ref, dtype, {0: 270, 1: 3 * page + 1, 3: 2},
                 page=page, edit=_mark_latent(H, D, R, C, Q, width), h_edit=h_edit, std=0.1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
def test_a_layer_reads_another_layers_rows_with_a_window_of_its_own(dtype, how):
    """The owner writes its rows; the reader, which has no latent projection, sees them through
    the same pages with other heads, another value size, and a wider window."""
    from crucible_b200.parts import MIXERS, LayerBinding
    R, C, width, page, T = 8, 40, 48, 8, 150
    own = dict(H=2, D=24, E=16, Q=24, window=21)
    other = dict(H=3, D=12, E=20, Q=16, window=64)
    marked = [2, 7, 8, 40, 85, 86]
    specs = {"own": _latent_spec(own["H"], own["D"], R, own["E"], C, own["Q"], width, own["window"], cache_window=64),
             "other": _latent_spec(other["H"], other["D"], R, other["E"], C, other["Q"], width, other["window"],
                                   reads_other=True, cache_window=64)}
    parts = {name: MIXERS.build(spec.kind, spec) for name, spec in specs.items()}
    assert parts["own"].cache_need() == parts["other"].cache_need() and parts["own"].cache_need().window == 64
    assert not any(d.name.startswith("dkv") for d in parts["other"].tensors())
    w = {name: _bind(parts[name], dtype, seed=5 + i, std=0.1,
                     edit=_mark_latent(d["H"], d["D"], R, C, d["Q"], width))
         for i, (name, d) in enumerate((("own", own), ("other", other)))}
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(9))
    h[:, 0] = 1.0
    h[:, 1] = 0.0
    h[marked, 1] = 4.0
    h = h.to(torch.bfloat16).float()
    h2 = (h + 0.1 * torch.randn(T, width, generator=torch.Generator().manual_seed(10))).to(torch.bfloat16).float()
    pos = torch.arange(T)
    cfgs = {name: _latent_cfg(d["H"], d["D"], R, d["E"], C, d["Q"], d["window"]) for name, d in (("own", own), ("other", other))}
    rows = plain.latent_rows(h.double(), w["own"], cfgs["own"], 1e-5, pos)
    ref_own = plain.latent_attention(h.double(), w["own"], cfgs["own"], 1e-5, pos, rows)
    ref_other = plain.latent_attention(h2.double(), w["other"], cfgs["other"], 1e-5, pos, rows)
    steps = Steps(dtype, cache_need=parts["own"].cache_need(), page=page, n_slots=3, max_tokens=T + page)
    write, read = LayerBinding(group=0, slot=0, write=True), LayerBinding(group=0, slot=0, write=False)
    got_own, got_other, at = [], [], 0
    for n in _cuts(T, how):
        ctx = steps.ctx([(1, n)], write)
        for part, rows_in, binding, out in ((parts["own"], h, write, got_own), (parts["other"], h2, read, got_other)):
            res = torch.zeros(n, width, device=DEV)
            part.forward(ctx, rows_in[at:at + n].to(dtype).to(DEV).contiguous(), res, binding)
            out.append(res)
        at += n
    assert rel(torch.cat(got_own), ref_own) < TOL[dtype]
    got_other = torch.cat(got_other)
    for j in marked:
        for i in (j + 20, j + 21, j + 63, j + 64):           # the owner's edge is not the reader's
            if i < T:
                assert rel(got_other[i], ref_other[i]) < TOL[dtype], (how, "key", j, "row", i)
    assert rel(got_other, ref_other) < TOL[dtype]
    narrow = plain.latent_attention(h2.double(), w["other"], dict(cfgs["other"], mask={"size": 21}), 1e-5, pos, rows)
    assert rel(narrow[85 + 30], ref_other[85 + 30]) > 0.05


def test_latent_gate_and_query_norm_matter():
    H, D, R, E, C, Q, width = 2, 12, 4, 8, 20, 10, 32
    cfg = _latent_cfg(H, D, R, E, C, Q, 9)
    g = torch.Generator().manual_seed(0)
    w = {"dq": torch.randn(Q, width, generator=g), "dq.norm": torch.rand(Q, generator=g) + 0.5,
         "uq": torch.randn(H * (D + R), Q, generator=g) * 0.3, "dkv": torch.randn(C + R, width, generator=g),
         "dkv.norm": torch.ones(C), "uk": torch.randn(H * D, C, generator=g) * 0.3, "uv": torch.randn(H * E, C, generator=g),
         "g": torch.randn(H * E, width, generator=g), "o": torch.randn(width, H * E, generator=g)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(25, width, generator=g).double()
    pos = torch.arange(25)
    rows = plain.latent_rows(h, w, cfg, 1e-5, pos)
    ref = plain.latent_attention(h, w, cfg, 1e-5, pos, rows)
    open_gate = dict(w); open_gate["g"] = torch.zeros_like(w["g"])
    assert rel(plain.latent_attention(h, open_gate, cfg, 1e-5, pos, rows), ref) > 0.1
    flat = dict(w); flat["dq.norm"] = torch.ones(Q, dtype=torch.float64)
    assert rel(plain.latent_attention(h, flat, cfg, 1e-5, pos, rows), ref) > 0.02


# ---------------------------------------------------------------------------
# the experts of a prompt step as grouped products on the tensor cores
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("experts,top,ff,width,rows", [(8, 2, 64, 128, 700), (5, 1, 40, 64, 300), (3, 3, 72, 48, 129)])
def test_grouped_products_follow_the_plan_on_the_device(experts, top, ff, width, rows, monkeypatch):
    """Many rows in bfloat16: the rows lie expert by expert and two grouped products run over
    tiles of 128 rows whose owners the device alone knows.  Experts with no rows, with one row
    and with more than a tile's worth all occur; the result is the plain one, and nothing of the
    step comes to the host (no per-expert product is launched)."""
    from crucible_b200 import ops
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.ops import moe as kernels
    from crucible_b200.parts import FEED_FORWARDS
    dtype = torch.bfloat16
    spec = FeedForwardSpec(kind="moe", width=width, intermediate=ff,
                           extra=(("experts", experts), ("top", top), ("shared_intermediate", None),
                                  ("router_bias", True), ("pair", (1.0, 1.702, 1.0))))
    part = FEED_FORWARDS.build("moe", spec)

    def edit(t):
        # expert 0 gets no token at all (unless all are used), the last one a single token
        bias = torch.linspace(1.0, 3.0, experts)
        bias[0] = -50.0 if top < experts else 0.0
        t["router.b"] = bias
        t["router"] *= 0.02
    w = _bind(part, dtype, seed=4, edit=edit)
    cfg = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": 1.0}}
    h = torch.randn(rows, width, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).float()
    ref = plain.experts(h.double(), w, cfg)
    calls = {"grouped": 0, "linear": 0}
    grouped, linear = kernels.grouped_linear, ops.linear
    monkeypatch.setattr(kernels, "grouped_linear", lambda *a, **k: calls.__setitem__("grouped", calls["grouped"] + 1) or grouped(*a, **k))
    monkeypatch.setattr(ops, "linear", lambda *a, **k: calls.__setitem__("linear", calls["linear"] + 1) or linear(*a, **k))
    res = torch.zeros(rows, width, device=DEV)
    part.forward(Steps(dtype).ctx([(0, rows)], None), h.to(dtype).to(DEV), res)
    assert rel(res, ref) < TOL[dtype]
    assert calls == {"grouped": 2, "linear": 1}          # the router's logits and the two grouped products
    assert part.count.tolist() == [0] * experts          # left ready for the next step


@pytest.mark.parametrize("rows,heads,a_head,k,n,out_head", [(200, 4, 96, 64, 96, 96), (2048, 8, 192, 128, 192, 256),
                                                            (333, 3, 256, 192, 40, 40), (129, 5, 72, 72, 136, 136),
                                                            (64, 1, 64, 64, 64, 64)])
@pytest.mark.parametrize("result", [torch.bfloat16, torch.float32])
def test_heads_products_of_many_rows_are_one_launch(rows, heads, a_head, k, n, out_head, result):
    """Every head's own matrix over its own columns of the rows, the head as the grid's third
    axis: against the sums in float64, and counted.  Sizes whose K is no multiple of 64 (the
    block's last columns belong to the next head and must meet zeros) and whose N is no
    multiple of the tile (the tile's last rows of W belong to the next head and are not stored);
    the columns between the heads' results stay as they were."""
    from crucible_b200 import ops
    from crucible_b200.ops import latent, tensor_core
    g = torch.Generator().manual_seed(rows + heads)
    a = torch.randn(rows, heads * a_head, generator=g).to(torch.bfloat16)
    w = (torch.randn(heads, n, k, generator=g) * 0.2).to(torch.bfloat16)
    ref = torch.einsum("thk,hnk->thn", a.double().view(rows, heads, a_head)[..., :k], w.double())
    wd = w.to(DEV).contiguous()
    ops.declare_weights(wd)
    if result == torch.float32:
        out = torch.full((rows, heads * out_head), 7.0, device=DEV, dtype=result)
        assert tensor_core.heads_linear(a.to(DEV), a_head, wd, out, out_head)
    else:
        out = torch.full((rows, heads * out_head), 7.0, device=DEV, dtype=result)
        before = ops.LAUNCHES[0]
        latent.heads_linear(a.to(DEV), a_head, wd, out, out_head)
        assert ops.LAUNCHES[0] - before == 1
    got = out.double().cpu().view(rows, heads, out_head)
    assert rel(got[..., :n], ref) < 1e-2
    if out_head > n:
        assert torch.all(got[..., n:] == 7.0)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("window,keep", [(70, 5), (40, 130), (200, 0)])
def test_unequal_portions_of_several_requests_in_one_step(D, window, keep, monkeypatch):
    """Steps of portions alone, of unequal sizes, from three requests whose pages are scattered:
    bfloat16 heads of 64 and 128 take the tensor-core tiles with the kept first tokens' tile
    ahead of the window's; every request agrees with the plain attention over itself alone,
    and a request that comes back in a later step goes on from its own keys."""
    from crucible_b200.parts import MIXERS, LayerBinding
    dtype, H, G, R, width, page = torch.bfloat16, 6, 3, D // 2, 64, 16
    spec = _attention_spec(H, G, D, D, R, window, keep, width, D ** -0.5)
    part = MIXERS.build(spec.kind, spec)
    w = _bind(part, dtype, seed=6, std=0.2)
    lengths = {0: 400, 1: 150, 2: 333}
    g = torch.Generator().manual_seed(12)
    h_of = {slot: torch.randn(n, width, generator=g).to(torch.bfloat16).float() for slot, n in lengths.items()}
    cfg = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"base": 700.0, "dims": R},
           "mask": {"size": window, "keep_first": keep}}
    steps = StepsWithValues(dtype, part.cache_need(), page, 3, 400 + page)
    binding = LayerBinding(group=0, slot=0, write=True)
    schedule = [[(0, 200), (1, 40), (2, 33)], [(2, 300), (0, 100)], [(1, 110), (0, 100)]]
    from crucible_b200.ops import tensor_core
    taken, inner = [], tensor_core._attention_tcgen05

    def counted(*args, **kwargs):
        taken.append(inner(*args, **kwargs))
        return taken[-1]
    monkeypatch.setattr(tensor_core, "_attention_tcgen05", counted)
    got = _run_part(part, steps, schedule, h_of, width, binding)
    assert taken == [True, True, True]           # every step ran on the tcgen05 tiles
    for slot, n in lengths.items():
        ref = plain.attention(h_of[slot].double(), w, cfg, 1e-5, torch.arange(n))
        assert rel(got[slot], ref) < TOL[dtype], slot
