"""Feed-forwards of this family: a dense one with a chosen activation, and a mixture of
experts.

`dense_act`: x += act(h Wup^T) Wdown^T; the activation is an option of the spec (relu2:
the square of ReLU; gelu_tanh; silu; tanh).

`glu_capped`: x += pair(h Wg^T, h Wu^T) Wdown^T with the capped gated pair: g' = min(g, limit),
u' = clamp(u, -limit, limit), pair = g' * sigmoid(alpha * g') * (u' + offset); `limit`, `alpha`
(default 1.702) and `offset` (default 1) are options of the spec.

`moe`: `experts` gated feed-forwards Wd_e (silu(Wg_e h) * (Wu_e h)) without biases, of
which a token uses the `top` with the largest router logits z = h Wr^T (float32; the lower
index on ties), weighted by the softmax over those `top` logits alone; an optional shared
expert of the same form runs for every token and is added.  Options: `router_bias` (the
logits are h Wr^T + b, tensor `router.b`), `pair` = (limit, alpha, offset): the experts use
the capped gated pair instead of silu(g) * u.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import FeedForwardSpec
from ..ops import moe as kernels
from .base import FEED_FORWARDS, FeedForward, TensorDecl
from .swiglu import SwiGLU


class ActivatedFeedForward(FeedForward):
    fuses_norm = True          # h goes into one product: few rows are normalised on their way in
    takes_prenormed = False

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.kind = str(spec.option("activation", "relu2"))
        if self.kind not in ops.ACTIVATIONS:
            raise ValueError(f"dense_act: unknown activation {self.kind!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.up = self.down = None

    def tensors(self):
        d, f = self.spec.width, self.spec.intermediate
        return [TensorDecl("up", (f, d)), TensorDecl("down", (d, f))]

    def bind(self, tensors, dtype, device):
        self.up, self.down = tensors["up"], tensors["down"]
        ops.declare_weights(self.up, self.down)
        self.dtype = dtype

    def forward(self, ctx, h, residual):
        z = ctx.scratch("ffn.z", (h.shape[0], self.spec.intermediate), self.dtype)
        ops.linear_act(h, self.up, z, self.kind)
        ops.linear(z, self.down, residual, accumulate=True, closes=ctx)


class CappedGLU(FeedForward):
    fuses_norm = True
    takes_prenormed = False

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.limit = float(spec.option("limit", 0.0))
        self.alpha = float(spec.option("alpha", 1.702))
        self.offset = float(spec.option("offset", 1.0))
        if not self.limit > 0:
            raise ValueError("glu_capped: the limit must be positive")
        self.gate_up = self.down = None

    def tensors(self):
        d, f = self.spec.width, self.spec.intermediate
        return [TensorDecl("gate", (f, d)), TensorDecl("up", (f, d)), TensorDecl("down", (d, f))]

    def bind(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down = tensors["down"]
        ops.declare_weights(self.gate_up, self.down)
        self.dtype = dtype

    def forward(self, ctx, h, residual):
        t, f = h.shape[0], self.spec.intermediate
        act = ctx.scratch("ffn.act", (t, f), self.dtype)
        ops.linear_swiglu(h, self.gate_up, act, ctx, pair=(self.limit, self.alpha, self.offset))
        ops.linear(act, self.down, residual, accumulate=True, closes=ctx)


class MixtureOfExperts(FeedForward):
    # Nothing of a step's routing comes to the host: the launches depend on the step's shape
    # alone, so prompt steps are captured as graphs like decode steps.
    SMALL_MAX_PAIRS = 256        # up to this many pairs the experts' weight rows are read by a warp each
    SORTED_MIN_PAIRS = 256       # from this many (token, expert) pairs on, a prompt step's experts
                                 # run as two grouped products over their rows side by side

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.n = int(spec.option("experts", 0))
        self.top = int(spec.option("top", 0))
        self.ff = int(spec.intermediate)
        shared = spec.option("shared_intermediate")
        self.has_bias = bool(spec.option("router_bias", False))
        pair = spec.option("pair")
        self.pair = tuple(float(v) for v in pair) if pair is not None else None
        if self.pair is not None and (len(self.pair) != 3 or not self.pair[0] > 0):
            raise ValueError("moe: pair is (limit > 0, alpha, offset)")
        if self.n <= 0 or not 0 < self.top <= self.n or self.ff <= 0:
            raise ValueError("moe: experts, top (at most experts) and the experts' ff must be positive")
        if self.n > 256 or self.top > 32:
            raise ValueError("moe: up to 256 experts, of which a token uses up to 32")
        self.shared = (SwiGLU(FeedForwardSpec(kind="swiglu", width=spec.width, intermediate=int(shared)))
                       if shared else None)

    def tensors(self):
        d, f = self.spec.width, self.ff
        out = [TensorDecl("router", (self.n, d))]
        if self.has_bias:
            out.append(TensorDecl("router.b", (self.n,), role="vector", init=("normal", 0.0, 0.5)))
        for e in range(self.n):
            out += [TensorDecl(f"e{e}.gate", (f, d)), TensorDecl(f"e{e}.up", (f, d)),
                    TensorDecl(f"e{e}.down", (d, f))]
        if self.shared is not None:
            out += [TensorDecl(f"shared.{t.name}", t.shape, t.role) for t in self.shared.tensors()]
        return out

    def bind(self, tensors, dtype, device):
        self.dtype = dtype
        self.router = tensors["router"]
        self.router_bias = tensors.get("router.b") if self.has_bias else None
        self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], 0)
                                    for e in range(self.n)], 0).contiguous()          # [E, 2F, d]
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(self.n)], 0).contiguous()   # [E, d, F]
        ops.declare_weights(self.router, self.gate_up, self.down)
        self.count = torch.zeros(self.n, dtype=torch.int32, device=device)     # zero between steps
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")},
                             dtype, device)

    def forward(self, ctx, h, residual):
        t, d, top, n, f = h.shape[0], self.spec.width, self.top, self.n, self.ff
        logits = ctx.scratch("moe.logits", (t, n), torch.float32)
        ops.linear(h, self.router, logits)
        # many rows of a prompt: the experts' rows side by side and two grouped products on the
        # tensor cores, by the plan on the device (tiles of 128 rows)
        grouped = (self.dtype == torch.bfloat16 and t * top >= self.SORTED_MIN_PAIRS
                   and ctx.host.max_new_tokens > 1 and d % 8 == 0 and f % 8 == 0)
        tile_rows = kernels.GROUPED_TILE_ROWS if grouped else 0
        tiles = kernels.max_tiles(t, top, n, tile_rows)
        idx = ctx.scratch("moe.idx", (t * top,), torch.int32)
        place = ctx.scratch("moe.place", (t * top,), torch.int32)
        order = ctx.scratch("moe.order", (t * top,), torch.int32)
        weight = ctx.scratch("moe.weight", (t * top,), torch.float32)
        plan = ctx.scratch("moe.plan", (kernels.plan_ints(n, tiles),), torch.int32)
        kernels.route(logits, top, idx, weight, place, self.count, plan, tiles, order, bias=self.router_bias,
                      rows=tile_rows)
        act = ctx.scratch("moe.act", (t * top, f), self.dtype)
        pair_out = ctx.scratch("moe.pair_out", (t * top, d), torch.float32)
        if grouped:
            rows = ctx.scratch("moe.rows", (t * top, d), self.dtype)
            kernels.gather(h, order, top, rows)
            down = ctx.scratch("moe.down", (t * top, d), torch.float32)
            if not (kernels.grouped_linear(rows, self.gate_up, act, plan, n, tiles, True, pair=self.pair)
                    and kernels.grouped_linear(act, self.down, down, plan, n, tiles, False)):
                raise RuntimeError("moe: the grouped product refused sizes its rule allows")
            kernels.scatter(down, order, weight, pair_out)
        elif (self.dtype == torch.bfloat16 and t * top <= self.SMALL_MAX_PAIRS
              and kernels.expert_rows_small(True, h, self.gate_up, f, plan, n, tiles, order, top, weight, act,
                                            pair=self.pair)):
            # few rows (decoded tokens): the weights are what moves; a warp per weight row
            if not kernels.expert_rows_small(False, act, self.down, d, plan, n, tiles, order, top, weight,
                                             pair_out):
                kernels.expert_tiles(False, act, self.down, d, plan, n, tiles, order, top, weight, pair_out)
        else:
            kernels.expert_tiles(True, h, self.gate_up, f, plan, n, tiles, order, top, weight, act,
                                 pair=self.pair)
            kernels.expert_tiles(False, act, self.down, d, plan, n, tiles, order, top, weight, pair_out)
        kernels.combine(pair_out, top, residual)
        if self.shared is not None:
            self.shared.forward(ctx, h, residual)


FEED_FORWARDS.register("dense_act", ActivatedFeedForward)
FEED_FORWARDS.register("glu_capped", CappedGLU)
FEED_FORWARDS.register("moe", MixtureOfExperts)
