"""Mixers with a matrix memory per head instead of a cache of keys.  Their state is
fp32 in the request's state slot (zero when the slot is handed out) and is carried
from step to step, so a prompt may be cut anywhere.

`gated_delta` (the gated delta rule): q, k [G, D] and v [H, E] pass a short causal
convolution per channel (`<tensor>.conv` [channels, taps], the last tap meets the
current token; its last taps - 1 inputs are state) and SiLU; q and k become unit
vectors per head (x / sqrt(sum x^2 + 1e-6)), q times D^-1/2.  Per head, with
beta = sigmoid(h Wb^T) and g = exp(-exp(A_log) * softplus(h Wa^T + dt_bias)):
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
o / rms(o) * norm [E] * silu(h Wg^T) goes through Wo.  Head i uses q/k head i // (H / G).

`mlstm` (the matrix memory of the xLSTM): q = h Wq^T * D^-1/2, k [H, D], v [H, E];
log gates i = cap * tanh((h Wi^T + bi) / cap), f = logsigmoid(cap * tanh((h Wf^T + bf) / cap));
with m (from 0):  m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;
n likewise with k alone;  o = S^T q / (max(|n . q|, exp(-m')) + 1e-6).
o / rms(o) per head, times norm [H * E], times sigmoid(h Wg^T), goes through Wo.

`wkv` (time mixing with a decay per key channel): with h' the row of the token before
(zeros at a sequence's start; the last row seen is state), each of r, k, v, g, w reads its
own mix  h + (h' - h) * mu_s.  r, k, v = W_s mix_s [H, D]; gate = silu(Wg mix_g); decay
w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per head and key channel (W_w1 has as many rows
as the checkpoint gives it).  Per head:
    o = (S + diag(u) k v^T)^T r;   S <- diag(w) S + k v^T.
o / rms(o) per head, times norm [H * D], times the gate, goes through Wo.

`mamba2` (state space): h W_in^T = [z: H*P | x: H*P | B: G*N | C: G*N | dt: H]; x, B, C pass
a short causal convolution per channel with bias (its last taps - 1 inputs are state) and
SiLU; dt = softplus(dt + dt_bias).  Per head (head i uses group i // (H / G)):
    S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x.
y * silu(z), then unit rms in `norm_groups` equal parts of the row, times norm [H * P], goes
through Wo.

`retention` (linear attention with a fixed decay per head, no softmax and no denominator):
q, k [H, D], v [H, E]; q and k turn by the spec's position encoding (the first rotary_dim
features of each head), k times D^-1/2 after the rotation.  Per head, with the constant
decay_h of the spec's option `decay`:
    S <- decay_h S + k v^T;   o = S^T q.
o / rms(o) per head (no weight), times silu(h Wg^T), goes through Wo.
"""
from __future__ import annotations

import torch

from ..config.model_config import MixerSpec
from ..ops import recurrent as kernels
from .. import ops
from .base import MIXERS, POSITIONS, Mixer, TensorDecl
from .branch import BranchMixer


def _round16(n: int) -> int:
    return (n + 15) // 16 * 16


class GatedDeltaRule(BranchMixer):
    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.G, self.D = s.n_heads, s.n_kv_heads, s.head_dim
        self.E = int(s.option("value_dim", s.head_dim))
        self.taps = int(s.option("conv_taps", 4))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.G <= 0 or self.H % self.G or self.D <= 0 or self.E <= 0 or self.taps < 1:
            raise ValueError("gated_delta: heads must be a multiple of kv_heads; sizes positive")
        if self.D > 256:
            raise ValueError("gated_delta: key size up to 256")
        self.C = 2 * self.G * self.D + self.H * self.E          # channels under the convolution
        self.s_bytes = _round16(4 * self.H * self.D * self.E)
        self.tail_bytes = 4 * (self.taps - 1) * self.C

    def tensors(self):
        d, H, G, D, E = self.spec.width, self.H, self.G, self.D, self.E
        conv = ("uniform", -0.5, 0.5)
        return [TensorDecl("q", (G * D, d)), TensorDecl("k", (G * D, d)), TensorDecl("v", (H * E, d)),
                TensorDecl("q.conv", (G * D, self.taps), role="vector", init=conv),
                TensorDecl("k.conv", (G * D, self.taps), role="vector", init=conv),
                TensorDecl("v.conv", (H * E, self.taps), role="vector", init=conv),
                TensorDecl("b", (H, d)), TensorDecl("a", (H, d)),
                TensorDecl("A_log", (H,), role="vector", init=("uniform", -1.0, 1.0)),
                TensorDecl("dt_bias", (H,), role="vector", init=("uniform", -1.0, 1.0)),
                TensorDecl("norm", (E,), role="vector"),
                TensorDecl("g", (H * E, d)), TensorDecl("o", (d, H * E))]

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], 0).contiguous()
        self.w_gates = torch.cat([tensors["b"], tensors["a"]], 0).contiguous()
        self.w_out = tensors["o"]
        self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], 0).contiguous()
        self.a_log, self.dt_bias, self.gain = tensors["A_log"], tensors["dt_bias"], tensors["norm"]
        self.dtype = dtype
        self._declare()

    def state_bytes(self) -> int:
        return self.s_bytes + self.tail_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        t, H, G, D, E, C = proj.shape[0], self.H, self.G, self.D, self.E, self.C
        state = ctx.state(binding)
        qkv = ctx.scratch("delta.qkv", (t, C), torch.float32)
        beta = ctx.scratch("delta.beta", (t, H), torch.float32)
        decay = ctx.scratch("delta.decay", (t, H), torch.float32)
        o = ctx.scratch("delta.o", (t, H * E), torch.float32)
        kernels.delta_prepare(proj, self.conv_w, self.taps, gates, self.a_log, self.dt_bias, ctx,
                              state, self.s_bytes, qkv, beta, decay, H, G, D, E)
        kernels.conv_tail_update(proj, self.taps, C, ctx, state, self.s_bytes)
        kernels.matrix_memory(kernels.DELTA, qkv, 0, G * D, 2 * G * D, decay, beta, ctx, state, 0, 0,
                              0, o, H, G, D, E)
        kernels.head_norm_gate(o, self.gain, False, proj[:, C:C + H * E], act, kernels.GATE_SILU, H, E,
                               self.eps, out_scale)


class MLSTM(BranchMixer):
    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.E = int(s.option("value_dim", s.head_dim))
        self.cap = float(s.option("gate_cap", 15.0))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.D <= 0 or self.E <= 0 or self.cap <= 0:
            raise ValueError("mlstm: heads, sizes and the gates' cap must be positive")
        if self.D > 256:
            raise ValueError("mlstm: key size up to 256")
        self.s_bytes = _round16(4 * self.H * self.D * self.E)
        self.n_bytes = _round16(4 * self.H * self.D)
        self.m_bytes = _round16(4 * self.H)

    def tensors(self):
        d, H, D, E = self.spec.width, self.H, self.D, self.E
        return [TensorDecl("q", (H * D, d)), TensorDecl("k", (H * D, d)), TensorDecl("v", (H * E, d)),
                TensorDecl("g", (H * E, d)), TensorDecl("o", (d, H * E)),
                TensorDecl("norm", (H * E,), role="vector"),
                TensorDecl("i", (H, d)), TensorDecl("i.b", (H,), role="vector", init=("normal", 0.0, 1.0)),
                TensorDecl("f", (H, d)), TensorDecl("f.b", (H,), role="vector", init=("uniform", 1.0, 4.0))]

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], 0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], 0).contiguous()
        self.w_out = tensors["o"]
        self.bias_i, self.bias_f, self.gain = tensors["i.b"], tensors["f.b"], tensors["norm"]
        self.dtype = dtype
        self._declare()

    def state_bytes(self) -> int:
        return self.s_bytes + self.n_bytes + self.m_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        t, H, D, E = proj.shape[0], self.H, self.D, self.E
        C = 2 * H * D + H * E
        state = ctx.state(binding)
        qkv = ctx.scratch("mlstm.qkv", (t, C), torch.float32)
        log_keep = ctx.scratch("mlstm.keep", (t, H), torch.float32)
        log_in = ctx.scratch("mlstm.in", (t, H), torch.float32)
        o = ctx.scratch("mlstm.o", (t, H * E), torch.float32)
        kernels.mlstm_prepare(proj, gates, self.bias_i, self.bias_f, self.cap, qkv, log_keep, log_in,
                              H, D, E)
        kernels.matrix_memory(kernels.MLSTM, qkv, 0, H * D, 2 * H * D, log_keep, log_in, ctx, state, 0,
                              self.s_bytes, self.s_bytes + self.n_bytes, o, H, H, D, E)
        kernels.head_norm_gate(o, self.gain, True, proj[:, C:C + H * E], act, kernels.GATE_SIGMOID, H, E,
                               self.eps, out_scale)


class WKVMixer(Mixer):
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.rank = int(s.option("decay_rank", 16))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.D <= 0 or self.rank <= 0:
            raise ValueError("wkv: heads, dim and the decay's rank must be positive")
        if self.D > 256:
            raise ValueError("wkv: key size up to 256")
        self.s_bytes = _round16(4 * self.H * self.D * self.D)
        self.prev_bytes = _round16(4 * s.width)

    def tensors(self):
        d, HD = self.spec.width, self.H * self.D
        out = [TensorDecl(f"mu.{m}", (d,), role="vector", init=("uniform", 0.0, 1.0)) for m in self.MIXES]
        out += [TensorDecl(m, (HD, d)) for m in ("r", "k", "v", "g")]
        out += [TensorDecl("w1", (self.rank, d), free_dims=(0,)),
                TensorDecl("w2", (HD, self.rank), free_dims=(1,)),
                TensorDecl("w0", (HD,), role="vector", init=("uniform", -3.0, 0.0)),
                TensorDecl("u", (self.H, self.D), role="vector", init=("normal", 0.0, 0.5)),
                TensorDecl("norm", (HD,), role="vector"), TensorDecl("o", (d, HD))]
        return out

    def bind(self, tensors, dtype, device):
        self.mu = torch.stack([tensors[f"mu.{m}"] for m in self.MIXES], 0).contiguous()
        self.w_proj = [tensors[m] for m in ("r", "k", "v", "g")]
        self.w1, self.w2, self.w_out = tensors["w1"], tensors["w2"], tensors["o"]
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"wkv: the decay's two matrices disagree on its rank "
                             f"({self.w1.shape[0]} and {self.w2.shape[1]})")
        self.rank = int(self.w1.shape[0])
        self.w0, self.u, self.gain = tensors["w0"], tensors["u"].contiguous(), tensors["norm"]
        self.dtype = dtype
        ops.declare_weights(*self.w_proj, self.w1, self.w2, self.w_out)

    def state_bytes(self) -> int:
        return self.s_bytes + self.prev_bytes

    def forward(self, ctx, h, residual, binding):
        t, d, H, D = h.shape[0], self.spec.width, self.H, self.D
        HD = H * D
        state = ctx.state(binding)
        mixes = ctx.scratch("wkv.mixes", (len(self.MIXES), t, d), self.dtype)
        kernels.shift_mix(h, self.mu, ctx, state, self.s_bytes, mixes)
        rkvg = ctx.scratch("wkv.rkvg", (4, t, HD), self.dtype)
        for i, w in enumerate(self.w_proj):
            ops.linear(mixes[i], w, rkvg[i])
        low = ctx.scratch("wkv.low", (t, self.rank), torch.float32)
        ops.linear(mixes[4], self.w1, low)
        low_t = ctx.scratch("wkv.low_t", (t, self.rank), self.dtype)
        ops.activation("tanh", low, low_t)
        logit = ctx.scratch("wkv.logit", (t, HD), torch.float32)
        ops.linear(low_t, self.w2, logit)
        qkv = ctx.scratch("wkv.qkv", (t, 4 * HD), torch.float32)
        kernels.wkv_prepare(rkvg, logit, self.w0, qkv, HD)
        o = ctx.scratch("wkv.o", (t, HD), torch.float32)
        kernels.matrix_memory(kernels.WKV, qkv, 0, HD, 2 * HD, None, None, ctx, state, 0, 0, 0, o,
                              H, H, D, D, w_off=3 * HD, per_head=self.u)
        act = ctx.scratch("wkv.act", (t, HD), self.dtype)
        kernels.head_norm_gate(o, self.gain, True, rkvg[3], act, kernels.GATE_SILU, H, D, self.eps, 1.0)
        ops.linear(act, self.w_out, residual, accumulate=True, closes=ctx)


class StateSpaceMixer(BranchMixer):
    fuses_norm = True          # h goes into products only: few rows are normalised on their way in
    takes_prenormed = False

    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.G, self.N = s.n_heads, s.n_kv_heads, s.head_dim
        self.P = int(s.option("value_dim", s.head_dim))
        self.taps = int(s.option("conv_taps", 4))
        self.parts = int(s.option("norm_groups", 1))
        self.eps = float(s.option("norm_eps", 1e-6))
        self.inner = self.H * self.P
        if self.H <= 0 or self.G <= 0 or self.H % self.G or self.N <= 0 or self.P <= 0 or self.taps < 1:
            raise ValueError("mamba2: heads must be a multiple of groups; sizes positive")
        if self.parts <= 0 or self.inner % self.parts:
            raise ValueError("mamba2: norm_groups must divide heads * vdim")
        if self.N > 256:
            raise ValueError("mamba2: state size up to 256")
        self.C = self.inner + 2 * self.G * self.N           # channels under the convolution
        self.s_bytes = _round16(4 * self.H * self.N * self.P)
        self.tail_bytes = 4 * (self.taps - 1) * self.C

    def tensors(self):
        d, H = self.spec.width, self.H
        return [TensorDecl("in", (self.inner + self.C + H, d)),
                TensorDecl("conv", (self.C, self.taps), role="vector", init=("uniform", -0.5, 0.5)),
                TensorDecl("conv.b", (self.C,), role="vector", init=("uniform", -0.2, 0.2)),
                TensorDecl("dt_bias", (H,), role="vector", init=("uniform", -2.0, 1.0)),
                TensorDecl("A_log", (H,), role="vector", init=("uniform", -1.0, 1.0)),
                TensorDecl("D", (H,), role="vector", init=("normal", 1.0, 0.3)),
                TensorDecl("norm", (self.inner,), role="vector"), TensorDecl("o", (d, self.inner))]

    def bind(self, tensors, dtype, device):
        n = self.inner + self.C
        self.w_in = tensors["in"][:n].contiguous()
        self.w_gates = tensors["in"][n:].contiguous()
        self.w_out = tensors["o"]
        self.conv_w, self.conv_b = tensors["conv"].contiguous(), tensors["conv.b"]
        self.a_log, self.dt_bias, self.skip = tensors["A_log"], tensors["dt_bias"], tensors["D"]
        self.gain = tensors["norm"]
        self.dtype = dtype
        self._declare()

    def state_bytes(self) -> int:
        return self.s_bytes + self.tail_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        if out_scale != 1.0:
            raise ValueError("mamba2: a branch scale other than 1 is not supported")
        t, H, G, N, P, C, inner = proj.shape[0], self.H, self.G, self.N, self.P, self.C, self.inner
        state = ctx.state(binding)
        xbc = ctx.scratch("ssd.xbc", (t, C), torch.float32)
        decay = ctx.scratch("ssd.decay", (t, H), torch.float32)
        step = ctx.scratch("ssd.step", (t, H), torch.float32)
        y = ctx.scratch("ssd.y", (t, inner), torch.float32)
        kernels.ssd_prepare(proj, inner, self.conv_w, self.conv_b, self.taps, gates, self.a_log,
                            self.dt_bias, ctx, state, self.s_bytes, xbc, decay, step, H, C)
        kernels.conv_tail_update(proj[:, inner:inner + C], self.taps, C, ctx, state, self.s_bytes)
        kernels.matrix_memory(kernels.SSD, xbc, inner + G * N, inner, 0, decay, step, ctx, state, 0, 0, 0,
                              y, H, G, N, P, per_head=self.skip)
        kernels.gate_group_norm(y, proj[:, :inner], self.gain, act, self.parts, self.eps)


class Retention(BranchMixer):
    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.E = int(s.option("value_dim", s.head_dim))
        self.eps = float(s.option("norm_eps", 1e-6))
        self.decay_values = tuple(float(x) for x in (s.option("decay") or ()))
        if self.H <= 0 or self.D <= 0 or self.E <= 0:
            raise ValueError("retention: heads and sizes must be positive")
        if self.D > 256:
            raise ValueError("retention: key size up to 256")
        if len(self.decay_values) != self.H or not all(0.0 <= x <= 1.0 for x in self.decay_values):
            raise ValueError("retention: one decay in [0, 1] for every head")
        self.position = POSITIONS.build(s.position.kind, s.position) if s.position is not None else None
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError("retention: the position encoding must give `frequencies()`")
        self.s_bytes = _round16(4 * self.H * self.D * self.E)

    def tensors(self):
        d, H, D, E = self.spec.width, self.H, self.D, self.E
        return [TensorDecl("q", (H * D, d)), TensorDecl("k", (H * D, d)), TensorDecl("v", (H * E, d)),
                TensorDecl("g", (H * E, d)), TensorDecl("o", (d, H * E))]

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], 0).contiguous()
        self.w_out = tensors["o"]
        # the decays are numbers of the configuration: float32 as they are; the state-space
        # rule's skip is zero here
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)
        self.no_skip = torch.zeros(self.H, dtype=torch.float32, device=device)
        self.dtype = dtype
        self._declare()
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def state_bytes(self) -> int:
        return self.s_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        t, H, D, E = proj.shape[0], self.H, self.D, self.E
        C = 2 * H * D + H * E
        state = ctx.state(binding)
        qkv = ctx.scratch("retention.qkv", (t, C), torch.float32)
        keep = ctx.scratch("retention.keep", (t, H), torch.float32)
        step = ctx.scratch("retention.step", (t, H), torch.float32)
        o = ctx.scratch("retention.o", (t, H * E), torch.float32)
        freq, rotary_dim = self.position.frequencies() if self.position is not None else (None, 0)
        split = bool(getattr(self.position, "split_halves", True))
        kernels.retention_prepare(proj, freq, rotary_dim, split, ctx, self.decay, float(D) ** -0.5, qkv,
                                  keep, step, H, D, E)
        kernels.matrix_memory(kernels.SSD, qkv, 0, H * D, 2 * H * D, keep, step, ctx, state, 0, 0, 0, o,
                              H, H, D, E, per_head=self.no_skip)
        kernels.head_norm_gate(o, None, False, proj[:, C:C + H * E], act, kernels.GATE_SILU, H, E,
                               self.eps, out_scale)


MIXERS.register("gated_delta", GatedDeltaRule)
MIXERS.register("retention", Retention)
MIXERS.register("wkv", WKVMixer)
MIXERS.register("mamba2", StateSpaceMixer)
MIXERS.register("mlstm", MLSTM)
