"""Grouped-query attention whose window keeps the first tokens, with a sink in the
softmax, unit-rms values, keys and values of sizes of their own, rotation of
interleaved pairs, and a sigmoid output gate.

q = h Wq^T [H, D], k = h Wk^T [G, D], v = h Wv^T [G, E]; query head i reads key/value
head i // (H / G).  q and k turn by the rotation of the spec's position encoding
(`rope_interleaved`); v / rms(v) (eps, no gain) is what the cache holds.  A row at
position p sees j <= p with p - j < window or j < keep_first (kept tokens keep their
own positions).  s_j = (q . k_j) * scale; the weights are exp(s_j - m) / (sum_j
exp(s_j - m) + exp(sink_i - m)): the sink of head i has no key and no value and is not
scaled.  The heads' results times sigmoid(h Wg^T) go through Wo.

Options of the spec: value_dim (default head_dim), keep_first (default 0), sink
(default true), value_norm_eps (None: values are cached as they are), gate (default
true or "element": a logit for every output feature, `g` [H * E, width]; "head": one logit a
head, `g` [H, width]; false: none), qk_norm_eps (default None; a number: every q and k head is
divided by its root mean square over D, that eps under the root, and multiplied by the weight
`q.norm` / `k.norm` of size D that all heads share, before the rotation), qk_norm_whole
(default false; true: the root mean square is taken over the whole projection, all H * D
features of q at once and all G * D of k, and the weights have those sizes).  `window` None
means every earlier key.
The position encoding says which features pair (`split_halves`: i with i + R/2, else
neighbours).
"""
from __future__ import annotations

import torch

from ..config.model_config import MixerSpec
from ..ops import sink_attention as kernels
from .base import MIXERS, POSITIONS, CacheNeed, TensorDecl
from .branch import BranchMixer


class SinkWindowAttention(BranchMixer):
    def __init__(self, spec: MixerSpec):
        if spec.n_heads <= 0 or spec.n_kv_heads <= 0 or spec.head_dim <= 0:
            raise ValueError("attention needs positive n_heads, n_kv_heads and head_dim")
        if spec.n_heads % spec.n_kv_heads != 0:
            raise ValueError(f"n_heads ({spec.n_heads}) is not divisible by "
                             f"n_kv_heads ({spec.n_kv_heads})")
        if spec.window is not None and spec.window <= 0:
            raise ValueError(f"window must be positive, got {spec.window}")
        self.spec = spec
        self.value_dim = int(spec.option("value_dim", spec.head_dim))
        self.keep_first = int(spec.option("keep_first", 0))
        self.has_sink = bool(spec.option("sink", True))
        gate = spec.option("gate", True)
        self.gate = {True: "element", False: None, None: None}.get(gate, gate)
        if self.gate not in (None, "element", "head"):
            raise ValueError(f"attention: gate is 'element', 'head' or none, got {gate!r}")
        self.has_gate = self.gate is not None
        self.qk_whole = bool(spec.option("qk_norm_whole", False))
        self.value_eps = spec.option("value_norm_eps")
        self.qk_eps = spec.option("qk_norm_eps")
        if self.keep_first < 0 or self.value_dim <= 0:
            raise ValueError("keep_first must not be negative and value_dim must be positive")
        self.position = (POSITIONS.build(spec.position.kind, spec.position)
                         if spec.position is not None else None)
        if self.position is not None and not hasattr(self.position, "frequencies"):
            raise ValueError("this attention turns interleaved pairs: its position encoding "
                             "must give `frequencies()`")
        self.sinks = None

    def tensors(self):
        s, d = self.spec, self.spec.width
        out = [TensorDecl("q", (s.n_heads * s.head_dim, d)), TensorDecl("k", (s.n_kv_heads * s.head_dim, d)),
               TensorDecl("v", (s.n_kv_heads * self.value_dim, d)),
               TensorDecl("o", (d, s.n_heads * self.value_dim))]
        if self.has_gate:
            out.append(TensorDecl("g", (s.n_heads * (self.value_dim if self.gate == "element" else 1), d)))
        if self.has_sink:
            out.append(TensorDecl("sink", (s.n_heads,), role="vector", init=("normal", 0.0, 1.0)))
        if self.qk_eps is not None:
            nq, nk = (s.n_heads, s.n_kv_heads) if self.qk_whole else (1, 1)
            out += [TensorDecl("q.norm", (nq * s.head_dim,), role="vector", init=("normal", 1.0, 0.1)),
                    TensorDecl("k.norm", (nk * s.head_dim,), role="vector", init=("normal", 1.0, 0.1))]
        return out

    def bind(self, tensors, dtype, device):
        parts = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.has_gate else [])
        # rows of zeros behind a gate of a few logits, so that a row of the joint projection is a
        # multiple of 16 bytes long (the tensor-core attention reads q in 16-byte pieces)
        spare = -sum(t.shape[0] for t in parts) % 8
        if spare and self.gate == "head":
            parts.append(torch.zeros((spare, parts[0].shape[1]), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_out = tensors["o"]
        self.sinks = tensors.get("sink") if self.has_sink else None
        self.q_gain = tensors.get("q.norm") if self.qk_eps is not None else None
        self.k_gain = tensors.get("k.norm") if self.qk_eps is not None else None
        self.dtype = dtype
        self._declare()
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def cache_need(self):
        s = self.spec
        return CacheNeed(kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window,
                         value_dim=self.value_dim if self.value_dim != s.head_dim else None,
                         keep_first=self.keep_first if s.window is not None else 0)

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        s = self.spec
        cache = ctx.cache(binding.group)
        freq, rotary_dim = (self.position.frequencies() if self.position is not None else (None, 0))
        split = bool(getattr(self.position, "split_halves", False))
        if self.qk_eps is None and not split and self.value_eps is not None:
            kernels.rotate_norm_append(proj, freq, rotary_dim, s.n_heads, s.n_kv_heads, s.head_dim,
                                       self.value_dim, float(self.value_eps), ctx, cache, binding)
        else:
            kernels.norm_rotate_append(proj, self.q_gain, self.k_gain,
                                       float(self.qk_eps) if self.qk_eps is not None else 0.0, freq,
                                       rotary_dim, split, s.n_heads, s.n_kv_heads, s.head_dim,
                                       self.value_dim, self.value_eps, ctx, cache, binding,
                                       whole_norm=self.qk_whole and self.qk_eps is not None)
        q_width = s.n_heads * s.head_dim
        g_at = q_width + s.n_kv_heads * (s.head_dim + self.value_dim)
        per_head = self.gate == "head"
        gate = (proj[:, g_at:g_at + s.n_heads * (1 if per_head else self.value_dim)]
                if self.has_gate else None)
        kernels.attention(proj[:, :q_width], gate, act, self.sinks, s.n_heads, s.n_kv_heads,
                          s.head_dim, self.value_dim, s.softmax_scale, s.window, self.keep_first,
                          out_scale, ctx, cache, binding, gate_per_head=per_head)


MIXERS.register("sink_attention", SinkWindowAttention)
