"""Attention over a cached latent with a rotated key part that all heads share.

q = h Wq^T, head by head [dim unrotated | rot rotated]; h Wdkv^T = [latent: rank | key
part: rot].  c = rmsnorm(latent) * gain; per head the unrotated key is W_uk c and the value
W_uv c; the score of head i is (q_plain_i . k_plain_i + rotate(q_rot_i) . rotate(key part))
* scale, softmax over the earlier tokens (all of them, or the last `window`), and the head's
output, gated, goes through Wo.  Only [c | rotated key part] is cached, one row per token
for all heads.

Options of the spec (beside heads, head_dim, softmax_scale, window, position):
  rot_dim, value_dim, kv_rank, norm_eps;
  q_rank      None: q = h Wq^T (tensor `q`).  A number: the queries go through a latent of
              their own, c_q = rmsnorm(h Wdq^T) * gain (`dq`, `dq.norm`), q = c_q Wuq^T (`uq`);
  gate        True or "head": the head's output times sigmoid(h Wg^T)_i, one logit a head
              (`g` [heads, width], logits in float32); "element": the concatenated heads times
              sigmoid(h Wg^T) feature by feature (`g` [heads * value_dim, width]); False: none;
  sink        True: a learned number per head (`sink` [heads]) joins the softmax's denominator
              as exp(sink), with no key and no value, unscaled;
  reads_other True: the layer has no Wdkv; it reads the rows another layer left in the pages
              (the run order names that layer: `RunEntry.cache_of`) with its own W_uk, W_uv,
              queries and window;
  cache_window  the window the pages are kept for, when other layers with other windows read
              them too (default: the layer's own window).

How it runs: each head's key matrix is folded into its query (q'_i = [W_uk_i^T q_plain_i |
rotated q_rot_i]), so a head's scores over the cache are q'_i . [c | key part]: the paged
attention of `heads` query heads over ONE key head of size rank + rot, whose cached row also
serves as the value; the first `rank` features of the result are sum_j p_j c_j, which W_uv_i
takes to the head's output.  The rotation is the spec's position encoding (any that gives
`frequencies()`; it says which features pair, `split_halves`, and may scale cos and sin,
`magnitude()`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import MixerSpec
from ..ops import latent as kernels
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, TensorDecl


class LatentAttention(Mixer):
    fuses_norm = True          # h goes into products only: few rows are normalised on their way in
    takes_prenormed = False

    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.R = int(s.option("rot_dim", 0))
        self.E = int(s.option("value_dim", s.head_dim))
        self.C = int(s.option("kv_rank", 0))
        self.eps = float(s.option("norm_eps", 1e-6))
        gate = s.option("gate", True)
        self.gate = {True: "head", False: None, None: None}.get(gate, gate)
        self.q_rank = s.option("q_rank")
        self.reads_other = bool(s.option("reads_other", False))
        self.has_sink = bool(s.option("sink", False))
        if self.H <= 0 or self.D <= 0 or self.E <= 0 or self.C <= 0 or self.R < 0 or self.R % 2:
            raise ValueError("latent attention: positive heads, dim, vdim and kv_rank; an even rot_dim")
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"latent attention: gate is 'head', 'element' or none, got {gate!r}")
        if self.q_rank is not None and int(self.q_rank) <= 0:
            raise ValueError("latent attention: q_rank must be positive")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window must be positive, got {s.window}")
        options = dict(s.extra)
        self.cache_window = options["cache_window"] if "cache_window" in options else s.window
        if self.cache_window is not None and (s.window is None or self.cache_window < s.window):
            raise ValueError("latent attention: the pages must be kept for at least the layer's own window")
        self.position = (POSITIONS.build(s.position.kind, s.position) if s.position is not None else None)
        if self.position is not None and (not hasattr(self.position, "frequencies")
                                          or self.position.spec.rotary_dim > self.R):
            raise ValueError("latent attention: the rotated part needs a position encoding that gives "
                             "`frequencies()` over at most rot_dim features")
        # of the rot_dim features the encoding's first rotary_dim turn, the rest pass unchanged
        self.turned = self.position.spec.rotary_dim if self.position is not None else 0

    def tensors(self):
        d, H, D, R, E, C = self.spec.width, self.H, self.D, self.R, self.E, self.C
        out = []
        if self.q_rank is None:
            out.append(TensorDecl("q", (H * (D + R), d)))
        else:
            r = int(self.q_rank)
            out += [TensorDecl("dq", (r, d)), TensorDecl("dq.norm", (r,), role="vector", init=("normal", 1.0, 0.1)),
                    TensorDecl("uq", (H * (D + R), r))]
        if not self.reads_other:
            out += [TensorDecl("dkv", (C + R, d)), TensorDecl("dkv.norm", (C,), role="vector")]
        out += [TensorDecl("uk", (H * D, C)), TensorDecl("uv", (H * E, C)), TensorDecl("o", (d, H * E))]
        if self.gate == "head":
            out.append(TensorDecl("g", (H, d)))
        elif self.gate == "element":
            out.append(TensorDecl("g", (H * E, d)))
        if self.has_sink:
            out.append(TensorDecl("sink", (H,), role="vector", init=("normal", 0.0, 1.0)))
        return out

    def bind(self, tensors, dtype, device):
        H, D, E, C = self.H, self.D, self.E, self.C
        # one joint product of everything that reads h and leaves in the engine dtype:
        # [q (unless it has a latent of its own) | dkv (unless another layer's rows are read) |
        #  the gate's logits (feature by feature)]
        joint, at = [], 0
        self.q_at = self.dkv_at = self.gate_at = None
        if self.q_rank is None:
            joint.append(tensors["q"]); self.q_at = at; at += tensors["q"].shape[0]
        if not self.reads_other:
            joint.append(tensors["dkv"]); self.dkv_at = at; at += tensors["dkv"].shape[0]
        if self.gate == "element":
            joint.append(tensors["g"]); self.gate_at = at; at += tensors["g"].shape[0]
        self.w_in = torch.cat(joint, 0).contiguous() if joint else None
        self.w_gate = tensors.get("g") if self.gate == "head" else None
        self.gain = tensors.get("dkv.norm")
        self.w_dq = tensors.get("dq")
        self.dq_gain = tensors.get("dq.norm")
        self.w_uq = tensors.get("uq")
        # head i's key matrix transposed: [rank, dim] takes q_plain_i to the latent's space
        self.uk_t = tensors["uk"].view(H, D, C).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(H, E, C).contiguous()
        self.w_out = tensors["o"]
        self.sinks = tensors.get("sink") if self.has_sink else None
        self.dtype = dtype
        ops.declare_weights(self.w_in, self.w_gate, self.uk_t, self.uv, self.w_out, self.w_dq, self.w_uq)
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def cache_need(self):
        return CacheNeed(kv_heads=1, head_dim=self.C + self.R, window=self.cache_window, values_are_keys=True)

    def forward(self, ctx, h, residual, binding):
        t, H, D, R, E, C = h.shape[0], self.H, self.D, self.R, self.E, self.C
        hq, row = H * (D + R), C + R
        if self.reads_other and binding.write:
            raise ValueError("latent attention: a layer without Wdkv must be run with another layer's cache")
        proj = None
        if self.w_in is not None:
            proj = ctx.scratch("latent.proj", (t, self.w_in.shape[0]), self.dtype)
            ops.linear(h, self.w_in, proj)
        if self.q_rank is None:
            q = proj[:, self.q_at:self.q_at + hq]
        else:
            # the queries' latent: the product leaves float32, the norm reads that
            r = int(self.q_rank)
            cq32 = ctx.scratch("latent.cq32", (t, r), torch.float32)
            ops.linear(h, self.w_dq, cq32)
            cq = ctx.scratch("latent.cq", (t, r), self.dtype)
            ops.rmsnorm(cq32, self.dq_gain, self.eps, cq)
            q = ctx.scratch("latent.q", (t, hq), self.dtype)
            ops.linear(cq, self.w_uq, q)
        cache = ctx.cache(binding.group)
        qx = ctx.scratch("latent.qx", (t, H * row), self.dtype)
        freq, mscale, split = None, 1.0, True
        if self.turned:
            freq = self.position.frequencies()[0]
            mscale = float(getattr(self.position, "magnitude", lambda: 1.0)())
            split = bool(getattr(self.position, "split_halves", True))
        dkv = proj[:, self.dkv_at:self.dkv_at + row] if (self.dkv_at is not None and binding.write) else None
        kernels.prepare(dkv, q, qx, self.gain, freq, mscale, self.eps, H, D, C, R, self.turned, ctx, cache,
                        binding, split_halves=split)
        kernels.heads_linear(q, D + R, self.uk_t, qx, row)
        ox = ctx.scratch("latent.ox", (t, H * row), self.dtype)
        if self.sinks is not None:
            # the softmax with one more term in its denominator: the attention that has a sink,
            # over the same ONE key head whose rows are keys and values at once
            from ..ops import sink_attention
            sink_attention.attention(qx, None, ox, self.sinks, H, 1, row, row, self.spec.softmax_scale,
                                     self.spec.window, 0, 1.0, ctx, cache, binding)
        else:
            ops.paged_attention(qx, ox, H, 1, row, self.spec.softmax_scale, self.spec.window, ctx, cache, binding)
        act = ctx.scratch("latent.act", (t, H * E), self.dtype)
        logit = gate_rows = None
        if self.w_gate is not None:
            logit = ctx.scratch("latent.gate", (t, H), torch.float32)
            ops.linear(h, self.w_gate, logit)
        elif self.gate_at is not None:
            gate_rows = proj[:, self.gate_at:self.gate_at + H * E]
        kernels.heads_linear(ox, row, self.uv, act, E, gate_logit=logit, gate_rows=gate_rows)
        ops.linear(act, self.w_out, residual, accumulate=True, closes=ctx)


MIXERS.register("latent_attention", LatentAttention)
