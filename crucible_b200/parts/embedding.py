"""Token embedding and LM head.

Embedding: x[t, :] = table[token[t], :], no scaling (`model.py:347`,
`engine/kernels/kernels.cu:1049-1059`); the gathered row is widened into the
fp32 residual stream; an id -(s + 1) stands for the token the engine last chose for
state slot s and is read on the device (`ctx.device_tokens`).  Head: logits = norm(x[rows]) W^T at the wanted rows only,
never [T, V] (`engine/src/gpu_model.rs:3590-3613`); W is the embedding table
when the model ties them (`model.py:289`), else its own matrix.  Logits are fp32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import EMBEDDINGS, HEADS, Embedding, Head, TensorDecl


class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, width: int):
        self.vocab_size = vocab_size
        self.width = width
        self.table = None

    def tensors(self):
        return [TensorDecl("table", (self.vocab_size, self.width))]

    def bind(self, tensors, dtype, device):
        self.table = tensors["table"]
        ops.declare_weights(self.table)

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        x = ctx.scratch("residual", (token_ids.shape[0], self.width), torch.float32)
        ops.embed_rows(self.table, token_ids, x, getattr(ctx, "device_tokens", None))
        return x


class NormedStreamsEmbedding(Embedding):
    """x0 = rmsnorm(table[token]) * gain, copied into every one of `streams` residual
    streams: fp32 [T, streams, width] (or [T, width] when `streams` is None).  Option
    `gain_offset`: the stored weight plus this number is the gain (a weight kept around zero)."""

    def __init__(self, spec, vocab_size: int, width: int):
        self.vocab_size = vocab_size
        self.width = width
        self.eps = float(spec.option("eps", 1e-6))
        self.streams = spec.option("streams")
        # the norm's weight may be stored around zero: the gain is then 1 + weight
        self.gain_offset = float(spec.option("gain_offset", 0.0))
        self.table = self.gain = None

    def tensors(self):
        init = ("normal", 0.0, 0.1) if self.gain_offset else None
        return [TensorDecl("table", (self.vocab_size, self.width)),
                TensorDecl("norm_gain", (self.width,), role="vector", init=init)]

    def bind(self, tensors, dtype, device):
        self.table, self.gain = tensors["table"], tensors["norm_gain"]
        if self.gain_offset:
            self.gain = (self.gain.to(torch.float32) + self.gain_offset).contiguous()
        ops.declare_weights(self.table)

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        from ..ops import streams
        n = int(self.streams or 1)
        x = ctx.scratch("residual", (token_ids.shape[0], n, self.width), torch.float32)
        streams.embed_norm(self.table, token_ids, self.gain, self.eps, x,
                           getattr(ctx, "device_tokens", None))
        return x if self.streams is not None else x.view(token_ids.shape[0], self.width)


class HashedPositionEmbedding(Embedding):
    """x = table[token] * scale + bigram[(previous * mul_prev + token * mul_cur) mod buckets]
    + positions[p].  The first token of a sequence takes the bigram row after the buckets.
    The bigram table and the learned positions are options of the spec (`bigram`: (buckets,
    mul_prev, mul_cur) or None; `max_positions`: rows of the position table or None).  The
    request's last token is state: a portion's first token needs it."""

    def __init__(self, spec, vocab_size: int, width: int):
        self.vocab_size = vocab_size
        self.width = width
        self.scale = float(spec.option("scale", 1.0))
        self.bigram_spec = spec.option("bigram")
        self.max_positions = spec.option("max_positions")
        self.table = self.bigram = self.positions = None
        self.state_binding = None

    def tensors(self):
        out = [TensorDecl("table", (self.vocab_size, self.width))]
        if self.bigram_spec is not None:
            out.append(TensorDecl("bigram", (int(self.bigram_spec[0]) + 1, self.width)))
        if self.max_positions is not None:
            out.append(TensorDecl("positions", (int(self.max_positions), self.width)))
        return out

    def state_bytes(self) -> int:
        return 4 if self.bigram_spec is not None else 0

    def bind(self, tensors, dtype, device):
        self.table = tensors["table"]
        self.bigram = tensors.get("bigram")
        self.positions = tensors.get("positions")
        ops.declare_weights(self.table, self.bigram, self.positions)

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        x = ctx.scratch("residual", (token_ids.shape[0], self.width), torch.float32)
        state = ctx.state(self.state_binding) if self.state_binding is not None else None
        buckets, mul_prev, mul_cur = self.bigram_spec if self.bigram_spec is not None else (0, 0, 0)
        ops.hashed_embedding(self.table, self.bigram, self.positions, token_ids, ctx, state, x, self.scale,
                             int(buckets), int(mul_prev), int(mul_cur),
                             getattr(ctx, "device_tokens", None))
        return x


class LMHead(Head):
    """logits = rows W^T; option `softcap` (a positive number c): logits <- c tanh(logits / c)."""

    def __init__(self, vocab_size: int, width: int, tied: bool, softcap=None):
        self.vocab_size = vocab_size
        self.width = width
        self.tied = tied
        self.weight = None
        self.softcap = float(softcap) if softcap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"the head's soft cap must be positive, got {softcap!r}")

    def tensors(self):
        return [] if self.tied else [TensorDecl("weight", (self.vocab_size, self.width))]

    def bind(self, tensors, dtype, device):
        if not self.tied:
            self.weight = tensors["weight"]
            ops.declare_weights(self.weight)

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, ctx, normed_rows: torch.Tensor) -> torch.Tensor:
        logits = ctx.scratch("logits", (normed_rows.shape[0], self.vocab_size), torch.float32)
        ops.linear(normed_rows, self.weight, logits)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits


EMBEDDINGS.register("token", lambda spec, vocab, width: TokenEmbedding(vocab, width))
EMBEDDINGS.register("token_normed_streams", NormedStreamsEmbedding)
EMBEDDINGS.register("token_hashed_positions", HashedPositionEmbedding)
HEADS.register("linear", lambda spec, vocab, width, tied: LMHead(vocab, width, tied, spec.option("softcap")))
