"""Wrappers of `csrc/sink_attention.cu`: attention whose window keeps the first
tokens and whose softmax has a sink; keys and values of sizes of their own."""
from __future__ import annotations

from typing import Optional

import torch

from . import KernelError, _c_float, _c_int, _check, _code, _need_cuda, _ptr, _stream, build


def rotate_norm_append(proj: torch.Tensor, freq: Optional[torch.Tensor], rotary_dim: int,
                       n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                       value_eps: float, ctx, cache, binding) -> None:
    """Rows of `proj` are [q | k | v | ...]: q and k turn by position * freq (interleaved
    pairs), q in place; k and the unit-rms v go to the token's place in the pages."""
    _need_cuda(proj, freq)
    if proj.stride(1) != 1:
        raise KernelError("rotate_norm_append: rows must be contiguous")
    if rotary_dim and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != rotary_dim):
        raise KernelError("rotate_norm_append: freq is float32 [rotary_dim / 2]")
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    if k_cache.dtype != proj.dtype:
        raise KernelError("rotate_norm_append: cache dtype differs from the activations'")
    if k_cache.shape[-1] != key_dim or v_cache.shape[-1] != value_dim:
        raise KernelError("rotate_norm_append: the pages' sizes differ from the heads'")
    table = ctx.block_table(binding.group)
    lib = build.load("sink_attention")
    _check(lib.cb_rotate_norm_append(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(freq), _c_int(rotary_dim),
        _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table), _c_int(table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), _c_int(proj.shape[0]), _c_int(n_heads), _c_int(n_kv_heads),
        _c_int(key_dim), _c_int(value_dim), _c_int(cache.page_tokens),
        _c_int(1 if binding.write else 0), _c_float(value_eps), _stream()), "rotate_norm_append")


def norm_rotate_append(proj: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                       qk_eps: float, freq: Optional[torch.Tensor], rotary_dim: int, split_halves: bool,
                       n_heads: int, n_kv_heads: int, key_dim: int, value_dim: int,
                       value_eps: Optional[float], ctx, cache, binding, whole_norm: bool = False) -> None:
    """The general preparation of rows [q | k | v | ...]: every q and k head is divided by its
    root mean square and multiplied by `q_gain` / `k_gain` (float32 [key_dim], shared by the
    heads; None: no norm), then its first `rotary_dim` features turn by position * freq, as
    neighbouring pairs or as split halves; q in place, k and v to the token's place in the
    pages; v divided by its root mean square if `value_eps` is given.  `whole_norm`: one root
    mean square over all of a token's q features and one over all of its k features instead of
    one per head; the gains are then float32 [n_heads * key_dim] and [n_kv_heads * key_dim]."""
    _need_cuda(proj, q_gain, k_gain, freq)
    if proj.stride(1) != 1:
        raise KernelError("norm_rotate_append: rows must be contiguous")
    if rotary_dim and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != rotary_dim):
        raise KernelError("norm_rotate_append: freq is float32 [rotary_dim / 2]")
    for g, heads in ((q_gain, n_heads), (k_gain, n_kv_heads)):
        if g is not None and (g.dtype != torch.float32 or not g.is_contiguous()
                              or g.numel() != (heads * key_dim if whole_norm else key_dim)):
            raise KernelError("norm_rotate_append: a gain is float32 [key_dim], or over all heads' "
                              "features when the norm is over the whole projection")
    if whole_norm and (q_gain is None or k_gain is None):
        raise KernelError("norm_rotate_append: a norm over the whole projection needs both gains")
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    if k_cache.dtype != proj.dtype:
        raise KernelError("norm_rotate_append: cache dtype differs from the activations'")
    if k_cache.shape[-1] != key_dim or v_cache.shape[-1] != value_dim:
        raise KernelError("norm_rotate_append: the pages' sizes differ from the heads'")
    table = ctx.block_table(binding.group)
    lib = build.load("sink_attention")
    _check(lib.cb_norm_rotate_append(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(q_gain), _ptr(k_gain),
        _c_float(qk_eps), _ptr(freq), _c_int(rotary_dim), _c_int(1 if split_halves else 0),
        _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table), _c_int(table.shape[1]),
        _ptr(k_cache), _ptr(v_cache), _c_int(proj.shape[0]), _c_int(n_heads), _c_int(n_kv_heads),
        _c_int(key_dim), _c_int(value_dim), _c_int(cache.page_tokens),
        _c_int(1 if binding.write else 0), _c_float(-1.0 if value_eps is None else value_eps),
        _c_int(1 if whole_norm else 0), _stream()), "norm_rotate_append")


def attention(q: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor,
              sinks: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, key_dim: int,
              value_dim: int, scale: float, window: Optional[int], keep_first: int,
              out_scale: float, ctx, cache, binding, gate_per_head: bool = False) -> None:
    """`q`, `gate`, `out`: views of rows (unit stride along features).  Position p sees
    j <= p with p - j < window or j < keep_first.  out = softmax-with-sink(q k) v, times
    sigmoid(gate) if given, times out_scale.  `gate`: rows laid out like `out` (a logit for
    every feature), or [rows, n_heads] with `gate_per_head` (one logit a head)."""
    _need_cuda(q, gate, out, sinks)
    for t in (q, gate, out):
        if t is not None and t.stride(1) != 1:
            raise KernelError("sink attention: rows must be contiguous along features")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads):
        raise KernelError("sink attention: one float32 sink per query head")
    k_cache, v_cache = cache.keys(binding.slot), cache.values(binding.slot)
    table = ctx.block_table(binding.group)
    if gate is not None and gate.dtype != q.dtype:
        raise KernelError("sink attention: the gate's logits are rows of the queries' dtype")
    if _tensor_cores(q, gate, out, sinks, n_heads, n_kv_heads, key_dim, value_dim, scale, window,
                     keep_first, out_scale, ctx, cache, k_cache, v_cache, table, gate_per_head):
        return
    lib = build.load("sink_attention")
    _check(lib.cb_sink_attention(
        _ptr(q), _c_int(q.stride(0)), _ptr(gate), _c_int(gate.stride(0) if gate is not None else 0),
        _ptr(out), _c_int(out.stride(0)), _ptr(k_cache), _ptr(v_cache), _c_int(_code(q.dtype)),
        _ptr(sinks), _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table), _c_int(table.shape[1]),
        _c_int(q.shape[0]), _c_int(n_heads), _c_int(n_kv_heads), _c_int(key_dim), _c_int(value_dim),
        _c_int(cache.page_tokens), _c_float(scale), _c_int(window or 0), _c_int(keep_first),
        _c_float(out_scale), _c_int(1 if gate_per_head else 0), _stream()), "sink attention")


TENSOR_CORES = True      # tests switch it off to reach the plain kernel with the same inputs


def _tensor_cores(q, gate, out, sinks, n_heads, n_kv_heads, key_dim, value_dim, scale, window,
                  keep_first, out_scale, ctx, cache, k_cache, v_cache, table, gate_per_head=False) -> bool:
    """For bfloat16 rows whose keys and values have one size: steps of prompts' portions alone
    with plain softmax and heads of 64 or 128 take the tcgen05 attention (`csrc/attention_tcgen05.cu`);
    everything else of a size that is a multiple of 16 up to 256 the mma.sync kernel of 64-row
    tiles (`csrc/attention_mma.cu`, its extended form): prompts' portions and decoded tokens in
    one launch, the rows of a request's query heads that share a key/value head packed into
    tiles.  Refuses anything else."""
    host = getattr(ctx, "host", None)
    if (not TENSOR_CORES or q.dtype != torch.bfloat16 or key_dim != value_dim or key_dim % 16
            or key_dim > 256 or host is None or q.stride(0) % 8 or out.stride(0) % 2
            or (gate is not None and not gate_per_head and gate.stride(0) % 2)):
        return False
    from . import tensor_core
    # a plain softmax over keys and values of 64 or 128 features, portions of prompts only: the
    # tcgen05 attention, whose tiles take the kept first tokens ahead of the window's
    if (sinks is None and (gate is None or gate_per_head) and out_scale == 1.0
            and tensor_core.prompt_attention(q, out, k_cache, v_cache, n_heads, n_kv_heads, key_dim, scale,
                                             window, keep_first, ctx, cache, table)):
        if gate is not None:
            # one logit a head: a pass over the heads' results behind the attention
            from . import latent
            latent.head_gate(out, gate, n_heads, value_dim)
        return True
    lib = build.load("attention_mma")
    # Few rows per request (decoded tokens, short portions): one row tile each, so the blocks
    # are few; the key tiles are then dealt to several blocks and merged.  The number of shares
    # is a function of the step's shape; any number gives the same sums up to rounding.
    max_rows = host.max_new_tokens * (n_heads // n_kv_heads)
    n_chunks, partial = 1, None
    if max_rows <= 64:
        reach = host.context_bucket if window is None else min(window + 64, host.context_bucket)
        tiles = -(-reach // 64) + (-(-keep_first // 64) if window is not None else 0)
        n_chunks = max(1, min(tiles // 2, 296 // max(1, n_kv_heads * ctx.n_requests), 32))
        if n_chunks > 1:
            partial = ctx.scratch("sink_attention.partial",
                                  (ctx.n_requests * n_kv_heads * n_chunks * max_rows * (key_dim + 2),),
                                  torch.float32)
    code = lib.cb_attention_mma_sink(
        _ptr(q), _c_int(q.stride(0)), _ptr(out), _c_int(out.stride(0)), _ptr(gate),
        _c_int(gate.stride(0) if gate is not None else 0), _ptr(k_cache), _ptr(v_cache), _ptr(sinks),
        _ptr(ctx.req_row_start), _ptr(ctx.req_first_pos), _ptr(table), _c_int(table.shape[1]),
        _c_int(ctx.n_requests), _c_int(host.max_new_tokens), _c_int(n_heads), _c_int(n_kv_heads),
        _c_int(key_dim), _c_int(cache.page_tokens), _c_float(scale), _c_int(window or 0),
        _c_int(keep_first), _c_float(out_scale), _ptr(partial), _c_int(n_chunks),
        _c_int(1 if gate_per_head else 0), _stream())
    if code == 100001:
        return False
    _check(code, "sink attention (tensor cores)")
    return True
