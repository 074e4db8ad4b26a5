"""Wrappers of `csrc/moe.cu`: routing, the plan of row tiles per expert, the experts'
products over those tiles, and the sum of a token's chosen experts."""
from __future__ import annotations

import ctypes

import torch

from . import KernelError, _c_int, _check, _code, _need_cuda, _ptr, _stream, build


def tile_rows() -> int:
    return int(build.load("moe").cb_moe_tile_rows())


GROUPED_TILE_ROWS = 128      # rows of a tile of the tensor cores' grouped product


def max_tiles(n_tokens: int, top: int, n_experts: int, rows: int = 0) -> int:
    """An upper bound of the row tiles of a step: every expert may end on a partial tile.
    `rows`: rows of a tile (0: those of this file's own kernels)."""
    return -(-n_tokens * top // (rows or tile_rows())) + n_experts


def plan_ints(n_experts: int, tiles: int) -> int:
    return 2 + n_experts + 3 * tiles


def _pair(pair):
    """(limit, alpha, offset) of the capped gated pair as C floats; None: silu(g) * u."""
    limit, alpha, offset = pair if pair is not None else (0.0, 1.0, 0.0)
    return ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(offset)


def route(logits, top: int, idx, weight, place, count, plan, tiles: int, sorted_pair, bias=None,
          rows: int = 0) -> None:
    """Per token the `top` largest logits (plus `bias`, float32 [experts], if given; the lower
    index on ties) and their softmax; then
    the sorted order of the (token, choice) pairs by expert and the tiles (of `rows` rows; 0: this
    file's own) over it.  `count`
    (int32 [experts]) is zero between calls: the kernels leave it so."""
    _need_cuda(logits, idx, weight, place, count, plan, sorted_pair, bias)
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("moe route takes contiguous float32 logits [tokens, experts]")
    t, e = logits.shape
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != e or not bias.is_contiguous()):
        raise KernelError("moe route: the bias is float32 [experts]")
    if idx.numel() < t * top or plan.numel() < plan_ints(e, tiles) or sorted_pair.numel() < t * top:
        raise KernelError("moe route: a buffer is too small")
    lib = build.load("moe")
    _check(lib.cb_moe_route(_ptr(logits), _ptr(bias), _c_int(t), _c_int(e), _c_int(top), _ptr(idx), _ptr(weight),
                            _ptr(place), _ptr(count), _ptr(plan), _c_int(tiles), _ptr(sorted_pair),
                            _c_int(rows), _stream()), "moe route")


def expert_tiles(gated: bool, a, w, n_out: int, plan, n_experts: int, tiles: int, sorted_pair, top: int,
                 weight, out, pair=None) -> None:
    """gated: out[sorted place] = silu(a[token] Wg^T) * (a[token] Wu^T) with w [experts, 2 n_out, K]
    (`pair` = (limit, alpha, offset): the capped pair instead, see `ops.glu`);
    else: out[pair] = weight[pair] * a[sorted place] Wd^T with w [experts, n_out, K], float32."""
    _need_cuda(a, w, plan, sorted_pair, weight, out)
    if a.dtype != w.dtype or a.stride(1) != 1 or not w.is_contiguous() or out.stride(1) != 1:
        raise KernelError("moe tiles: rows and weights of one dtype, contiguous rows")
    if (not gated) and out.dtype != torch.float32:
        raise KernelError("moe tiles: the down product writes float32")
    lib = build.load("moe")
    _check(lib.cb_moe_tiles(_c_int(1 if gated else 0), _ptr(a), _c_int(a.stride(0)), _ptr(w),
                            ctypes.c_long(w.stride(0)), _c_int(_code(a.dtype)), _c_int(n_out),
                            _c_int(w.shape[2]), _ptr(plan), _c_int(n_experts), _c_int(tiles),
                            _ptr(sorted_pair), _c_int(top), _ptr(weight), _ptr(out),
                            _c_int(out.stride(0)), *_pair(pair), _stream()),
           "moe gate/up" if gated else "moe down")


def expert_rows_small(gated: bool, a, w, n_out: int, plan, n_experts: int, tiles: int, sorted_pair,
                      top: int, weight, out, pair=None) -> bool:
    """`expert_tiles` for steps of few rows: every weight row is read once by one warp.  False:
    the sizes do not allow it (K not a multiple of 8, rows not 16-byte aligned)."""
    _need_cuda(a, w, plan, sorted_pair, weight, out)
    if a.dtype != w.dtype or a.stride(1) != 1 or not w.is_contiguous() or out.stride(1) != 1:
        raise KernelError("moe rows: rows and weights of one dtype, contiguous rows")
    lib = build.load("moe")
    code = lib.cb_moe_rows_small(_c_int(1 if gated else 0), _ptr(a), _c_int(a.stride(0)), _ptr(w),
                                 ctypes.c_long(w.stride(0)), _c_int(_code(a.dtype)), _c_int(n_out),
                                 _c_int(w.shape[2]), _ptr(plan), _c_int(n_experts), _c_int(tiles),
                                 _ptr(sorted_pair), _c_int(top), _ptr(weight), _ptr(out),
                                 _c_int(out.stride(0)), *_pair(pair), _stream())
    if code == 100001:
        return False
    _check(code, "moe gate/up (few rows)" if gated else "moe down (few rows)")
    return True


def combine(pair_out, top: int, residual) -> None:
    """residual[t] += sum over the token's choices, in their order."""
    _need_cuda(pair_out, residual)
    if pair_out.dtype != torch.float32 or residual.dtype != torch.float32 or not residual.is_contiguous():
        raise KernelError("moe combine adds float32 rows into the float32 residual")
    lib = build.load("moe")
    _check(lib.cb_moe_combine(_ptr(pair_out), _c_int(top), _ptr(residual), _c_int(residual.shape[0]),
                              _c_int(residual.shape[1]), _stream()), "moe combine")


def gather(h, sorted_pair, top: int, out) -> None:
    """out[i] = h[token of the i-th pair in sorted order]."""
    _need_cuda(h, sorted_pair, out)
    lib = build.load("moe")
    _check(lib.cb_moe_gather(_ptr(h), _c_int(h.stride(0)), _c_int(_code(h.dtype)), _ptr(sorted_pair),
                             _c_int(top), _ptr(out), _c_int(out.shape[0]), _c_int(h.shape[1]), _stream()),
           "moe gather")


def scatter(rows, sorted_pair, weight, pair_out) -> None:
    """pair_out[pair] = weight[pair] * rows[the pair's sorted place]."""
    _need_cuda(rows, sorted_pair, weight, pair_out)
    lib = build.load("moe")
    _check(lib.cb_moe_scatter(_ptr(rows), _ptr(sorted_pair), _ptr(weight), _ptr(pair_out),
                              _c_int(rows.shape[0]), _c_int(rows.shape[1]), _stream()), "moe scatter")


def grouped_linear(rows_sorted, w, out, plan, n_experts: int, tiles: int, gated: bool, pair=None) -> bool:
    """The experts' products over their rows side by side, on the tensor cores, by the plan on
    the device (tiles of `GROUPED_TILE_ROWS` rows): out[i] = rows_sorted[i] . W[expert of row i]^T
    with w [experts, N, K]; gated: w [experts, 2 F, K] and out [pairs, F] = the gated pair of
    the two halves (`pair`: the capped form).  False: the sizes do not allow it."""
    from . import tensor_core
    return tensor_core.grouped_linear(rows_sorted, w, out, plan, n_experts, tiles, gated, pair)
