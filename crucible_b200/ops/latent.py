"""Wrappers of `csrc/latent_attention.cu`: what surrounds the attention over a cached
latent (the latent's norm, the rotations, the write into the pages, the heads' gates)."""
from __future__ import annotations

import torch

from . import KernelError, _c_float, _c_int, _check, _code, _need_cuda, _ptr, _stream, build


def prepare(dkv, q, qx, gain, freq, mscale: float, eps: float, n_heads: int, dim: int, rank: int,
            rot: int, turned: int, ctx, cache, binding, split_halves: bool = True) -> None:
    """Rows of `dkv` are [latent: rank | shared key part: rot], rows of `q` [heads, dim + rot].
    Writes [rmsnorm(latent) * gain | rotated key part] to the token's place in the pages and the
    last `rot` features of every head of q, rotated, into the last `rot` of that head in `qx`
    [heads, rank + rot].  Of the `rot` features the first `turned` turn (`split_halves`: feature
    i with i + turned / 2, else neighbours), the rest pass unchanged.  `q` and `qx` None: the
    pages' part alone; `dkv` None (a binding that does not write): the queries' part alone."""
    _need_cuda(dkv, q, qx, gain, freq)
    rows = [t for t in (dkv, q, qx) if t is not None]
    if any(t.stride(1) != 1 or t.dtype != rows[0].dtype for t in rows) or (q is None) != (qx is None):
        raise KernelError("latent prepare: contiguous rows of one dtype")
    if (dkv is None and binding.write) or (q is None and not binding.write):
        raise KernelError("latent prepare: a writing layer brings its rows, a reading one its queries")
    if turned and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != turned):
        raise KernelError("latent prepare: freq is float32 [turned / 2]")
    pages = cache.keys(binding.slot)
    if pages.dtype != rows[0].dtype or pages.shape[-1] != rank + rot or cache.kv_heads != 1:
        raise KernelError("latent prepare: the pages hold one row of rank + rot features per token "
                          "in the activations' dtype")
    table = ctx.block_table(binding.group)
    lib = build.load("latent_attention")
    _check(lib.cb_latent_prepare(
        _ptr(dkv), _c_int(dkv.stride(0) if dkv is not None else 0), _ptr(q),
        _c_int(q.stride(0) if q is not None else 0), _ptr(qx), _c_int(qx.stride(0) if qx is not None else 0),
        _c_int(_code(rows[0].dtype)), _ptr(gain), _ptr(freq), _c_float(mscale), _c_float(eps),
        _ptr(ctx.positions), _ptr(ctx.row_request), _ptr(table), _c_int(table.shape[1]), _ptr(pages),
        _c_int(rows[0].shape[0]), _c_int(n_heads), _c_int(dim), _c_int(rank), _c_int(rot), _c_int(turned),
        _c_int(cache.page_tokens), _c_int(1 if binding.write else 0), _c_int(1 if split_halves else 0),
        _stream()), "latent_prepare")


def head_gate(x, logit, n_heads: int, head_width: int) -> None:
    """x[t, h, :] *= sigmoid(logit[t, h]) in place; `logit` [rows, heads] in float32 or in the
    rows' own dtype (columns of a joint projection)."""
    _need_cuda(x, logit)
    if (logit.dtype not in (torch.float32, x.dtype) or logit.stride(1) != 1 or x.stride(1) != 1
            or x.shape[1] != n_heads * head_width or logit.shape[1] != n_heads):
        raise KernelError("head_gate: rows [T, heads * width] and logits [T, heads], float32 or the rows' dtype")
    lib = build.load("latent_attention")
    _check(lib.cb_head_gate(_ptr(x), _c_int(x.stride(0)), _c_int(_code(x.dtype)), _ptr(logit),
                            _c_int(_code(logit.dtype)), _c_int(logit.stride(0)), _c_int(x.shape[0]),
                            _c_int(n_heads), _c_int(head_width), _stream()), "head_gate")


def rows_gate(x, g) -> None:
    """x[t, i] *= sigmoid(g[t, i]) in place: a gate with a logit of its own for every feature."""
    _need_cuda(x, g)
    if x.shape != g.shape or x.dtype != g.dtype or x.stride(1) != 1 or g.stride(1) != 1:
        raise KernelError("rows_gate: rows and logits of one shape and dtype")
    lib = build.load("latent_attention")
    _check(lib.cb_rows_gate(_ptr(x), _c_int(x.stride(0)), _ptr(g), _c_int(g.stride(0)), _c_int(_code(x.dtype)),
                            _c_int(x.shape[0]), _c_int(x.shape[1]), _stream()), "rows_gate")


SMALL_ROWS = 16      # steps of up to this many rows take the heads' products in one launch
HEADS_IN_ONE_LAUNCH = True   # many bfloat16 rows: the heads as the third axis of one tensor-core launch
                             # (tests switch it off to reach the product per head with the same inputs)


def heads_linear(a, a_head: int, w, out, out_head: int, gate_logit=None, gate_rows=None) -> None:
    """out[t, h * out_head + n] = sum_k a[t, h * a_head + k] * w[h, n, k] for every head h of
    `w` [heads, N, K].  Steps of a few bfloat16 rows run as one launch whose warps each read one
    weight row once; many bfloat16 rows as one launch of tensor-core tiles with the head as the
    grid's third axis; otherwise one product per head through `ops.linear` (in float32 always, so
    that a row's sums never depend on the step).
    `gate_logit` (float32 [rows, heads]): every head's results times sigmoid(logit), in the same
    launch for few rows, by `head_gate` otherwise.  `gate_rows` (rows of the activations' dtype,
    [rows, heads * N]): every result times the sigmoid of its own logit, likewise."""
    from . import linear
    heads, n, k = w.shape
    if gate_rows is not None and (out_head != n or gate_rows.shape != (a.shape[0], heads * n)
                                  or gate_rows.dtype != out.dtype or gate_rows.stride(1) != 1):
        raise KernelError("heads_linear: gate rows are [rows, heads * N] of the results' dtype")
    if a.dtype == torch.bfloat16 and a.shape[0] <= SMALL_ROWS:
        _need_cuda(a, w, out, gate_rows)
        if a.stride(1) != 1 or out.stride(1) != 1 or not w.is_contiguous() or out.dtype != a.dtype:
            raise KernelError("heads_linear: contiguous rows of one dtype and contiguous weights")
        lib = build.load("latent_attention")
        _check(lib.cb_heads_linear_small(_ptr(a), _c_int(a.stride(0)), _c_int(a_head), _ptr(w), _ptr(out),
                                         _c_int(out.stride(0)), _c_int(out_head), _c_int(_code(a.dtype)),
                                         _c_int(a.shape[0]), _c_int(heads), _c_int(n), _c_int(k),
                                         _ptr(gate_logit),
                                         _c_int(gate_logit.stride(0) if gate_logit is not None else 0),
                                         _ptr(gate_rows),
                                         _c_int(gate_rows.stride(0) if gate_rows is not None else 0),
                                         _stream()),
               "heads_linear (few rows)")
        return
    from . import is_weight, tensor_core
    if not (HEADS_IN_ONE_LAUNCH and a.dtype == torch.bfloat16 and is_weight(w)
            and tensor_core.heads_linear(a, a_head, w, out, out_head)):
        for i in range(heads):
            linear(a[:, i * a_head:i * a_head + k], w[i], out[:, i * out_head:i * out_head + n])
    if gate_logit is not None:
        if out.shape[1] != heads * out_head:
            raise KernelError("heads_linear: a gate needs the heads' results side by side")
        head_gate(out, gate_logit, heads, out_head)
    if gate_rows is not None:
        rows_gate(out[:, :heads * n] if out.shape[1] != heads * n else out, gate_rows)
