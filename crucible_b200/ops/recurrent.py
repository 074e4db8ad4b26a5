"""Wrappers of `csrc/recurrent.cu`: mixers that carry a matrix per head from token to
token in the request's state slot (the gated delta rule, the mLSTM, the wkv rule, the
state-space rule)."""
from __future__ import annotations

import ctypes

import torch

from . import KernelError, _c_float, _c_int, _check, _code, _need_cuda, _ptr, _stream, build

_c_long = ctypes.c_long
DELTA, MLSTM, WKV, SSD = 0, 1, 2, 3
GATE_SILU, GATE_SIGMOID = 0, 1


def _state_args(state: torch.Tensor):
    if state.dtype != torch.uint8 or state.dim() != 2 or state.stride(1) != 1:
        raise KernelError("a mixer's state is a uint8 view [slots, bytes]")
    if state.data_ptr() % 16:
        raise KernelError("a mixer's state must start on a 16-byte boundary")
    return _ptr(state), _c_long(state.stride(0))


def delta_prepare(proj, conv_w, taps, gates, a_log, dt_bias, ctx, state, tail_off, qkv, beta,
                  decay, n_heads, n_kv_heads, key_dim, value_dim) -> None:
    _need_cuda(proj, conv_w, gates, a_log, dt_bias, state, qkv, beta, decay)
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_delta_prepare(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(conv_w), _c_int(taps),
        _ptr(gates), _c_int(gates.stride(0)), _ptr(a_log), _ptr(dt_bias), _ptr(ctx.row_request), _ptr(ctx.req_row_start),
        _ptr(ctx.req_state_slot), sp, stride, _c_long(tail_off), _ptr(qkv), _ptr(beta), _ptr(decay),
        _c_int(proj.shape[0]), _c_int(n_heads), _c_int(n_kv_heads), _c_int(key_dim),
        _c_int(value_dim), _stream()), "delta_prepare")


def conv_tail_update(proj, taps, channels, ctx, state, tail_off) -> None:
    _need_cuda(proj, state)
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_conv_tail_update(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _c_int(taps), _c_int(channels),
        _ptr(ctx.req_row_start), _ptr(ctx.req_state_slot), sp, stride, _c_long(tail_off),
        _c_int(ctx.n_requests), _stream()), "conv_tail_update")


def mlstm_prepare(proj, gates, bias_i, bias_f, cap, qkv, log_keep, log_in, n_heads, key_dim,
                  value_dim) -> None:
    _need_cuda(proj, gates, bias_i, bias_f, qkv, log_keep, log_in)
    lib = build.load("recurrent")
    _check(lib.cb_mlstm_prepare(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(gates), _c_int(gates.stride(0)), _ptr(bias_i),
        _ptr(bias_f), _c_float(cap), _ptr(qkv), _ptr(log_keep), _ptr(log_in), _c_int(proj.shape[0]),
        _c_int(n_heads), _c_int(key_dim), _c_int(value_dim), _stream()), "mlstm_prepare")


def retention_prepare(proj, freq, rotary_dim: int, split_halves: bool, ctx, head_decay, k_scale: float,
                      qkv, keep, step, n_heads: int, key_dim: int, value_dim: int) -> None:
    """Rows of `proj` are [q: H*D | k: H*D | v: H*E | ...]: the first `rotary_dim` features of
    every q and k head turn by position * freq (float32), k times `k_scale` afterwards; qkv =
    float32 [q | k | v]; keep[t, h] = head_decay[h], step[t, h] = 1 (what the state-space rule
    of `matrix_memory` reads for S <- decay S + k v^T)."""
    _need_cuda(proj, freq, head_decay, qkv, keep, step)
    if (proj.stride(1) != 1 or qkv.dtype != torch.float32 or not qkv.is_contiguous()
            or qkv.shape[1] != n_heads * (2 * key_dim + value_dim)
            or head_decay.dtype != torch.float32 or head_decay.numel() != n_heads
            or keep.dtype != torch.float32 or step.dtype != torch.float32
            or not keep.is_contiguous() or not step.is_contiguous()):
        raise KernelError("retention_prepare: contiguous rows, float32 outputs [rows, H (2D + E)] and "
                          "[rows, H], one float32 decay per head")
    if rotary_dim and (freq is None or freq.dtype != torch.float32 or freq.numel() * 2 != rotary_dim):
        raise KernelError("retention_prepare: freq is float32 [rotary_dim / 2]")
    lib = build.load("recurrent")
    _check(lib.cb_retention_prepare(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(freq), _c_int(rotary_dim),
        _c_int(1 if split_halves else 0), _ptr(ctx.positions), _ptr(head_decay), _c_float(k_scale),
        _ptr(qkv), _ptr(keep), _ptr(step), _c_int(proj.shape[0]), _c_int(n_heads), _c_int(key_dim),
        _c_int(value_dim), _stream()), "retention_prepare")


def matrix_memory(rule, qkv, q_off, k_off, v_off, sc0, sc1, ctx, state, s_off, n_off, m_off, out,
                  n_heads, n_qk_heads, key_dim, value_dim, w_off=0, per_head=None) -> None:
    """Walks every request's tokens in order through its heads' matrices (see the kernel).
    `w_off`: where the wkv rule's decay vectors lie in the rows of `qkv`; `per_head`: float32
    constants, the wkv rule's bonus [heads, key_dim] or the state-space rule's skip [heads]."""
    _need_cuda(qkv, sc0, sc1, state, out, per_head)
    if per_head is not None and (per_head.dtype != torch.float32 or not per_head.is_contiguous()):
        raise KernelError("matrix_memory: the per-head constants are contiguous float32")
    if qkv.dtype != torch.float32 or out.dtype != torch.float32 or not qkv.is_contiguous():
        raise KernelError("matrix_memory takes prepared float32 rows")
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_matrix_memory(
        _c_int(rule), _ptr(qkv), _c_int(qkv.shape[1]), _c_int(q_off), _c_int(k_off), _c_int(v_off),
        _ptr(sc0), _ptr(sc1), _ptr(ctx.req_row_start), _ptr(ctx.req_state_slot), sp, stride,
        _c_long(s_off), _c_long(n_off), _c_long(m_off), _ptr(out), _c_int(ctx.n_requests),
        _c_int(n_heads), _c_int(n_qk_heads), _c_int(key_dim), _c_int(value_dim), _c_int(w_off),
        _ptr(per_head), _stream()), "matrix_memory")


def head_norm_gate(o, gain, gain_per_head, gate, out, gate_kind, n_heads, value_dim, eps,
                   out_scale) -> None:
    """out = o / rms(o over a head) * gain * act(gate) * out_scale; `gate` and `out` are
    views of rows in the engine dtype.  `gain` None: a norm without a weight."""
    _need_cuda(o, gain, gate, out)
    if o.dtype != torch.float32 or gate.dtype != out.dtype or gate.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_norm_gate: float32 input, gate and output rows of one dtype")
    lib = build.load("recurrent")
    _check(lib.cb_head_norm_gate(
        _ptr(o), _ptr(gain), _c_int(value_dim if gain_per_head else 0), _ptr(gate),
        _c_int(gate.stride(0)), _ptr(out), _c_int(out.stride(0)), _c_int(_code(out.dtype)),
        _c_int(gate_kind), _c_int(o.shape[0]), _c_int(n_heads), _c_int(value_dim), _c_float(eps),
        _c_float(out_scale), _stream()), "head_norm_gate")


def shift_mix(h, mu, ctx, state, prev_off, out) -> None:
    """out[s, t] = h[t] + (h[t-1] - h[t]) * mu[s]; the row before a portion's first row is the
    request's state (float32 [width] at `prev_off`), which then becomes the portion's last row."""
    _need_cuda(h, mu, state, out)
    if (mu.dtype != torch.float32 or not mu.is_contiguous() or h.stride(1) != 1 or out.dtype != h.dtype
            or not out.is_contiguous() or tuple(out.shape) != (mu.shape[0], h.shape[0], h.shape[1])):
        raise KernelError("shift_mix: float32 mixes [n, width], rows of one dtype, output [n, rows, width]")
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_shift_mix(
        _ptr(h), _c_int(h.stride(0)), _c_int(_code(h.dtype)), _ptr(mu), _c_int(mu.shape[0]),
        _ptr(ctx.row_request), _ptr(ctx.req_row_start), _ptr(ctx.req_state_slot), sp, stride,
        _c_long(prev_off), _ptr(out), _c_int(h.shape[0]), _c_int(h.shape[1]), _stream()), "shift_mix")


def wkv_prepare(rkv, logit, w0, qkv, n_channels) -> None:
    """`rkv`: [>= 3, rows, channels] (r, k, v); qkv = float32 [r | k | v | exp(-exp(logit + w0))],
    each of `n_channels` columns."""
    _need_cuda(rkv, logit, w0, qkv)
    if (logit.dtype != torch.float32 or qkv.dtype != torch.float32 or not logit.is_contiguous()
            or not qkv.is_contiguous() or rkv.dim() != 3 or rkv.shape[0] < 3 or not rkv.is_contiguous()
            or rkv.shape[2] != n_channels or qkv.shape[1] != 4 * n_channels):
        raise KernelError("wkv_prepare: planes [3, rows, channels], float32 logits and output "
                          "[rows, 4 * channels]")
    lib = build.load("recurrent")
    _check(lib.cb_wkv_prepare(_ptr(rkv), _c_long(rkv.stride(0)), _c_int(_code(rkv.dtype)), _ptr(logit),
                              _ptr(w0), _ptr(qkv), _c_int(rkv.shape[1]), _c_int(n_channels), _stream()),
           "wkv_prepare")


def ssd_prepare(proj, conv_at, conv_w, conv_b, taps, gates, a_log, dt_bias, ctx, state, tail_off, xbc,
                decay, step, n_heads, channels) -> None:
    """Causal convolution with bias + SiLU over `channels` columns of `proj` from `conv_at`
    on; step size softplus(gate + dt_bias) and decay exp(-exp(A_log) * step) per head."""
    _need_cuda(proj, conv_w, conv_b, gates, a_log, dt_bias, state, xbc, decay, step)
    if proj.stride(1) != 1 or gates.dtype != torch.float32 or xbc.dtype != torch.float32:
        raise KernelError("ssd_prepare: contiguous rows, float32 gates and output")
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_ssd_prepare(
        _ptr(proj), _c_int(proj.stride(0)), _c_int(conv_at), _c_int(_code(proj.dtype)), _ptr(conv_w),
        _ptr(conv_b), _c_int(taps), _ptr(gates), _c_int(gates.stride(0)), _ptr(a_log), _ptr(dt_bias),
        _ptr(ctx.row_request), _ptr(ctx.req_row_start), _ptr(ctx.req_state_slot), sp, stride,
        _c_long(tail_off), _ptr(xbc), _ptr(decay), _ptr(step), _c_int(proj.shape[0]), _c_int(n_heads),
        _c_int(channels), _stream()), "ssd_prepare")


def gate_group_norm(y, gate, gain, out, parts, eps) -> None:
    """out = unit-rms, in `parts` equal parts of a row, of y * silu(gate), times gain."""
    _need_cuda(y, gate, gain, out)
    if (y.dtype != torch.float32 or not y.is_contiguous() or gate.dtype != out.dtype
            or gate.stride(1) != 1 or out.stride(1) != 1 or y.shape[1] % parts):
        raise KernelError("gate_group_norm: float32 input, gate and output rows of one dtype, "
                          "a width that the parts divide")
    lib = build.load("recurrent")
    _check(lib.cb_gate_group_norm(_ptr(y), _ptr(gate), _c_int(gate.stride(0)), _ptr(gain), _ptr(out),
                                  _c_int(out.stride(0)), _c_int(_code(out.dtype)), _c_int(y.shape[0]),
                                  _c_int(y.shape[1]), _c_int(parts), _c_float(eps), _stream()),
           "gate_group_norm")
