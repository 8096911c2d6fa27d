"""Wrappers of `csrc/recurrent.cu`: mixers that carry a matrix per head from token to
token in the request's state slot (the gated delta rule, the mLSTM)."""
from __future__ import annotations

import ctypes

import torch

from . import KernelError, _c_float, _c_int, _check, _code, _need_cuda, _ptr, _stream, build

_c_long = ctypes.c_long
DELTA, MLSTM = 0, 1
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


def matrix_memory(rule, qkv, q_off, k_off, v_off, sc0, sc1, ctx, state, s_off, n_off, m_off, out,
                  n_heads, n_qk_heads, key_dim, value_dim) -> None:
    """Walks every request's tokens in order through its heads' matrices (see the kernel)."""
    _need_cuda(qkv, sc0, sc1, state, out)
    if qkv.dtype != torch.float32 or out.dtype != torch.float32 or not qkv.is_contiguous():
        raise KernelError("matrix_memory takes prepared float32 rows")
    sp, stride = _state_args(state)
    lib = build.load("recurrent")
    _check(lib.cb_matrix_memory(
        _c_int(rule), _ptr(qkv), _c_int(qkv.shape[1]), _c_int(q_off), _c_int(k_off), _c_int(v_off),
        _ptr(sc0), _ptr(sc1), _ptr(ctx.req_row_start), _ptr(ctx.req_state_slot), sp, stride,
        _c_long(s_off), _c_long(n_off), _c_long(m_off), _ptr(out), _c_int(ctx.n_requests),
        _c_int(n_heads), _c_int(n_qk_heads), _c_int(key_dim), _c_int(value_dim), _stream()),
        "matrix_memory")


def head_norm_gate(o, gain, gain_per_head, gate, out, gate_kind, n_heads, value_dim, eps,
                   out_scale) -> None:
    """out = o / rms(o over a head) * gain * act(gate) * out_scale; `gate` and `out` are
    views of rows in the engine dtype."""
    _need_cuda(o, gain, gate, out)
    if o.dtype != torch.float32 or gate.dtype != out.dtype or gate.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_norm_gate: float32 input, gate and output rows of one dtype")
    lib = build.load("recurrent")
    _check(lib.cb_head_norm_gate(
        _ptr(o), _ptr(gain), _c_int(value_dim if gain_per_head else 0), _ptr(gate),
        _c_int(gate.stride(0)), _ptr(out), _c_int(out.stride(0)), _c_int(_code(out.dtype)),
        _c_int(gate_kind), _c_int(o.shape[0]), _c_int(n_heads), _c_int(value_dim), _c_float(eps),
        _c_float(out_scale), _stream()), "head_norm_gate")
