"""The plain C++ references of the kernels (csrc/plain_reference.cu), callable with host tensors.

Every function takes and returns float32 tensors on the host and runs the loop nest of the same name in
C++; the tests compare each kernel with it.  Nothing on the product path calls these.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library


def _f32(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.detach().to("cpu", torch.float32).contiguous()


def _i32(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.detach().to("cpu", torch.int32).contiguous()


def _p(tensor: Optional[torch.Tensor]):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def _library():
    return load_library("plain_reference")


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    ids, table = _i32(ids), _f32(table)
    out = torch.zeros(ids.numel(), table.shape[1])
    bad = _library().pr_embedding(_p(ids), _p(table), ids.numel(), table.shape[1], table.shape[0], _p(out))
    if bad:
        raise IndexError(f"{bad} token ids lie outside the table of {table.shape[0]} rows")
    return out


def add_rms_norm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """Returns (residual + delta, its norm)."""
    residual, weight = _f32(residual), _f32(weight)
    delta = None if delta is None else _f32(delta)
    rows, width = residual.shape
    summed, out = torch.empty_like(residual), torch.empty_like(residual)
    _library().pr_add_rms_norm(_p(residual), _p(delta), _p(weight), ctypes.c_float(eps), rows, width, _p(summed), _p(out))
    return summed, out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    x, weight = _f32(x), _f32(weight)
    bias = None if bias is None else _f32(bias)
    out = torch.empty(x.shape[0], weight.shape[0])
    _library().pr_linear(_p(x), _p(weight), _p(bias), x.shape[0], weight.shape[0], x.shape[1], _p(out))
    return out


def gated_mul(gate_up: torch.Tensor, activation: str = "silu") -> torch.Tensor:
    gate_up = _f32(gate_up)
    rows, inner = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty(rows, inner)
    _library().pr_gated_mul(_p(gate_up), rows, inner, {"silu": 0, "gelu_tanh": 1}[activation], _p(out))
    return out


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: Optional[int] = None,
         interleaved: bool = False) -> torch.Tensor:
    """x [rows, heads, head_dim]; returns the rotated copy."""
    out, positions, inv_freq = _f32(x).clone(), _i32(positions), _f32(inv_freq)
    rows, heads, head_dim = out.shape
    _library().pr_rope(_p(out), _p(positions), _p(inv_freq), rows, heads, head_dim,
                       head_dim if rotary_dim is None else rotary_dim, int(interleaved))
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None,
              first_position: int = 0) -> torch.Tensor:
    """q [rows, n_q, d] at positions first_position..; k, v [first_position + rows, n_kv, d]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    rows, n_q, d = q.shape
    out = torch.empty_like(q)
    scratch = torch.empty(first_position + rows, dtype=torch.float64)
    _library().pr_attention(_p(q), _p(k), _p(v), rows, first_position, n_q, k.shape[1], d, ctypes.c_float(scale),
                            int(window or 0), _p(out), _p(scratch))
    return out


def argmax(logits: torch.Tensor) -> int:
    logits = _f32(logits)
    return _library().pr_argmax(_p(logits), logits.numel())


def sample(logits: torch.Tensor, temperature: float, u: float) -> int:
    logits = _f32(logits)
    return _library().pr_sample(_p(logits), logits.numel(), ctypes.c_float(temperature), ctypes.c_float(u))
