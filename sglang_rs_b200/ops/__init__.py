"""Python face of the CUDA kernels.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity), launches on torch's current stream and raises :class:`KernelError` with the
library's message if the kernel refuses the sizes.  Nothing here computes on the host
and nothing falls back to another implementation.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library
from . import records, trace
from .trace import traced

F32, BF16 = 0, 1

# Products of more than a few rows go to cuBLAS (``library_product``), on a handle whose math mode forbids
# partial sums of a split along K in bfloat16: every product of this engine accumulates in 32 bits to the
# end.  The same is asked of torch's own handle, for callers that mix torch's products with this package.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(tensor: Optional[torch.Tensor]):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


_scoped_stream = None


def _stream():
    if _scoped_stream is not None:
        return _scoped_stream
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks up torch's current stream once for all kernel launches inside the ``with`` block
    (the look-up costs as much as a small launch).  The current stream must not change inside."""

    def __enter__(self):
        global _scoped_stream
        self._previous = _scoped_stream
        _scoped_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._previous
        return False


def _need(tensor: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor; this engine has no host path")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {tensor.dtype}")


#: kernels of this package launched so far (the bench reports the count of a timed region)
launch_count = 0


def _check(library, status: int, launches: int = 1) -> None:
    global launch_count
    launch_count += launches
    if status != 0:
        raise KernelError(library.srb_last_error().decode("utf-8", "replace") or f"kernel status {status}")


#: the compute capability the kernels are compiled for (sm_100a: tcgen05, tensor memory, TMA)
REQUIRED_CAPABILITY = (10, 0)
_sm_counts: dict = {}


def require_supported_device(device) -> None:
    """Fails at start-up, with the device's name, on a GPU that the kernels are not built for (the
    reference decides the same from the SM version, crates/sglang-srt/src/backend.rs:355-366); without
    this check the first tcgen05 launch would fail with a bare CUDA error."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is visible; this engine has no host path")
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    capability = torch.cuda.get_device_capability(index)
    if tuple(capability) != REQUIRED_CAPABILITY:
        raise KernelError(
            f"device cuda:{index} ({torch.cuda.get_device_name(index)}) has compute capability "
            f"{capability[0]}.{capability[1]}; the kernels of this engine are built for sm_100a "
            f"({REQUIRED_CAPABILITY[0]}.{REQUIRED_CAPABILITY[1]}, B200) only")


def sm_count(device=None) -> int:
    """SMs of ``device`` (default: the current one), asked once."""
    index = torch.cuda.current_device() if device is None or torch.device(device).index is None \
        else torch.device(device).index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return count


def new_error_word(device) -> torch.Tensor:
    """Device-side word that kernels OR fault bits into (bad token, slot or page)."""
    return torch.zeros(1, dtype=torch.int32, device=device)


ERROR_BITS = {1: "token id outside the vocabulary", 2: "cache slot outside the pool",
              4: "page id outside the pool", 8: "a device-side wait ran out",
              16: "a row of a split attention run has more key splits than the launch was given"}


def raise_on_error_word(word: torch.Tensor) -> None:
    raise_on_error_value(int(word.item()), word)


def raise_on_error_value(value: int, word: torch.Tensor) -> None:
    """``value``: what ``word`` held when it was last copied to the host."""
    if value:
        word.zero_()
        what = [text for bit, text in ERROR_BITS.items() if value & bit]
        raise KernelError("device-side check failed: " + "; ".join(what))


# --------------------------------------------------------------------------- rows

@traced("embedding")
def embedding(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, error_word: torch.Tensor) -> None:
    """residual[r, :] = float(table[ids[r], :])"""
    _need(ids, "ids", torch.int32); _need(table, "table"); _need(residual, "residual", torch.float32)
    rows, width = residual.shape
    if ids.numel() != rows or table.shape[1] != width:
        raise KernelError("embedding: shapes of ids, table and residual do not agree")
    lib = load_library("elementwise")
    _check(lib, lib.srb_embedding(_ptr(ids), _ptr(table), _ptr(residual), rows, width, table.shape[0],
                                  _ptr(error_word), dtype_code(table.dtype), _stream()))


@traced("embedding")
def take_tokens(tokens: torch.Tensor, source: torch.Tensor, index: torch.Tensor, error_word: torch.Tensor) -> None:
    """tokens[i] = source[index[i]] where index[i] >= 0 (int32, on the device): the token ids that the
    step before chose and that have not been to the host yet."""
    _need(tokens, "tokens", torch.int32); _need(source, "source", torch.int32); _need(index, "index", torch.int32)
    if index.numel() < tokens.numel():
        raise KernelError("take_tokens: one index per token is needed")
    lib = load_library("elementwise")
    _check(lib, lib.srb_take_tokens(_ptr(tokens), _ptr(source), _ptr(index), tokens.numel(), source.numel(),
                                    _ptr(error_word), _stream()))


@traced("norm")
def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, row_index: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """x = residual (+ delta); residual = x if asked; out = x / sqrt(mean(x^2) + eps) * weight.

    ``delta`` is [rows, width] of ``out``'s dtype, or float32 [parts, rows, width]: partial sums
    of a product cut along K, added in order.  With ``row_index`` the rows ``row_index[i]`` are
    read and ``out[i]`` is written."""
    _need(residual, "residual", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    width = residual.shape[1]
    rows = out.shape[0]
    whole = parts = None
    num_parts = part_stride = 0
    if delta is not None and delta.dim() == 3:
        _need(delta, "delta", torch.float32)
        if delta.shape[1:] != residual.shape:
            raise KernelError("add_rmsnorm: partial sums and residual differ in shape")
        parts, num_parts, part_stride = delta, delta.shape[0], delta.stride(0)
    elif delta is not None:
        _need(delta, "delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("add_rmsnorm: delta and residual differ in shape")
        whole = delta
    if row_index is not None:
        _need(row_index, "row_index", torch.int32)
        if row_index.numel() != rows:
            raise KernelError("add_rmsnorm: one output row per index is needed")
    elif rows != residual.shape[0]:
        raise KernelError("add_rmsnorm: out and residual differ in rows")
    if weight.numel() != width or out.shape[1] != width:
        raise KernelError("add_rmsnorm: widths do not agree")
    lib = load_library("elementwise")
    _check(lib, lib.srb_add_rmsnorm(_ptr(residual), _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride),
                                    _ptr(weight), _ptr(out), _ptr(row_index), rows, width, ctypes.c_float(eps),
                                    int(write_residual), dtype_code(out.dtype), _stream()))


#: activations of a gated feed-forward, act(gate) * up, by the numbers of csrc/activations.cuh
ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def activation_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"unknown activation {name!r}; the kernels have {sorted(ACTIVATIONS)}") from None


@traced("activation")
def gated_mul(gate_up: torch.Tensor, out: torch.Tensor, activation: str = "silu") -> None:
    """out[r, j] = act(gate_up[r, j]) * gate_up[r, inner + j]"""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    rows, inner = out.shape
    if gate_up.shape != (rows, 2 * inner):
        raise KernelError("gated_mul: gate_up must be [rows, 2 * inner]")
    lib = load_library("elementwise")
    _check(lib, lib.srb_gated_mul(_ptr(gate_up), _ptr(out), rows, inner, activation_code(activation),
                                  dtype_code(out.dtype), _stream()))


@traced("bias")
def add_bias(values: torch.Tensor, bias: torch.Tensor) -> None:
    _need(values, "values"); _need(bias, "bias", torch.float32)
    rows, width = values.shape
    if bias.numel() != width:
        raise KernelError("add_bias: bias width differs")
    lib = load_library("elementwise")
    _check(lib, lib.srb_add_bias(_ptr(values), _ptr(bias), rows, width, dtype_code(values.dtype), _stream()))


# --------------------------------------------------------------------------- attention

@traced("rope_kv")
def qk_norm_rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                    v_pool: Optional[torch.Tensor], positions: torch.Tensor, slots: Optional[torch.Tensor],
                    q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], eps: float,
                    inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, n_q: int, n_kv: int,
                    head_dim: int, error_word: torch.Tensor, angles: Optional[torch.Tensor] = None,
                    cos_sin: Optional[torch.Tensor] = None) -> None:
    """Per-head norm of q and k, rotation of q and k, q to ``q_out``, k and v into the pages.

    ``qkv`` is [rows, >= (n_q + 2 n_kv) head_dim] with q heads, k heads, v heads in that order,
    of ``q_out``'s dtype, or float32 [parts, rows, width] partial sums that are added in order;
    pools are [pages, n_kv, page_size, head_dim]; ``slots[r]`` = page * page_size + offset.
    With ``slots`` None nothing is written to the pages.  The rotation takes its angles as
    ``positions[r] * inv_freq[i]`` or, if ``angles`` (float32 [rows, rotary_dim / 2]) is given,
    from there.  ``cos_sin``: the table of :func:`rope_table` for these rows; the kernel for many rows
    then reads the cosines and sines instead of computing them (the same values)."""
    _need(qkv, "qkv"); _need(q_out, "q_out"); _need(positions, "positions", torch.int32)
    if angles is not None:
        _need(angles, "angles", torch.float32)
        if angles.shape != (qkv.shape[-2], rotary_dim // 2):
            raise KernelError("qk_norm_rope_kv: angles must be [rows, rotary_dim / 2]")
    whole = parts = None
    num_parts = part_stride = 0
    if qkv.dim() == 3:
        _need(qkv, "qkv", torch.float32)
        parts, num_parts, part_stride = qkv, qkv.shape[0], qkv.stride(0)
    else:
        _need(qkv, "qkv", q_out.dtype)
        whole = qkv
    rows = qkv.shape[-2]
    page_size = num_pages = 1
    if slots is not None:
        _need(slots, "slots", torch.int32); _need(k_pool, "k_pool", q_out.dtype); _need(v_pool, "v_pool", q_out.dtype)
        num_pages, pool_heads, page_size, pool_dim = k_pool.shape
        if (pool_heads, pool_dim) != (n_kv, head_dim) or v_pool.shape != k_pool.shape:
            raise KernelError("qk_norm_rope_kv: pools must be [pages, n_kv, page_size, head_dim]")
        if qkv.shape[-1] < (n_q + 2 * n_kv) * head_dim:
            raise KernelError("qk_norm_rope_kv: qkv is narrower than q, k and v together")
    for name, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None:
            _need(w, name, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_kv: {name} must have head_dim elements")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise KernelError("qk_norm_rope_kv: inv_freq must have rotary_dim / 2 elements")
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape != (rows, rotary_dim):
            raise KernelError("qk_norm_rope_kv: cos_sin must be [rows, rotary_dim]")
    lib = load_library("rope_kv")
    _check(lib, lib.srb_qk_norm_rope_kv_table(
        _ptr(whole), _ptr(parts), num_parts, ctypes.c_longlong(part_stride), qkv.stride(-2), _ptr(q_out), _ptr(k_pool),
        _ptr(v_pool), _ptr(positions), _ptr(slots), _ptr(q_norm), _ptr(k_norm), ctypes.c_float(eps), _ptr(inv_freq),
        _ptr(angles), _ptr(cos_sin), rotary_dim, int(interleaved), rows, n_q, n_kv, head_dim, page_size, num_pages,
        _ptr(error_word), dtype_code(q_out.dtype), _stream()))


@traced("rope_kv")
def rope_table(positions: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int,
               angles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [rows, rotary_dim]: per row the cosines, then the sines, of ``positions[r] * inv_freq[i]`` (or of
    ``angles[r, i]``), computed once for a step; the step executor hands it to the rope kernel of every layer."""
    _need(positions, "positions", torch.int32)
    rows = positions.numel()
    out = torch.empty((rows, rotary_dim), dtype=torch.float32, device=positions.device)
    lib = load_library("rope_kv")
    _check(lib, lib.srb_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(angles), rows, rotary_dim, _ptr(out), _stream()))
    return out


def attention_scratch_sizes(rows: int, n_q: int, head_dim: int, max_splits: int) -> tuple[int, int]:
    """Floats of scratch that a split run needs: (partial accumulators, partial max and sum)."""
    return rows * n_q * max_splits * head_dim, rows * n_q * max_splits * 2


@traced("attention_generic")
def paged_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    positions: torch.Tensor, row_request: torch.Tensor, block_table: torch.Tensor, *,
                    scale: float, window: int, split_size: int, max_splits: int,
                    scratch_acc: Optional[torch.Tensor], scratch_ml: Optional[torch.Tensor],
                    error_word: torch.Tensor) -> None:
    """out[r, h, :] = softmax over the keys row r may see of (q . k) * scale, times v.

    q, out: [rows, n_q, head_dim]; pools [pages, n_kv, page_size, head_dim]; block_table
    [requests, stride].  ``split_size`` 0 walks all keys in one block per (row, kv head);
    otherwise partials go through the scratch tensors and are merged in split order.
    This is the generic kernel (any head_dim that is a multiple of 16, float32 or bfloat16)."""
    _need(q, "q"); _need(out, "out", q.dtype); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype)
    _need(positions, "positions", torch.int32); _need(row_request, "row_request", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape:
        raise KernelError("paged_attention: shapes of q, out and the pools do not agree")
    if split_size:
        need_acc, need_ml = attention_scratch_sizes(rows, n_q, head_dim, max_splits)
        if scratch_acc is None or scratch_ml is None or scratch_acc.numel() < need_acc or scratch_ml.numel() < need_ml:
            raise KernelError("paged_attention: scratch tensors are too small for this split run")
        _need(scratch_acc, "scratch_acc", torch.float32); _need(scratch_ml, "scratch_ml", torch.float32)
    lib = load_library("attention")
    _check(lib, lib.srb_paged_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch_acc), _ptr(scratch_ml), _ptr(positions),
        _ptr(row_request), _ptr(block_table), block_table.stride(0), rows, n_q, n_kv, head_dim, page_size,
        num_pages, int(window), int(split_size), int(max_splits), ctypes.c_float(scale), _ptr(error_word),
        dtype_code(q.dtype), _stream()), launches=2 if split_size else 1)





#: the most blocks per (row, kv head) that :func:`decode_splits` ever returns
DECODE_MAX_SPLITS = 64


def decode_attention_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """True if the tensor-core kernel for decoded tokens takes these sizes (the rule of
    srb_decode_attention_supports, asked here so that other models never compile it)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0 and n_q // n_kv <= 16




def decode_splits(rows: int, n_kv: int, max_keys: Optional[int] = None, sms: Optional[int] = None) -> int:
    """Blocks per (row, kv head).  A function of the shape and of the device's SM count (``sms``;
    default: the current device's) only; defined in csrc/step_exec.cu, where the step executor uses it too.

    Without ``max_keys`` (the most keys any row sees): as many as make about three blocks per SM.
    With it, the count that makes the step shortest under a simple model: the blocks run in waves
    of three per SM, and a wave lasts as long as one block's share of the keys plus a fixed cost.
    Many rows then still get their keys cut (512 blocks are 1.15 waves: nearly half the second
    wave's time is lost), and no block walks fewer than two 64-key units."""
    return records.library().sx_decode_splits(int(rows), int(n_kv), -1 if max_keys is None else int(max_keys),
                                              int(sms if sms is not None else sm_count()))


def decode_splits_bound(max_keys: int) -> int:
    """No call of :func:`decode_splits` with this ``max_keys`` returns more, whatever the rows and heads."""
    return records.library().sx_decode_splits_bound(int(max_keys))


@traced("attention_decode")
def decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                     positions: torch.Tensor, row_request: torch.Tensor, block_table: torch.Tensor, *,
                     scale: float, window: int, scratch_acc: torch.Tensor, scratch_ml: torch.Tensor,
                     counters: torch.Tensor, error_word: torch.Tensor, max_keys: Optional[int] = None) -> None:
    """Attention of decoded tokens (one row each), bfloat16, head_dim 64 or 128.

    The keys of a (row, kv head) are shared by ``decode_splits(rows, n_kv, max_keys)`` blocks
    (``max_keys``: the most keys any row sees, if known); the block that finishes last merges them.  ``counters``: int32, zero, at least rows * n_kv entries; they
    are zero again afterwards.  Scratch: rows * n_q * splits * head_dim and rows * n_q * splits * 2
    floats."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(positions, "positions", torch.int32)
    _need(row_request, "row_request", torch.int32); _need(block_table, "block_table", torch.int32)
    _need(scratch_acc, "scratch_acc", torch.float32); _need(scratch_ml, "scratch_ml", torch.float32)
    _need(counters, "counters", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape:
        raise KernelError("decode_attention: shapes of q, out and the pools do not agree")
    # never more blocks than the scratch memory holds partial results for
    splits = max(1, min(decode_splits(rows, n_kv, max_keys), scratch_acc.numel() // (rows * n_q * head_dim),
                        scratch_ml.numel() // (rows * n_q * 2)))
    if scratch_acc.numel() < rows * n_q * splits * head_dim or scratch_ml.numel() < rows * n_q * splits * 2:
        raise KernelError("decode_attention: scratch tensors are too small")
    if counters.numel() < rows * n_kv:
        raise KernelError("decode_attention: too few counters")
    lib = load_library("attention_decode")
    _check(lib, lib.srb_decode_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(scratch_acc), _ptr(scratch_ml), _ptr(counters),
        _ptr(positions), _ptr(row_request), _ptr(block_table), block_table.stride(0), rows, n_q, n_kv, head_dim,
        page_size, num_pages, int(window), splits, ctypes.c_float(scale), _ptr(error_word), _stream()))


def tiled_attention_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int) -> bool:
    """True if the tensor-core kernel for prompt portions takes these sizes."""
    # the same rule as srb_prefill_attention_supports, asked here so that a model the kernel
    # does not take never compiles it
    return dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0


@traced("attention_prefill")
def tiled_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                    tiles: torch.Tensor, block_table: torch.Tensor, *, scale: float, window: int,
                    error_word: torch.Tensor) -> None:
    """Attention of prompt portions, bfloat16.  ``tiles`` is int32 [n, 4]: first row of the
    step, rows (at most 64, consecutive rows of one request), request index, first position.
    Rows outside the tiles are left untouched."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(tiles, "tiles", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape or tiles.shape[-1] != 4:
        raise KernelError("tiled_attention: shapes of q, out, the pools and the tiles do not agree")
    lib = load_library("attention_prefill")
    _check(lib, lib.srb_prefill_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(tiles), tiles.shape[0], _ptr(block_table),
        block_table.stride(0), n_q, n_kv, head_dim, page_size, num_pages, int(window), ctypes.c_float(scale),
        _ptr(error_word), _stream()))


TC_TILE_ROWS = 128


def tiled_attention_tc_takes(dtype: torch.dtype, n_q: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """True if the tcgen05 kernel for prompt portions takes these sizes (the rule of
    srb_prefill_tc_supports)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_q % n_kv == 0
            and page_size >= 8 and page_size % 8 == 0 and 64 % page_size == 0)


@traced("attention_prefill")
def tiled_attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                       tiles: torch.Tensor, block_table: torch.Tensor, *, scale: float, window: int,
                       error_word: torch.Tensor) -> None:
    """Attention of prompt portions on tcgen05 tensor cores (S, P and O in tensor memory, operands
    by TMA).  ``tiles`` as for :func:`tiled_attention`, with at most 128 rows per tile."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(tiles, "tiles", torch.int32)
    _need(block_table, "block_table", torch.int32)
    rows, n_q, head_dim = q.shape
    num_pages, n_kv, page_size, pool_dim = k_pool.shape
    if pool_dim != head_dim or v_pool.shape != k_pool.shape or out.shape != q.shape or tiles.shape[-1] != 4:
        raise KernelError("tiled_attention_tc: shapes of q, out, the pools and the tiles do not agree")
    lib = load_library("attention_prefill_tc")
    _check(lib, lib.srb_prefill_attention_tc(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(tiles), tiles.shape[0], rows, _ptr(block_table),
        block_table.stride(0), n_q, n_kv, head_dim, page_size, num_pages, int(window), ctypes.c_float(scale),
        _ptr(error_word), _stream()))


# --------------------------------------------------------------------------- matrix products

#: The two thresholds below were measured at Qwen3-8B sizes on a B200; they are tunables (the environment
#: variables SRB_OWN_GEMM_MAX_TOKENS and SRB_PAIR_GEMM_MIN_TOKENS set them), read at every step.
#: up to this many rows a bfloat16 product runs on this package's tcgen05 kernel for few tokens.  With 65 to
#: 128 rows the kernel has one block per SM and no cut along K, and the library is twice as fast
#: (Qwen3-8B sizes on B200, chained in a graph: QKV 12 against 20 us, down 23 against 52 us; a 12-layer
#: decode step at batch 128 takes 3.80 ms instead of 4.48 ms)
OWN_GEMM_MAX_TOKENS = int(os.environ.get("SRB_OWN_GEMM_MAX_TOKENS", "64"))
#: from this many rows on the gate/up product runs on the persistent CTA-pair kernel, which takes SiLU(gate) * up
#: into its epilogue.  Measured at Qwen3-8B sizes on B200, chained in a graph, against the library's product
#: followed by the SiLU kernel: 64.8 against 53.7 us at 256 rows (96 tiles of 256 tokens leave the second
#: round of the 74 pairs mostly empty), 155 against 155 us at 1,024, 214 against 219 us at 1,536, 280 against
#: 301 us at 2,048.  The plain products stay with the library at every size: the pair kernel reaches 0.92 to
#: 1.0 of it alone, and whole prefill steps measured no gain from switching them.
PAIR_GEMM_MIN_TOKENS = int(os.environ.get("SRB_PAIR_GEMM_MIN_TOKENS", "1280"))


def gemm_splits(tokens: int, features: int, k: int, sms: Optional[int] = None) -> int:
    """Into how many partial sums a small-batch product is cut along K.  A function of the
    shape and of the device's SM count only: blocks of 128 weight rows alone cannot occupy the SMs when
    there are few of them, so K is cut until about two blocks per SM exist (two fit), each with at least
    8 K blocks.  Defined in csrc/step_exec.cu, where the step executor uses it too."""
    return records.library().sx_gemm_splits(int(tokens), int(features), int(k), int(sms if sms is not None else sm_count()),
                                            OWN_GEMM_MAX_TOKENS)


@traced("gemm")
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, error_word: Optional[torch.Tensor] = None,
           partial_ok: bool = False) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in], row-major.

    float32: the FFMA kernel of this package, true 32-bit.  bfloat16: up to
    ``OWN_GEMM_MAX_TOKENS`` rows the tcgen05 kernel of this package, above that cuBLAS
    (:func:`library_product`: what the reference's engine calls for every projection,
    crates/sglang-kernel/src/cublas.rs:383-410); both accumulate in 32-bit.  ``out_dtype``
    float32 keeps the accumulator's precision (used for the logits).  With ``partial_ok`` the
    result may be float32 [parts, rows, out]: partial sums over K that the consumer adds in
    order (``add_rmsnorm`` and ``qk_norm_rope_kv`` do)."""
    _need(x, "x"); _need(weight, "weight", x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} and weight {tuple(weight.shape)} do not fit")
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        if bias is not None:
            _need(bias, "bias", torch.float32)
        lib = load_library("gemm_f32")
        _check(lib, lib.srb_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k, x.stride(0),
                                     weight.stride(0), out.stride(0), _stream()))
        return out
    if m <= OWN_GEMM_MAX_TOKENS and error_word is not None and gemm_bf16_takes(k):
        splits = gemm_splits(m, n, k) if partial_ok else 1
        if splits > 1:
            out = gemm_bf16(x, weight, error_word, mode="partial", splits=splits)
            if bias is not None:
                add_bias(out[0], bias)
            return out
        out = gemm_bf16(x, weight, error_word, mode="f32" if out_dtype == torch.float32 else "bf16")
    else:
        out = library_product(x, weight, torch.float32 if out_dtype == torch.float32 else torch.bfloat16)
    if bias is not None:
        add_bias(out, bias)
    return out


def library_product(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """y = x @ weight^T by cuBLAS (``cublasGemmEx``, bfloat16 operands, 32-bit accumulation to the end), the
    call the reference's engine makes for every projection (crates/sglang-kernel/src/cublas.rs:383-410).  The
    same call, through the same handle and scratch memory, takes the products of many rows inside the step
    executor."""
    records.ensure_cublas(x.device)
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    lib = records.library()
    _check(lib, lib.sx_cublas_product(_ptr(x), _ptr(weight), _ptr(out), m, n, k, x.stride(0), weight.stride(0), out.stride(0),
                                      int(out_dtype == torch.float32), _stream()))
    return out


@traced("gemm")
def gated_product(x: torch.Tensor, weight: torch.Tensor, inner: int, error_word: Optional[torch.Tensor] = None,
                  activation: str = "silu") -> torch.Tensor:
    """act(x gate^T) * (x up^T) for ``weight`` = gate rows stacked over up rows [2 inner, in].

    bfloat16 with few rows: one tcgen05 kernel whose epilogue takes the product of its two
    accumulators, so the [rows, 2 inner] intermediate never exists; with many rows the CTA-pair
    kernel does the same.  Otherwise the product (``linear``) followed by the activation kernel."""
    if (x.dtype == torch.bfloat16 and x.shape[0] <= OWN_GEMM_MAX_TOKENS and error_word is not None
            and gemm_bf16_takes(x.shape[1])):
        return gemm_bf16(x, weight, error_word, mode="gated", features=inner, up_row_offset=inner, activation=activation)
    if (x.dtype == torch.bfloat16 and error_word is not None and weight.shape[0] == 2 * inner
            and pair_gemm_takes(x.shape[0], inner, x.shape[1])):
        return gemm_bf16_pair(x, weight, error_word, mode="gated", features=inner, up_row_offset=inner,
                              activation=activation)
    gate_up = linear(x, weight, error_word=error_word)
    act = torch.empty((x.shape[0], inner), dtype=x.dtype, device=x.device)
    gated_mul(gate_up, act, activation)
    return act


GEMM_MODES = {"bf16": 0, "f32": 1, "gated": 2, "partial": 3, "add": 4}
#: the blocks of a thread-block cluster: at most this many K splits add their sums inside the kernel
GEMM_CLUSTER_SPLITS = 8


@traced("gemm")
def gemm_bf16(x: torch.Tensor, w: torch.Tensor, error_word: torch.Tensor, *, mode: str = "bf16",
              features: Optional[int] = None, up_row_offset: int = 0, splits: int = 1,
              out: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """y = x @ w^T on tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    x [tokens, k], w [rows, k], k a multiple of 8.  ``mode``: ``bf16`` / ``f32`` store
    [tokens, features]; ``gated`` treats w as gate rows [0, features) stacked over up rows
    [up_row_offset, up_row_offset + features) and stores act(gate) * up (``activation``: a name of
    ``ACTIVATIONS``); ``partial`` stores
    ``splits`` float partial sums [splits, tokens, features] that the consumer adds in order;
    ``add`` adds the product to ``out`` (float32 [tokens, features], e.g. the residual stream) in
    place, K cut into at most ``GEMM_CLUSTER_SPLITS`` blocks that sum inside the kernel in block order.
    (The engine's decode steps do not use ``add``: measured at Qwen3-8B sizes, partial sums that the
    next norm kernel adds are quicker, 3.22 / 3.48 / 7.21 ms per step at batch 1 / 8 / 64 against
    3.37 / 3.52 / 7.69 ms, because clusters of 8 blocks start later and end with two cluster barriers.)"""
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
    tokens, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_bf16: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    if features is None:
        features = rows
    code = GEMM_MODES[mode]
    pitch = features
    if mode == "partial":
        out = torch.empty((splits, tokens, features), dtype=torch.float32, device=x.device)
    elif mode == "add":
        if out is None or not out.is_cuda or out.dtype != torch.float32 or out.dim() != 2 or out.stride(1) != 1:
            raise KernelError("gemm_bf16: the tensor added to must be a float32 CUDA matrix with dense rows")
        if out.shape[0] != tokens or out.shape[1] != features or not 1 <= splits <= GEMM_CLUSTER_SPLITS:
            raise KernelError("gemm_bf16: the tensor added to must be [tokens, features], the splits at most "
                              f"{GEMM_CLUSTER_SPLITS}")
        pitch = out.stride(0)
    else:
        splits = 1
        out = torch.empty((tokens, features), dtype=torch.float32 if mode == "f32" else torch.bfloat16, device=x.device)
    lib = load_library("gemm_bf16")
    _check(lib, lib.srb_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), tokens, features, k, x.stride(0), w.stride(0), pitch,
                                  rows, int(up_row_offset), code, int(splits), activation_code(activation),
                                  _ptr(error_word), _stream()))
    return out


@traced("gemm")
def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, error_word: torch.Tensor, *, mode: str = "bf16",
                   features: Optional[int] = None, up_row_offset: int = 0, activation: str = "silu") -> torch.Tensor:
    """y = x @ w^T for many tokens: 256 x 256 tiles on pairs of CTAs (``tcgen05.mma.cta_group::2``) in a
    persistent kernel.  ``mode`` ``bf16`` or ``gated`` as in :func:`gemm_bf16`; the result is bfloat16."""
    _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
    tokens, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k or mode not in ("bf16", "gated"):
        raise KernelError(f"gemm_bf16_pair: x {tuple(x.shape)}, w {tuple(w.shape)} or mode {mode!r} do not fit")
    if features is None:
        features = rows
    pitch = -(-features // 8) * 8
    out = torch.empty((tokens, pitch), dtype=torch.bfloat16, device=x.device)
    lib = load_library("gemm_bf16_pair")
    _check(lib, lib.srb_gemm_bf16_pair(_ptr(x), _ptr(w), _ptr(out), tokens, features, k, x.stride(0), w.stride(0), pitch,
                                       rows, int(up_row_offset), GEMM_MODES[mode], activation_code(activation),
                                       _ptr(error_word), _stream()))
    return out if pitch == features else out[:, :features]


def pair_gemm_takes(tokens: int, features: int, k: int) -> bool:
    """True if a bfloat16 gate/up product of this shape goes to the CTA-pair kernel."""
    return tokens >= PAIR_GEMM_MIN_TOKENS and features % 8 == 0 and k % 8 == 0


def gemm_bf16_takes(k: int) -> bool:
    """TMA needs 16-byte rows: the inner size must be a multiple of 8 bfloat16 values."""
    return k % 8 == 0


# --------------------------------------------------------------------------- sampling

@traced("sampling")
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of 32-bit logits: argmax where temperature is None or <= 0, else
    inverse-CDF sampling of softmax(logits / temperature) with the row's uniform number."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32)
    if temperature is not None:
        _need(temperature, "temperature", torch.float32); _need(uniform, "uniform", torch.float32)
    lib = load_library("sampling")
    scratch = torch.empty(lib.srb_sample_scratch_floats(rows), dtype=torch.float32, device=logits.device)
    _check(lib, lib.srb_sample(_ptr(logits), rows, vocab, logits.stride(0), _ptr(temperature), _ptr(uniform),
                               _ptr(out), _ptr(scratch), _stream()), launches=2)
    return out


@traced("sampling")
def sample_filtered(logits: torch.Tensor, rows_index: Optional[torch.Tensor], temperature: torch.Tensor,
                    top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor,
                    out: torch.Tensor) -> None:
    """Sampling with top-k, top-p and min-p for the rows named in ``rows_index`` (int32; None: all rows),
    into ``out[row]``.  The option tensors hold one entry per row of ``logits``: temperature > 0, top_k
    (int32; <= 0: off), top_p (>= 1: off), min_p (<= 0: off), uniform in [0, 1)."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32); _need(min_p, "min_p", torch.float32); _need(uniform, "uniform", torch.float32)
    rows, vocab = logits.shape
    for name, tensor in (("temperature", temperature), ("top_k", top_k), ("top_p", top_p), ("min_p", min_p),
                         ("uniform", uniform), ("out", out)):
        if tensor.numel() < rows:
            raise KernelError(f"sample_filtered: {name} needs one entry per row")
    count = rows
    if rows_index is not None:
        _need(rows_index, "rows_index", torch.int32)
        count = rows_index.numel()
    if count == 0:
        return
    lib = load_library("sampling")
    # the rows' probabilities, each row padded to a multiple of four
    scratch = torch.empty(count * ((vocab + 3) & ~3), dtype=torch.float32, device=logits.device)
    _check(lib, lib.srb_sample_filtered(_ptr(logits), vocab, ctypes.c_longlong(logits.stride(0)), _ptr(rows_index), count,
                                        _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                                        _ptr(scratch), _ptr(out), _stream()))


@traced("sampling")
def count_tokens(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts_row[t] += 1`` for every token id in ``tokens`` (int32, on the device)."""
    _need(counts_row, "counts_row", torch.int32); _need(tokens, "tokens", torch.int32)
    lib = load_library("sampling")
    _check(lib, lib.srb_count_tokens(_ptr(counts_row), _ptr(tokens), tokens.numel(), counts_row.numel(), _stream()))


@traced("sampling")
def apply_penalties(logits: torch.Tensor, counts: torch.Tensor, index: torch.Tensor, presence: torch.Tensor,
                    frequency: torch.Tensor, repetition: torch.Tensor) -> None:
    """Penalises ``logits`` in place: row r uses the counts of ``counts[index[r]]`` (``index[r] < 0``: none).
    A token seen c > 0 times: divided by ``repetition[r]`` if positive, multiplied if negative, then
    lowered by ``presence[r] + frequency[r] * c``."""
    _need(logits, "logits", torch.float32); _need(counts, "counts", torch.int32); _need(index, "index", torch.int32)
    _need(presence, "presence", torch.float32); _need(frequency, "frequency", torch.float32)
    _need(repetition, "repetition", torch.float32)
    rows, vocab = logits.shape
    if counts.dim() != 2 or counts.shape[1] != vocab:
        raise KernelError("apply_penalties: counts must be [table rows, vocab]")
    lib = load_library("sampling")
    _check(lib, lib.srb_apply_penalties(_ptr(logits), rows, vocab, ctypes.c_longlong(logits.stride(0)), _ptr(counts),
                                        _ptr(index), _ptr(presence), _ptr(frequency), _ptr(repetition), _stream()))


@traced("sampling")
def count_picked(counts: torch.Tensor, index: torch.Tensor, picked: torch.Tensor) -> None:
    """``counts[index[r], picked[r]] += 1`` for every row with ``index[r] >= 0``."""
    _need(counts, "counts", torch.int32); _need(index, "index", torch.int32); _need(picked, "picked", torch.int32)
    lib = load_library("sampling")
    _check(lib, lib.srb_count_picked(_ptr(counts), counts.shape[1], _ptr(index), _ptr(picked), picked.numel(), _stream()))
