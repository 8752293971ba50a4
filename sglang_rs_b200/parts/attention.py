"""Grouped-query attention over the paged cache.

Order as in the reference (crates/sglang-srt/src/cpu_reference.rs:442-546): q, k, v
projections (+ bias if the checkpoint has them); RMSNorm of each q and k head with a
shared [head_dim] weight, before the rotation; rotation of q and k; k and v stored at the
row's slot; scores (q . k) * scale over the keys the row may see, kv head = q head /
(n_q / n_kv) (crates/sglang-kernel/src/cpu.rs:475-479); softmax; weighted sum of v; output
projection.  q, k and v come from one product with the row-wise concatenation of the
three matrices, made at load time.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Mixer, PagedKV, PositionEncoding, TensorSpec, matrix_to, scale_to


@dataclass(frozen=True)
class AttentionNames:
    q: str
    k: str
    v: str
    o: str
    q_norm: Optional[str] = None
    k_norm: Optional[str] = None
    q_bias: Optional[str] = None
    k_bias: Optional[str] = None
    v_bias: Optional[str] = None
    o_bias: Optional[str] = None


class GroupedQueryAttention(Mixer):
    graph_safe = True
    #: what the attention kernels take: the generic one gives a warp to each query head of a kv head (at most
    #: 32 warps a block) and keeps up to 16 values of a head per lane
    MAX_HEAD_DIM = 512
    MAX_HEADS_PER_KV_HEAD = 32

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 position: PositionEncoding, names: AttentionNames, *, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if not 0 < head_dim <= self.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {head_dim} is outside what the attention kernels take (1 to {self.MAX_HEAD_DIM})")
        if num_heads // num_kv_heads > self.MAX_HEADS_PER_KV_HEAD:
            raise ValueError(f"{num_heads // num_kv_heads} query heads per kv head exceed the "
                             f"{self.MAX_HEADS_PER_KV_HEAD} that the attention kernels take")
        self.hidden, self.n_q, self.n_kv, self.d = int(hidden), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.position, self.names = float(scale), position, names
        self.qk_norm_eps, self.window = qk_norm_eps, window
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_norm = self.k_norm = None

    def cache_need(self) -> PagedKV:
        return PagedKV(self.n_kv, self.d, self.window)

    def split_scratch(self):
        return (self.n_q * self.d, self.n_q * 2)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names
        specs = {
            n.q: TensorSpec((self.n_q * self.d, self.hidden)),
            n.k: TensorSpec((self.n_kv * self.d, self.hidden)),
            n.v: TensorSpec((self.n_kv * self.d, self.hidden)),
            n.o: TensorSpec((self.hidden, self.n_q * self.d)),
        }
        if n.q_norm:
            specs[n.q_norm] = TensorSpec((self.d,), "scale")
        if n.k_norm:
            specs[n.k_norm] = TensorSpec((self.d,), "scale")
        for name, width in ((n.q_bias, self.n_q * self.d), (n.k_bias, self.n_kv * self.d),
                            (n.v_bias, self.n_kv * self.d), (n.o_bias, self.hidden)):
            if name:
                specs[name] = TensorSpec((width,))
        specs.update(self.position.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n = self.names
        self.w_qkv = matrix_to(torch.cat([tensors[n.q], tensors[n.k], tensors[n.v]], dim=0), device, dtype)
        self.w_o = matrix_to(tensors[n.o], device, dtype)
        self.q_norm = scale_to(tensors[n.q_norm], device) if n.q_norm else None
        self.k_norm = scale_to(tensors[n.k_norm], device) if n.k_norm else None
        if n.q_bias or n.k_bias or n.v_bias:
            parts = []
            for name, width in ((n.q_bias, self.n_q * self.d), (n.k_bias, self.n_kv * self.d),
                                (n.v_bias, self.n_kv * self.d)):
                parts.append(tensors[name].to(torch.float32) if name else torch.zeros(width))
            self.b_qkv = scale_to(torch.cat(parts), device)
        self.b_o = scale_to(tensors[n.o_bias], device) if n.o_bias else None
        self.position.load(tensors, device, dtype)

    def native_record(self):
        """This mixer for the step executor, or None if its position encoding is not of the kind the fused
        kernel applies from a frequency table (an encoding that computes its angles in Python keeps the
        part-by-part path)."""
        from ..ops.records import SxAttention, linear_record
        if self.w_qkv is None or not self.position.fused:
            return None
        rotary = self.position.fused_rotary()
        if rotary is not None and (rotary.angles is not None or rotary.inv_freq is None):
            return None
        return SxAttention(
            linear_record(self.w_qkv, self.b_qkv), linear_record(self.w_o, self.b_o),
            None if self.q_norm is None else self.q_norm.data_ptr(), None if self.k_norm is None else self.k_norm.data_ptr(),
            None if rotary is None else rotary.inv_freq.data_ptr(),
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, self.scale,
            rotary.rotary_dim if rotary is not None else 0, int(rotary.interleaved) if rotary is not None else 0,
            self.n_q, self.n_kv, self.d, self.window or 0)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        batch = ctx.paged[cache.group]
        rows = x.shape[0]
        qkv = ops.linear(x, self.w_qkv, self.b_qkv, error_word=ctx.error_word, partial_ok=True)
        q = torch.empty((rows, self.n_q, self.d), dtype=x.dtype, device=x.device)
        rotary = self.position.fused_rotary() if self.position.fused else None
        if not self.position.fused:
            raise NotImplementedError("a position encoding with kernels of its own is applied by its mixer")
        ops.qk_norm_rope_kv(
            qkv, q, cache.k_pool if cache.writable else None, cache.v_pool if cache.writable else None,
            ctx.positions, batch.slots if cache.writable else None, self.q_norm, self.k_norm,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
            rotary.inv_freq if rotary else None, rotary.rotary_dim if rotary else 0,
            rotary.interleaved if rotary else False, self.n_q, self.n_kv, self.d, ctx.error_word,
            angles=rotary.angles(ctx.positions) if rotary is not None and rotary.angles is not None else None)
        out = torch.empty_like(q)
        for launch in batch.launches:
            b, e = launch.begin, launch.end
            if launch.wide_tiles is not None and ops.tiled_attention_tc_takes(q.dtype, self.n_q, self.n_kv, self.d,
                                                                              cache.k_pool.shape[2]):
                ops.tiled_attention_tc(q, cache.k_pool, cache.v_pool, out, launch.wide_tiles, batch.block_table,
                                       scale=self.scale, window=self.window or 0, error_word=ctx.error_word)
                continue
            if launch.tiles is not None and ops.tiled_attention_takes(q.dtype, self.n_q, self.n_kv, self.d):
                ops.tiled_attention(q, cache.k_pool, cache.v_pool, out, launch.tiles, batch.block_table,
                                    scale=self.scale, window=self.window or 0, error_word=ctx.error_word)
                continue
            if (launch.tiles is None and launch.split_size and batch.counters is not None
                    and batch.counters.numel() >= (e - b) * self.n_kv
                    and ops.decode_attention_takes(q.dtype, self.n_q, self.n_kv, self.d)):
                ops.decode_attention(q[b:e], cache.k_pool, cache.v_pool, out[b:e], ctx.positions[b:e],
                                     ctx.row_request[b:e], batch.block_table, scale=self.scale,
                                     window=self.window or 0, scratch_acc=batch.scratch_acc,
                                     scratch_ml=batch.scratch_ml, counters=batch.counters,
                                     error_word=ctx.error_word, max_keys=launch.max_keys)
                continue
            ops.paged_attention(q[b:e], cache.k_pool, cache.v_pool, out[b:e], ctx.positions[b:e],
                                ctx.row_request[b:e], batch.block_table, scale=self.scale,
                                window=self.window or 0, split_size=launch.split_size,
                                max_splits=launch.max_splits, scratch_acc=batch.scratch_acc,
                                scratch_ml=batch.scratch_ml, error_word=ctx.error_word)
        return ops.linear(out.view(rows, self.n_q * self.d), self.w_o, self.b_o, error_word=ctx.error_word,
                          partial_ok=True)
