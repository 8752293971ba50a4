"""The Python face of the step executor (csrc/step_exec.cu): a whole model step in one native call.

A model whose every part offers a ``native_record()`` (the parts of this package do: RMSNorm, grouped-query
attention with a rotation of the table kind, the gated feed-forward, the pre-norm block) is turned into
one ``SxModel`` record when its runner is made.  ``NativeModel.run`` then fills the record of a step from the
step's context and makes one call; the C++ side launches every kernel of every layer call.  A model
with a part that has no record (a mixer defined in a test, a rotation whose angles come from a Python
function) keeps running part by part through ``DecoderModel.forward``; both ways launch the same kernels
with the same arguments.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..ops import records
from ..ops.records import (SX_MAX_GROUPS, SxBlock, SxCall, SxLaunch, SxModel, SxStep, library, linear_record)


def _pointer(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def prepare(native: "NativeModel", page_size: int) -> None:
    """Hands the executor the kernels this model can reach and readies cuBLAS on the model's device."""
    wanted = {"elementwise", "rope_kv", "attention"}
    dtype = native.dtype
    if dtype == torch.float32:
        wanted.add("gemm_f32")
    else:
        wanted |= {"gemm_bf16", "gemm_bf16_pair"}
        for n_q, n_kv, head_dim in native.attention_shapes():
            if ops.decode_attention_takes(dtype, n_q, n_kv, head_dim):
                wanted.add("attention_decode")
            if ops.tiled_attention_tc_takes(dtype, n_q, n_kv, head_dim, page_size):
                wanted.add("attention_prefill_tc")
            elif ops.tiled_attention_takes(dtype, n_q, n_kv, head_dim):
                wanted.add("attention_prefill")
        records.ensure_cublas(native.device)
    records.hand_over_kernels(sorted(wanted))


class NativeModel:
    """The records of one loaded model, and the call that runs a step through them."""

    def __init__(self, model, blocks: List[SxBlock]):
        # what is needed of the model, not the model itself: the model refers to this object, and a cycle would keep
        # the weights alive until a collection of garbage
        self.program, self.vocab_size = list(model.program), model.vocab_size
        self.device, self.dtype = model.device, model.dtype
        self._blocks = (SxBlock * len(blocks))(*blocks)
        self._calls = None
        self._calls_of = None
        self._record = SxModel()
        r = self._record
        r.dtype = ops.dtype_code(self.dtype)
        r.vocab, r.hidden = model.vocab_size, model.embedding.width
        r.embedding = model.embedding.table.data_ptr()
        r.final_norm = model.final_norm.native_record()
        head = model.head.weight if model.head.weight_name else model.head.embedding.table
        r.head = linear_record(head, None)
        r.num_blocks = len(blocks)
        r.blocks = ctypes.cast(self._blocks, ctypes.POINTER(SxBlock))
        self._step = SxStep()
        self._lib = library()
        #: scratch memory between the kernels of a step: kept from step to step and grown when a step needs more
        #: (steps run one after another on one stream).  A step that is being captured into a CUDA graph takes
        #: memory of its own from the graph's pool instead, which then belongs to that graph's replays.
        self._workspace: Optional[torch.Tensor] = None

    @classmethod
    def of(cls, model) -> Optional["NativeModel"]:
        """The records of ``model``, or None if one of its parts has none."""
        blocks = []
        for part in (model.embedding, model.final_norm, model.head):
            if not hasattr(part, "native_record") or part.native_record() is None:
                return None
        for layer in model.layers:
            record = layer.native_record() if hasattr(layer, "native_record") else None
            if not isinstance(record, SxBlock):
                return None
            blocks.append(record)
        return cls(model, blocks)

    def attention_shapes(self) -> List[tuple]:
        return [(b.mixer.n_q, b.mixer.n_kv, b.mixer.head_dim) for b in self._blocks]

    def _bind_caches(self, ctx, caches: Sequence) -> None:
        """The program's calls with the pools they read and write (made once per set of caches)."""
        groups = list(ctx.paged)
        calls = (SxCall * len(self.program))()
        for index, call in enumerate(self.program):
            source = caches[index if call.cache_from is None else call.cache_from]
            record = calls[index]
            record.block = call.layer
            record.group = groups.index(source.group)
            record.writable = int(call.cache_from is None and source.writable)
            record.page_size, record.num_pages = source.k_pool.shape[2], source.k_pool.shape[0]
            record.k_pool, record.v_pool = source.k_pool.data_ptr(), source.v_pool.data_ptr()
        self._calls, self._calls_of = calls, (caches[0], caches[-1], len(caches), tuple(groups))
        self._record.num_calls = len(calls)
        self._record.calls = ctypes.cast(calls, ctypes.POINTER(SxCall))

    def run(self, ctx, caches: Sequence, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        groups = list(ctx.paged)
        if len(groups) > SX_MAX_GROUPS:
            raise ops.KernelError(f"a step with {len(groups)} cache groups exceeds the executor's {SX_MAX_GROUPS}")
        bound = self._calls_of
        if bound is None or bound[0] is not caches[0] or bound[1] is not caches[-1] or bound[2] != len(caches) \
                or bound[3] != tuple(groups):
            self._bind_caches(ctx, caches)
        step = self._step
        step.rows = ctx.num_rows
        wanted = 0 if logit_rows is None else logit_rows.numel()
        step.num_wanted = wanted
        step.sms = ops.sm_count(self.device)
        step.own_gemm_max_tokens, step.pair_gemm_min_tokens = ops.OWN_GEMM_MAX_TOKENS, ops.PAIR_GEMM_MIN_TOKENS
        step.num_groups = len(groups)
        step.skip = records.skip
        step.token_ids, step.positions = ctx.token_ids.data_ptr(), ctx.positions.data_ptr()
        step.row_request = ctx.row_request.data_ptr()
        step.logit_rows = logit_rows.data_ptr() if wanted else None
        step.error_word = ctx.error_word.data_ptr()
        step.stream = ops._stream()
        keep = []
        for g, key in enumerate(groups):
            batch, record = ctx.paged[key], step.groups[g]
            record.block_table, record.table_stride = batch.block_table.data_ptr(), batch.block_table.stride(0)
            record.slots = batch.slots.data_ptr()
            record.scratch_acc, record.scratch_ml = _pointer(batch.scratch_acc), _pointer(batch.scratch_ml)
            record.scratch_acc_floats = 0 if batch.scratch_acc is None else batch.scratch_acc.numel()
            record.scratch_ml_floats = 0 if batch.scratch_ml is None else batch.scratch_ml.numel()
            record.counters = _pointer(batch.counters)
            record.num_counters = 0 if batch.counters is None else batch.counters.numel()
            launches = (SxLaunch * max(len(batch.launches), 1))()
            for i, launch in enumerate(batch.launches):
                item = launches[i]
                item.begin, item.end, item.split_size, item.max_splits = launch.begin, launch.end, launch.split_size, launch.max_splits
                item.max_keys = -1 if launch.max_keys is None else int(launch.max_keys)
                item.tiles = _pointer(launch.tiles)
                item.num_tiles = 0 if launch.tiles is None else launch.tiles.shape[0]
                item.wide_tiles = _pointer(launch.wide_tiles)
                item.num_wide_tiles = 0 if launch.wide_tiles is None else launch.wide_tiles.shape[0]
            record.num_launches = len(batch.launches)
            record.launches = ctypes.cast(launches, ctypes.POINTER(SxLaunch))
            keep.append(launches)
        step.workspace, step.workspace_bytes = None, 0
        need = self._lib.sx_workspace_bytes(ctypes.byref(self._record), ctypes.byref(step))
        if torch.cuda.is_current_stream_capturing():
            workspace = torch.empty(need + 256, dtype=torch.uint8, device=self.device)
        else:
            if self._workspace is None or self._workspace.numel() < need + 256:
                self._workspace = None                          # the old one goes back before the new one is asked for
                self._workspace = torch.empty(int((need + 256) * 1.25), dtype=torch.uint8, device=self.device)
            workspace = self._workspace
        address = workspace.data_ptr()
        step.workspace = (address + 255) // 256 * 256
        step.workspace_bytes = need
        logits = None
        if wanted:
            logits = torch.empty((wanted, self.vocab_size), dtype=torch.float32, device=self.device)
            step.logits = logits.data_ptr()
        else:
            step.logits = None
        launched = self._lib.sx_run(ctypes.byref(self._record), ctypes.byref(step))
        if launched < 0:
            raise ops.KernelError(self._lib.srb_last_error().decode("utf-8", "replace") or f"step executor status {launched}")
        ops.launch_count += launched
        return logits
