"""Records of the step executor (csrc/step_exec.h) as ctypes structures, the executor's library, and cuBLAS.

The structures mirror csrc/step_exec.h field by field.  A part of a model fills the record of its kind
(``native_record()``); engine/native.py puts them together into the record of a model and fills the record
of a step.  The library also holds the launch heuristics that are functions of the shape (``gemm_splits``,
``decode_splits``) and the cuBLAS call that takes the products of many rows; both are used by the
part-by-part Python face as well, so there is one definition of each.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from ..csrc.build import load_library


class SxLinear(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("out_features", ctypes.c_int),
                ("in_features", ctypes.c_int)]


class SxNorm(ctypes.Structure):
    _fields_ = [("weight", ctypes.c_void_p), ("eps", ctypes.c_float), ("width", ctypes.c_int)]


class SxAttention(ctypes.Structure):
    _fields_ = [("qkv", SxLinear), ("o", SxLinear), ("q_norm", ctypes.c_void_p), ("k_norm", ctypes.c_void_p),
                ("inv_freq", ctypes.c_void_p), ("qk_eps", ctypes.c_float), ("scale", ctypes.c_float),
                ("rotary_dim", ctypes.c_int), ("interleaved", ctypes.c_int), ("n_q", ctypes.c_int), ("n_kv", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("window", ctypes.c_int)]


class SxGatedMlp(ctypes.Structure):
    _fields_ = [("gate_up", SxLinear), ("down", SxLinear), ("inner", ctypes.c_int), ("activation", ctypes.c_int)]


class SxBlock(ctypes.Structure):
    _fields_ = [("input_norm", SxNorm), ("mixer", SxAttention), ("post_norm", SxNorm), ("feed_forward", SxGatedMlp)]


class SxCall(ctypes.Structure):
    _fields_ = [("block", ctypes.c_int), ("group", ctypes.c_int), ("writable", ctypes.c_int), ("page_size", ctypes.c_int),
                ("num_pages", ctypes.c_int), ("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p)]


class SxModel(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int), ("vocab", ctypes.c_int), ("hidden", ctypes.c_int), ("embedding", ctypes.c_void_p),
                ("final_norm", SxNorm), ("head", SxLinear), ("num_blocks", ctypes.c_int), ("num_calls", ctypes.c_int),
                ("blocks", ctypes.POINTER(SxBlock)), ("calls", ctypes.POINTER(SxCall))]


class SxLaunch(ctypes.Structure):
    _fields_ = [("begin", ctypes.c_int), ("end", ctypes.c_int), ("split_size", ctypes.c_int), ("max_splits", ctypes.c_int),
                ("max_keys", ctypes.c_int), ("num_tiles", ctypes.c_int), ("num_wide_tiles", ctypes.c_int),
                ("reserved", ctypes.c_int), ("tiles", ctypes.c_void_p), ("wide_tiles", ctypes.c_void_p)]


class SxGroup(ctypes.Structure):
    _fields_ = [("block_table", ctypes.c_void_p), ("slots", ctypes.c_void_p), ("scratch_acc", ctypes.c_void_p),
                ("scratch_ml", ctypes.c_void_p), ("counters", ctypes.c_void_p), ("scratch_acc_floats", ctypes.c_longlong),
                ("scratch_ml_floats", ctypes.c_longlong), ("table_stride", ctypes.c_int), ("num_counters", ctypes.c_int),
                ("num_launches", ctypes.c_int), ("reserved", ctypes.c_int), ("launches", ctypes.POINTER(SxLaunch))]


SX_MAX_GROUPS = 4
#: kernels of a step that a measurement may leave out (``skip`` below): the SX_SKIP_* bits of csrc/step_exec.h
SKIP_BITS = {"norm": 1, "rope": 2, "attention": 4, "qkv": 8, "o": 16, "gate_up": 32, "down": 64, "head": 128}
#: bits that every step run by the executor leaves out; 0 except inside ``bench.py --mode ablate``
skip = 0


class SxStep(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int), ("num_wanted", ctypes.c_int), ("sms", ctypes.c_int),
                ("own_gemm_max_tokens", ctypes.c_int), ("pair_gemm_min_tokens", ctypes.c_int), ("num_groups", ctypes.c_int),
                ("skip", ctypes.c_int), ("reserved", ctypes.c_int),
                ("token_ids", ctypes.c_void_p), ("positions", ctypes.c_void_p), ("row_request", ctypes.c_void_p),
                ("logit_rows", ctypes.c_void_p), ("error_word", ctypes.c_void_p), ("workspace", ctypes.c_void_p),
                ("workspace_bytes", ctypes.c_longlong), ("logits", ctypes.c_void_p), ("stream", ctypes.c_void_p),
                ("groups", SxGroup * SX_MAX_GROUPS)]


#: the kernels of the table, in the order of SxKernels: (slot, library, exported name)
KERNEL_SLOTS = (
    ("embedding", "elementwise", "srb_embedding"), ("add_rmsnorm", "elementwise", "srb_add_rmsnorm"),
    ("gated_mul", "elementwise", "srb_gated_mul"), ("add_bias", "elementwise", "srb_add_bias"),
    ("gemm_f32", "gemm_f32", "srb_gemm_f32"), ("gemm_bf16", "gemm_bf16", "srb_gemm_bf16"),
    ("gemm_bf16_pair", "gemm_bf16_pair", "srb_gemm_bf16_pair"), ("qk_norm_rope_kv", "rope_kv", "srb_qk_norm_rope_kv_table"),
    ("rope_table", "rope_kv", "srb_rope_table"),
    ("paged_attention", "attention", "srb_paged_attention"), ("decode_attention", "attention_decode", "srb_decode_attention"),
    ("prefill_attention", "attention_prefill", "srb_prefill_attention"),
    ("prefill_attention_tc", "attention_prefill_tc", "srb_prefill_attention_tc"),
)


class SxKernels(ctypes.Structure):
    _fields_ = [field for slot, _, _ in KERNEL_SLOTS for field in ((slot, ctypes.c_void_p), (slot + "_error", ctypes.c_void_p))]


def _pointer(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def linear_record(weight: torch.Tensor, bias: Optional[torch.Tensor]) -> SxLinear:
    return SxLinear(_pointer(weight), _pointer(bias), weight.shape[0], weight.shape[1])


_library = None
_handed_over: set = set()
_workspaces: dict = {}


def library():
    """The executor's library with its prototypes set (it compiles and loads without a GPU: the heuristics of
    the kernels' launch shapes live in it and are asked for on the host)."""
    global _library
    if _library is None:
        lib = load_library("step_exec")
        lib.sx_workspace_bytes.restype = ctypes.c_longlong
        lib.sx_workspace_bytes.argtypes = [ctypes.POINTER(SxModel), ctypes.POINTER(SxStep)]
        lib.sx_run.argtypes = [ctypes.POINTER(SxModel), ctypes.POINTER(SxStep)]
        lib.sx_set_kernels.argtypes = [ctypes.POINTER(SxKernels)]
        lib.sx_load_cublas.argtypes = [ctypes.c_char_p]
        lib.sx_set_cublas_workspace.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        lib.sx_cublas_product.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 7 + [ctypes.c_void_p]
        _library = lib
    return _library


def _loaded_cublas_path() -> str:
    """The cuBLAS library that torch brought into the process, from the process's own map of libraries."""
    try:
        with open("/proc/self/maps") as handle:
            for line in handle:
                path = line.rsplit(" ", 1)[-1].strip()
                if "libcublas.so" in os.path.basename(path):
                    return path
    except OSError:
        pass
    return ""


#: bytes of scratch memory that cuBLAS is given per device (what torch gives it on this generation of GPUs)
CUBLAS_WORKSPACE_BYTES = 32 << 20


def hand_over_kernels(libraries: Sequence[str]) -> None:
    """Gives the executor the entry points of the named kernel libraries (beside those it has already).  Only
    libraries that a model can reach are named, so that no kernel is compiled that is never launched."""
    new = set(libraries) - _handed_over
    if not new:
        return
    _handed_over.update(new)
    table = SxKernels()
    for slot, name, symbol in KERNEL_SLOTS:
        if name in _handed_over:
            kernels = load_library(name)
            setattr(table, slot, ctypes.cast(getattr(kernels, symbol), ctypes.c_void_p).value)
            setattr(table, slot + "_error", ctypes.cast(kernels.srb_last_error, ctypes.c_void_p).value)
    library().sx_set_kernels(ctypes.byref(table))


def ensure_cublas(device) -> None:
    """cuBLAS for the products of many rows: the library that torch has loaded into the process is looked up
    (never a second copy), and it is given scratch memory of this package's on ``device``, so that it
    allocates nothing of its own (which it may not do while a stream is captured into a graph)."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index in _workspaces:
        return
    lib = library()
    with torch.cuda.device(index):
        torch.cuda.current_blas_handle()                       # torch loads and initialises cuBLAS
        if lib.sx_load_cublas(_loaded_cublas_path().encode()) != 0:
            raise RuntimeError(lib.srb_last_error().decode("utf-8", "replace"))
        workspace = torch.empty(CUBLAS_WORKSPACE_BYTES, dtype=torch.uint8, device=torch.device("cuda", index))
        if lib.sx_set_cublas_workspace(workspace.data_ptr(), CUBLAS_WORKSPACE_BYTES) != 0:
            raise RuntimeError(lib.srb_last_error().decode("utf-8", "replace"))
        _workspaces[index] = workspace


