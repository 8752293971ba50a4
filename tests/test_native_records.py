"""The step executor's records: the ctypes structures agree with the C header field by field, the launch
heuristics answer on the host, and a model's parts hand over records only when they can (no GPU)."""
import ctypes
import os
import subprocess

import pytest

from sglang_rs_b200.ops import records

STRUCTS = [records.SxLinear, records.SxNorm, records.SxAttention, records.SxGatedMlp, records.SxBlock, records.SxCall,
           records.SxModel, records.SxLaunch, records.SxGroup, records.SxStep, records.SxKernels]


def test_structures_agree_with_the_header(tmp_path):
    """Every field of every structure has the offset, and every structure the size, that a C compiler gives
    the header's declaration of the same name."""
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "step_exec.h"', "int main(void) {"]
    expected = []
    for struct in STRUCTS:
        name = struct.__name__
        lines.append(f'  printf("%zu\\n", sizeof({name}));')
        expected.append(ctypes.sizeof(struct))
        for field, _ in struct._fields_:
            lines.append(f'  printf("%zu\\n", offsetof({name}, {field}));')
            expected.append(getattr(struct, field).offset)
    lines += ["  return 0;", "}"]
    source = tmp_path / "offsets.c"
    source.write_text("\n".join(lines))
    include = os.path.join(os.path.dirname(records.__file__), "..", "csrc")
    binary = tmp_path / "offsets"
    subprocess.check_call(["gcc", "-I", include, str(source), "-o", str(binary)])
    got = [int(x) for x in subprocess.check_output([str(binary)]).split()]
    assert got == expected


def test_heuristics_answer_on_the_host():
    from sglang_rs_b200 import ops
    # Qwen3-8B sizes on 148 SMs: QKV 6144 x 4096 has 48 tiles of 128 rows and 64 blocks of K
    assert ops.gemm_splits(8, 6144, 4096, sms=148) == 6
    assert ops.gemm_splits(8, 4096, 12288, sms=148) == 9
    assert ops.gemm_splits(65, 4096, 12288, sms=148) == 1            # above the few-token kernel's rows
    assert ops.gemm_splits(1, 151936, 4096, sms=148) == 1            # enough tiles without a cut
    for tokens in (1, 16, 64):
        for features, k in ((6144, 4096), (4096, 4096), (4096, 12288), (2048, 6144), (100, 72), (256, 512)):
            splits = ops.gemm_splits(tokens, features, k, sms=148)
            blocks = -(-k // 64)
            per = -(-blocks // splits)
            assert splits >= 1 and -(-blocks // per) == splits       # no split is left without work


def test_parts_without_a_record_keep_the_model_on_the_part_by_part_path():
    import torch
    from plain_model import TINY_A
    from sglang_rs_b200.engine.native import NativeModel
    from sglang_rs_b200.parts.base import Mixer
    from sglang_rs_b200.weights import build_model, random_tensors
    model, _ = build_model(dict(TINY_A))
    assert model.layers[0].native_record() is None                   # no weights yet
    tensors = random_tensors(model.tensor_specs(), 1, "cpu", torch.float32)
    model.load(tensors, "cpu", torch.float32)
    native = NativeModel.of(model)
    assert native is not None and native._record.num_blocks == 2 and native._record.hidden == TINY_A["hidden_size"]
    block = native._blocks[1]
    assert (block.mixer.n_q, block.mixer.n_kv, block.mixer.head_dim) == (4, 2, 16)
    assert block.feed_forward.inner == TINY_A["intermediate_size"] and block.mixer.rotary_dim == 16
    assert abs(block.input_norm.eps - TINY_A["rms_norm_eps"]) < 1e-12 and block.mixer.qkv.out_features == (4 + 2 + 2) * 16

    class Toy(Mixer):                                               # a mixer the executor knows nothing of
        def forward(self, ctx, cache, x):
            return x
    model.layers[1].mixer = Toy()
    assert model.layers[1].native_record() is None and NativeModel.of(model) is None
