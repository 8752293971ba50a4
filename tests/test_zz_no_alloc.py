"""The allocation-free entry point of the split-key attention, called through its exported
C symbol, against the ordinary entry point and against the plain implementation.

Some programs that load this library may not allocate device memory themselves (all of it
was handed to their own pools at start-up, or they run inside another allocator).  For them
``srb_paged_attention_noalloc`` keeps its scratch in an array inside the library.  This test
calls it twice in a row with different inputs, so that what the first call left in the
shared array would show in the second if anything relied on a clean start.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def load_symbol():
    from sglang_rs_b200.csrc.build import compile_library
    library = ctypes.CDLL(compile_library("attention_noalloc"))
    library.srb_last_error.restype = ctypes.c_char_p
    function = library.srb_paged_attention_noalloc
    function.restype = ctypes.c_int
    function.argtypes = ([ctypes.c_void_p] * 7 + [ctypes.c_int] * 10 + [ctypes.c_float, ctypes.c_void_p, ctypes.c_int,
                                                                         ctypes.c_void_p])
    library.srb_noalloc_scratch_floats.restype = ctypes.c_int
    return library, function


def make_case(dtype, seed, n_q=8, n_kv=2, d=64, page=16, lengths=(700, 257, 90, 1)):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // page) for n in lengths) + 2
    order = torch.randperm(pages, generator=g).tolist()
    k_pool = torch.randn(pages, n_kv, page, d, generator=g).to(DEV, dtype)
    v_pool = torch.randn(pages, n_kv, page, d, generator=g).to(DEV, dtype)
    table = torch.full((len(lengths), max(-(-n // page) for n in lengths)), -1, dtype=torch.int32)
    for r, n in enumerate(lengths):
        for j in range(-(-n // page)):
            table[r, j] = order.pop()
    q = torch.randn(len(lengths), n_q, d, generator=g).to(DEV, dtype)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    row_request = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, table.to(DEV), positions, row_request


def plain_rows(q, k_pool, v_pool, table, lengths):
    """Each row's attention by the plain implementation, over the keys gathered from the pages on the host
    (64-bit): the row is the last token of a sequence of ``lengths[r]`` keys."""
    page = k_pool.shape[2]
    out = torch.zeros(q.shape, dtype=torch.float64)
    k_host, v_host, table = k_pool.double().cpu(), v_pool.double().cpu(), table.cpu()
    for r, n in enumerate(lengths):
        pages = table[r, : -(-n // page)].long()
        k = k_host[pages].permute(0, 2, 1, 3).reshape(-1, k_pool.shape[1], k_pool.shape[3])[:n]
        v = v_host[pages].permute(0, 2, 1, 3).reshape(-1, v_pool.shape[1], v_pool.shape[3])[:n]
        out[r] = pm.plain_attention(q[r:r + 1].double().cpu(), k, v, 1.0 / math.sqrt(q.shape[2]), first_position=n - 1)[0]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype):
    from sglang_rs_b200 import ops
    library, function = load_symbol()
    split = 256
    for call, seed in enumerate((1, 2)):
        q, k_pool, v_pool, table, positions, row_request = make_case(dtype, seed)
        rows, n_q, d = q.shape
        max_splits = int((positions.cpu() // split + 1).max())
        scale = 1.0 / math.sqrt(d)
        word = ops.new_error_word(DEV)

        want = torch.empty_like(q)
        acc_n, ml_n = ops.attention_scratch_sizes(rows, n_q, d, max_splits)
        ops.paged_attention(q, k_pool, v_pool, want, positions, row_request, table, scale=scale, window=0,
                            split_size=split, max_splits=max_splits, scratch_acc=torch.empty(acc_n, device=DEV),
                            scratch_ml=torch.empty(ml_n, device=DEV), error_word=word)

        got = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        status = function(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), got.data_ptr(), positions.data_ptr(),
                          row_request.data_ptr(), table.data_ptr(), table.stride(0), rows, n_q, k_pool.shape[1], d,
                          k_pool.shape[2], k_pool.shape[0], 0, split, max_splits, scale, word.data_ptr(),
                          ops.dtype_code(dtype), torch.cuda.current_stream().cuda_stream)
        assert status == 0, library.srb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        ops.raise_on_error_word(word)
        tolerance = 1e-5 if dtype == torch.float32 else 1e-2
        error = float((got.double() - want.double()).abs().max() / want.double().abs().max())
        assert error <= tolerance, f"call {call}: {error:.3e}"
        # and against the plain implementation, which shares nothing with either entry point
        plain = plain_rows(q, k_pool, v_pool, table, [int(p) + 1 for p in positions.cpu()])
        error = float((got.double().cpu() - plain).abs().max() / plain.abs().max())
        assert error <= tolerance, f"call {call} against the plain implementation: {error:.3e}"


def test_no_alloc_entry_point_flags_a_row_with_more_splits_than_the_launch():
    """A caller that gives too small a ``max_splits`` for one of its rows gets a bit in the error word
    instead of a silently wrong row; a padding row (position -1) is skipped."""
    from sglang_rs_b200 import ops
    library, function = load_symbol()
    q, k_pool, v_pool, table, positions, row_request = make_case(torch.float32, 5)
    rows, n_q, d = q.shape
    split = 256
    enough = int((positions.cpu() // split + 1).max())          # the row of 700 keys needs 3 splits
    word = ops.new_error_word(DEV)
    out = torch.zeros_like(q)

    def call(splits, pos):
        return function(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), pos.data_ptr(),
                        row_request.data_ptr(), table.data_ptr(), table.stride(0), rows, n_q, k_pool.shape[1], d,
                        k_pool.shape[2], k_pool.shape[0], 0, split, splits, 1.0 / math.sqrt(d), word.data_ptr(), 0,
                        torch.cuda.current_stream().cuda_stream)
    assert call(enough, positions) == 0
    assert int(word.item()) == 0
    assert call(enough - 1, positions) == 0
    assert int(word.item()) == 16                                # SRB_FLAG_TOO_FEW_SPLITS
    with pytest.raises(ops.KernelError, match="more key splits"):
        ops.raise_on_error_word(word)
    padded = positions.clone()
    padded[1] = -1
    out.fill_(7.0)
    assert call(enough, padded) == 0
    torch.cuda.synchronize()
    assert int(word.item()) == 0 and bool((out[1] == 7.0).all())   # nothing was written for the padding row


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    library, function = load_symbol()
    q, k_pool, v_pool, table, positions, row_request = make_case(torch.float32, 3)
    rows, n_q, d = q.shape
    limit = library.srb_noalloc_scratch_floats()
    too_many = limit // (rows * n_q * (d + 2)) + 1
    out = torch.empty_like(q)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    args = lambda split, splits: (q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(),  # noqa: E731
                                  positions.data_ptr(), row_request.data_ptr(), table.data_ptr(), table.stride(0), rows,
                                  n_q, k_pool.shape[1], d, k_pool.shape[2], k_pool.shape[0], 0, split, splits, 0.125,
                                  word.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert function(*args(256, too_many)) != 0
    assert "exceed the built-in" in library.srb_last_error().decode()
    assert function(*args(0, 1)) != 0
    assert "split_size" in library.srb_last_error().decode()
