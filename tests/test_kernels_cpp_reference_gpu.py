"""Each kernel against the plain C++ reference of the same name (csrc/plain_reference.cu), in 32-bit and in
bfloat16, at sizes that are no multiple of a tile.  The other kernel tests compare with the plain Python
implementation; the two oracles are compared with each other in test_cpp_reference.py."""
import math

import pytest
import torch

from sglang_rs_b200 import ops
from sglang_rs_b200.ops import plain_reference as cpp
from test_kernels_gpu import DEV, DTYPES, close, paged_case, rounded, run_attention, run_decode, run_tiled

pytestmark = pytest.mark.gpu


def seen(t, dtype):
    """What the kernel sees of ``t``: the value after storage in ``dtype``, as float32 for the C++ side."""
    return rounded(t, dtype).float()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_norm_and_gated_product(dtype):
    g = torch.Generator().manual_seed(4)
    table = torch.randn(300, 136, generator=g)
    ids = torch.randint(0, 300, (9,), generator=g).to(torch.int32)
    residual = torch.empty(9, 136, device=DEV)
    word = ops.new_error_word(DEV)
    ops.embedding(ids.to(DEV), table.to(DEV, dtype), residual, word)
    close(residual, cpp.embedding(ids, seen(table, dtype)), dtype, "embedding")
    delta, weight = torch.randn(9, 136, generator=g), 1 + 0.1 * torch.randn(136, generator=g)
    want_sum, want_norm = cpp.add_rms_norm(residual.cpu(), seen(delta, dtype), weight, 1e-6)
    out = torch.empty(9, 136, device=DEV, dtype=dtype)
    ops.add_rmsnorm(residual, delta.to(DEV, dtype), weight.to(DEV), 1e-6, out)
    close(residual, want_sum, torch.float32, "residual + delta")
    close(out, want_norm, dtype, "norm")
    gate_up = torch.randn(7, 2 * 200, generator=g) * 3
    for activation in ("silu", "gelu_tanh"):
        act = torch.empty(7, 200, device=DEV, dtype=dtype)
        ops.gated_mul(gate_up.to(DEV, dtype), act, activation)
        close(act, cpp.gated_mul(seen(gate_up, dtype), activation), dtype, activation)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 200, 136), (8, 333, 72), (64, 130, 512), (70, 257, 264), (300, 96, 200)])
def test_products(dtype, m, n, k):
    """Few rows (this package's tcgen05 kernel in bfloat16, partial sums and all), more rows (the library), and
    the 32-bit FFMA kernel, against the triple loop."""
    g = torch.Generator().manual_seed(m + n)
    x, w, bias = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g) * 0.1, torch.randn(n, generator=g)
    want = cpp.linear(seen(x, dtype), seen(w, dtype), bias)
    word = ops.new_error_word(DEV)
    got = ops.linear(x.to(DEV, dtype), w.to(DEV, dtype), bias.to(DEV), error_word=word, partial_ok=True)
    if got.dim() == 3:                                        # partial sums of a product cut along K
        got = got.sum(0)
    ops.raise_on_error_word(word)
    close(got, want, dtype, f"product {m} x {n} x {k}")
    if dtype == torch.bfloat16:
        both = cpp.linear(seen(x, dtype), seen(torch.cat([w, w.flip(0)]), dtype))
        want = cpp.gated_mul(both)
        got = ops.gated_product(x.to(DEV, dtype), torch.cat([w, w.flip(0)]).to(DEV, dtype), n, word)
        ops.raise_on_error_word(word)
        close(got, want, dtype, "gated product")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,n_q,n_kv,d", [(5, 4, 2, 18), (40, 6, 3, 128), (300, 8, 2, 128)])
def test_q_k_norm_rotation_and_page_write(dtype, rows, n_q, n_kv, d):
    g = torch.Generator().manual_seed(rows)
    page = 8
    pages = -(-rows // page) + 1
    qkv = torch.randn(rows, (n_q + 2 * n_kv) * d, generator=g)
    qn, kn = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.randint(0, 4000, (rows,), generator=g).to(torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:rows].to(torch.int32)
    inv = (1e6 ** (-torch.arange(0, d, 2).double() / d)).float()
    k_pool = torch.zeros(pages, n_kv, page, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(rows, n_q, d, device=DEV, dtype=dtype)
    word = ops.new_error_word(DEV)
    ops.qk_norm_rope_kv(qkv.to(DEV, dtype), q_out, k_pool, v_pool, positions.to(DEV), slots.to(DEV), qn.to(DEV), kn.to(DEV),
                        1e-6, inv.to(DEV), d, False, n_q, n_kv, d, word)
    ops.raise_on_error_word(word)
    values = seen(qkv, dtype)

    def heads(first, count, weight):
        flat = values[:, first * d:(first + count) * d].reshape(rows * count, d)
        _, normed = cpp.add_rms_norm(flat, None, weight, 1e-6)
        return cpp.rope(normed.view(rows, count, d), positions, inv)
    close(q_out, heads(0, n_q, qn), dtype, "q")
    at = (slots.long() // page, slots.long() % page)
    close(k_pool.cpu()[at[0], :, at[1]], heads(n_q, n_kv, kn), dtype, "k in its pages")
    close(v_pool.cpu()[at[0], :, at[1]], values[:, (n_q + n_kv) * d:].view(rows, n_kv, d), dtype, "v in its pages")


def reference_attention(case, scale):
    outs = []
    for k, v, q, n, rows in zip(case["ks"], case["vs"], case["qs"], case["lengths"], case["rows"]):
        outs.append(cpp.attention(seen(q, case["dtype"]), seen(k, case["dtype"]), seen(v, case["dtype"]), scale,
                                  window=case["window"], first_position=n - rows))
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(6, 2, 40, 16, None), (4, 2, 64, 8, 37), (8, 2, 128, 16, None)])
def test_attention_kernels(dtype, n_q, n_kv, d, page, window):
    """The generic kernel (unsplit and split), and in bfloat16 with head_dim 64 or 128 the three tensor-core
    kernels, all against the same loop nest."""
    scale = 0.8 / math.sqrt(d)
    portions = paged_case(dtype, n_q, n_kv, d, page, (1, 33, 300, 257), (1, 5, 140, 64), window, seed=d)
    want = reference_attention(portions, scale)
    for split in (0, 128):
        close(run_attention(portions, scale, split), want, dtype, f"generic, split {split}")
    if dtype == torch.bfloat16 and d in (64, 128):
        close(run_tiled(portions, scale), want, dtype, "mma.sync kernel for portions")
        if ops.tiled_attention_tc_takes(dtype, n_q, n_kv, d, page):
            close(run_tiled(portions, scale, tensor_memory=True), want, dtype, "tcgen05 kernel for portions")
        decoded = paged_case(dtype, n_q, n_kv, d, page, (1, 129, 700, 64), (1, 1, 1, 1), window, seed=d + 1)
        counters = torch.zeros(4 * n_kv, dtype=torch.int32, device=DEV)
        close(run_decode(decoded, scale, counters, max_keys=700), reference_attention(decoded, scale), dtype,
              "decode kernel")


def test_argmax_and_temperature_sampling():
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(5, 2049, generator=g) * 3
    picked = ops.sample(logits.to(DEV), None, None).cpu().tolist()
    assert picked == [cpp.argmax(row) for row in logits]
    temperature = torch.tensor([0.7, 1.0, 1.5, 0.3, 1.0])
    agree = total = 0
    for trial in range(10):
        u = torch.rand(5, generator=g)
        got = ops.sample(logits.to(DEV), temperature.to(DEV), u.to(DEV)).cpu().tolist()
        for r in range(5):
            total += 1
            agree += got[r] == cpp.sample(logits[r], float(temperature[r]), float(u[r]))
    assert agree >= total - 1                                 # a uniform number on the edge of two tokens may fall either way
