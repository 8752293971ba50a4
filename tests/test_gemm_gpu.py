"""The tcgen05 / TMEM / TMA matrix product alone, against a 64-bit product of the same
bfloat16 values, at sizes that are no multiple of any tile."""
import math

import pytest
import torch

import plain_model as pm
from sglang_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def operands(tokens, features, k, seed, rows=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(rows or features, k, generator=g) * 0.5).to(torch.bfloat16)
    return x, w


def relative_error(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max())


@pytest.mark.parametrize("tokens,features,k", [(1, 128, 64), (8, 256, 128), (3, 331, 72), (17, 130, 200), (64, 512, 4096),
                                               (100, 96, 1000), (300, 640, 328), (1, 6144, 4096), (513, 257, 136)])
def test_plain_product(tokens, features, k):
    x, w = operands(tokens, features, k, seed=tokens + k)
    word = ops.new_error_word(DEV)
    want = pm.plain_linear(x.double(), w.double())
    got = ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="f32")
    ops.raise_on_error_word(word)
    assert relative_error(got, want) < 1e-5           # 32-bit accumulation of exact bfloat16 products
    rounded = ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="bf16")
    assert rounded.dtype == torch.bfloat16 and relative_error(rounded, want) < 5e-3
    ops.raise_on_error_word(word)


@pytest.mark.parametrize("tokens,features,k,splits", [(2, 128, 256, 2), (8, 200, 4096, 5), (33, 384, 1000, 16), (64, 64, 328, 3)])
def test_partial_sums_over_k(tokens, features, k, splits):
    x, w = operands(tokens, features, k, seed=7)
    word = ops.new_error_word(DEV)
    parts = ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="partial", splits=splits)
    ops.raise_on_error_word(word)
    assert parts.shape == (splits, tokens, features)
    want = pm.plain_linear(x.double(), w.double())
    assert relative_error(parts.double().sum(0), want) < 1e-5
    assert float(parts[-1].abs().max()) > 0        # the last split did its share


@pytest.mark.parametrize("tokens,features,k,splits", [(1, 128, 64, 1), (8, 4096, 4096, 8), (5, 200, 1000, 3), (33, 384, 1000, 8),
                                                      (64, 70, 328, 2), (128, 257, 520, 5), (100, 300, 200, 4)])
def test_product_added_to_a_float_tensor_inside_a_cluster(tokens, features, k, splits):
    """The K splits of a tile form a thread-block cluster and add their sum, in block order, onto a
    float tensor in place (the residual stream): against the 64-bit product, twice in a row (the
    second call adds again), and the same bits every time."""
    x, w = operands(tokens, features, k, seed=11 + tokens)
    g = torch.Generator().manual_seed(3)
    start = torch.randn(tokens, features, generator=g)
    word = ops.new_error_word(DEV)
    want = pm.plain_linear(x.double(), w.double())
    into = start.to(DEV)
    ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="add", splits=splits, out=into)
    ops.raise_on_error_word(word)
    scale = float(want.abs().max())
    assert float((into.double().cpu() - (start.double() + want)).abs().max()) < 1e-5 * scale
    first = into.clone()
    ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="add", splits=splits, out=into)
    assert float((into.double().cpu() - (start.double() + 2 * want)).abs().max()) < 2e-5 * scale
    again = start.to(DEV)
    ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="add", splits=splits, out=again)
    assert torch.equal(again, first)
    # a tensor with a wider row pitch (a view of a larger buffer) is taken; other columns stay
    wide = torch.zeros(tokens, features + 24, device=DEV)
    ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="add", splits=splits, out=wide[:, :features])
    ops.raise_on_error_word(word)
    assert float(wide[:, features:].abs().max()) == 0.0
    assert float((wide[:, :features].double().cpu() - want).abs().max()) < 1e-5 * scale
    with pytest.raises(ops.KernelError, match="at most"):
        ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="add", splits=9, out=into)


def gelu_tanh_mul(gate, up):
    """The second activation of the kernels, written out: g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u.
    No model of this package uses it; it shows that the activation is an argument, not a kernel."""
    return 0.5 * gate * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (gate + 0.044715 * gate ** 3))) * up


GATED = {"silu": pm.plain_silu_mul, "gelu_tanh": gelu_tanh_mul}


@pytest.mark.parametrize("activation", list(GATED))
@pytest.mark.parametrize("tokens,inner,k", [(1, 128, 64), (8, 200, 72), (70, 256, 512), (129, 130, 200)])
def test_gate_up_with_the_activation_in_the_epilogue(tokens, inner, k, activation):
    x, w = operands(tokens, inner, k, seed=11, rows=2 * inner)
    x = x * 3                                                 # gate values where the activations differ
    word = ops.new_error_word(DEV)
    got = ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="gated", features=inner, up_row_offset=inner,
                        activation=activation)
    ops.raise_on_error_word(word)
    both = pm.plain_linear(x.double(), w.double())
    want = GATED[activation](both[:, :inner], both[:, inner:])
    assert got.shape == (tokens, inner) and relative_error(got, want) < 5e-3
    with pytest.raises(ops.KernelError, match="unknown activation"):
        ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="gated", features=inner, up_row_offset=inner, activation="relu6")


def test_a_rows_result_does_not_depend_on_the_rows_beside_it():
    x, w = operands(40, 256, 512, seed=5)
    word = ops.new_error_word(DEV)
    together = ops.gemm_bf16(x.to(DEV), w.to(DEV), word, mode="f32")
    alone = ops.gemm_bf16(x[17:18].contiguous().to(DEV), w.to(DEV), word, mode="f32")
    assert torch.equal(together[17], alone[0])


def test_sizes_tma_cannot_take_are_refused():
    x, w = operands(4, 128, 68, seed=1)
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_bf16(x.to(DEV), w.to(DEV), ops.new_error_word(DEV))
    assert not ops.gemm_bf16_takes(68) and ops.gemm_bf16_takes(72)


@pytest.mark.parametrize("tokens,features,k", [(256, 256, 64), (300, 640, 328), (2048, 512, 1024), (513, 257, 136),
                                               (130, 1000, 200), (1100, 96, 4096)])
def test_product_on_pairs_of_ctas(tokens, features, k):
    """The persistent kernel for many tokens: 256 x 256 tiles on CTA pairs (cta_group::2), two
    accumulators in tensor memory; sizes that are no multiple of a tile, several tiles per pair."""
    x, w = operands(tokens, features, k, seed=tokens + features)
    word = ops.new_error_word(DEV)
    want = pm.plain_linear(x.double(), w.double())
    got = ops.gemm_bf16_pair(x.to(DEV), w.to(DEV), word, mode="bf16")
    ops.raise_on_error_word(word)
    assert got.shape == (tokens, features) and relative_error(got, want) < 5e-3
    again = ops.gemm_bf16_pair(x.to(DEV), w.to(DEV), word, mode="bf16")
    assert torch.equal(again, got)


@pytest.mark.parametrize("activation", list(GATED))
@pytest.mark.parametrize("tokens,inner,k", [(256, 128, 64), (700, 200, 72), (1030, 256, 512), (300, 130, 200)])
def test_gate_up_with_the_activation_on_pairs_of_ctas(tokens, inner, k, activation):
    x, w = operands(tokens, 2 * inner, k, seed=5 + inner)
    x = x * 3
    word = ops.new_error_word(DEV)
    got = ops.gemm_bf16_pair(x.to(DEV), w.to(DEV), word, mode="gated", features=inner, up_row_offset=inner,
                             activation=activation)
    ops.raise_on_error_word(word)
    gate_up = pm.plain_linear(x.double(), w.double())
    want = GATED[activation](gate_up[:, :inner], gate_up[:, inner:])
    assert got.shape == (tokens, inner) and relative_error(got, want) < 1e-2


@pytest.mark.parametrize("activation", list(GATED))
@pytest.mark.parametrize("tokens", [3, 64, 65, 300, 1279, 1280, 1400])
def test_gate_up_takes_the_kernel_of_its_row_count(tokens, activation):
    """`gated_product` runs the few-token kernel, the library's product with the activation kernel, or the
    CTA-pair kernel, by the number of rows: the same result from each."""
    inner, k = 264, 200
    x, w = operands(tokens, 2 * inner, k, seed=tokens)
    word = ops.new_error_word(DEV)
    got = ops.gated_product(x.to(DEV), w.to(DEV), inner, word, activation)
    ops.raise_on_error_word(word)
    gate_up = pm.plain_linear(x.double(), w.double())
    want = GATED[activation](gate_up[:, :inner], gate_up[:, inner:])
    assert got.shape == (tokens, inner) and relative_error(got, want) < 1e-2
