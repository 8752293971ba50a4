"""The plain C++ references of the kernels (csrc/plain_reference.cu) against the plain Python implementation:
two restatements of the reference's formulas, written apart, that must agree (no GPU)."""
import math

import pytest
import torch

import plain_model as pm
from sglang_rs_b200.ops import plain_reference as cpp


def close(a, b, bound=2e-6):
    scale = float(b.abs().max()) or 1.0
    assert float((a.double() - b.double()).abs().max()) <= bound * scale


def test_norm_linear_and_gated_product():
    g = torch.Generator().manual_seed(1)
    x, delta = torch.randn(5, 72, generator=g), torch.randn(5, 72, generator=g)
    w = 1 + 0.1 * torch.randn(72, generator=g)
    summed, normed = cpp.add_rms_norm(x, delta, w, 1e-5)
    close(summed, x.double() + delta.double())
    close(normed, pm.plain_rms_norm(x.double() + delta.double(), w.double(), 1e-5))
    _, alone = cpp.add_rms_norm(x, None, w, 3e-6)
    close(alone, pm.plain_rms_norm(x.double(), w.double(), 3e-6))
    weight, bias = torch.randn(33, 72, generator=g), torch.randn(33, generator=g)
    close(cpp.linear(x, weight, bias), pm.plain_linear(x.double(), weight.double(), bias.double()))
    close(cpp.linear(x, weight), pm.plain_linear(x.double(), weight.double()))
    gate_up = torch.randn(4, 2 * 50, generator=g) * 3
    close(cpp.gated_mul(gate_up), pm.plain_silu_mul(gate_up[:, :50].double(), gate_up[:, 50:].double()))
    g_, u_ = gate_up[:, :50].double(), gate_up[:, 50:].double()
    close(cpp.gated_mul(gate_up, "gelu_tanh"),
          0.5 * g_ * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g_ + 0.044715 * g_ ** 3))) * u_)


def test_embedding_rope_and_attention():
    g = torch.Generator().manual_seed(2)
    table = torch.randn(40, 24, generator=g)
    ids = torch.tensor([3, 39, 0, 3])
    assert torch.equal(cpp.embedding(ids, table), table[ids])
    with pytest.raises(IndexError):
        cpp.embedding(torch.tensor([40]), table)
    rows, n_q, n_kv, d = 37, 6, 2, 48
    positions = torch.randint(0, 3000, (rows,), generator=g)
    inv = pm.plain_inverse_frequencies(50000.0, d)
    x = torch.randn(rows, n_q, d, generator=g)
    close(cpp.rope(x, positions, inv), pm.plain_rope_neox(x.double(), positions, inv), 2e-5)   # float32 angles
    q, k, v = (torch.randn(rows, n, d, generator=g) for n in (n_q, n_kv, n_kv))
    close(cpp.attention(q, k, v, 0.2), pm.plain_attention(q.double(), k.double(), v.double(), 0.2))
    close(cpp.attention(q, k, v, 0.2, window=9), pm.plain_attention(q.double(), k.double(), v.double(), 0.2, window=9))
    tail = cpp.attention(q[30:], k, v, 0.2, first_position=30)
    close(tail, pm.plain_attention(q.double(), k.double(), v.double(), 0.2)[30:])


def test_argmax_and_sampling():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(1531, generator=g) * 3
    logits[100] = logits[900] = 50.0
    assert cpp.argmax(logits) == pm.plain_argmax(logits) == 100
    for trial in range(20):
        u = float(torch.rand(1, generator=g))
        assert cpp.sample(logits, 0.7, u) == pm.plain_temperature_sample(logits, 0.7, u)
