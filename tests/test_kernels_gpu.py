"""Each kernel alone against the plain implementation's function for the same part, at
sizes other than the engine's tests use, in 32-bit and in bfloat16."""
import math

import pytest
import torch

import plain_model as pm
from sglang_rs_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 1e-2       # relative to the largest |expected|


def close(got, want, dtype, what=""):
    want = want.to(torch.float64).cpu()
    got = got.to(torch.float64).cpu()
    scale = max(float(want.abs().max()), 1e-30)
    err = float((got - want).abs().max()) / scale
    assert err <= tol(dtype), f"{what}: error {err:.3e} of scale (tolerance {tol(dtype)})"


def rounded(t, dtype):
    """What the kernel sees: the value after storage in ``dtype``, widened to 64-bit."""
    return t.to(dtype).to(torch.float64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_bad_token(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(331, 72, generator=g)
    ids = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32)
    out = torch.empty(5, 72, device=DEV)
    word = ops.new_error_word(DEV)
    ops.embedding(ids.to(DEV), table.to(DEV, dtype), out, word)
    assert torch.equal(out.cpu().double(), rounded(table, dtype)[ids.long()])
    ops.raise_on_error_word(word)
    ops.embedding(torch.tensor([3, 331, -1], dtype=torch.int32, device=DEV), table.to(DEV, dtype), out[:3], word)
    assert torch.equal(out[1:3].cpu(), torch.zeros(2, 72))
    with pytest.raises(ops.KernelError, match="token id outside"):
        ops.raise_on_error_word(word)
    ops.raise_on_error_word(word)                         # reading it cleared it


def test_tokens_taken_from_the_step_before():
    """Rows whose token was chosen on the device by the step before take it from there; the others
    keep what the host wrote; an index outside the source is flagged and the row left alone."""
    g = torch.Generator().manual_seed(1)
    rows = 300
    tokens = torch.randint(0, 1000, (rows,), generator=g, dtype=torch.int32)
    source = torch.randint(1000, 2000, (77,), generator=g, dtype=torch.int32)
    index = torch.full((rows,), -1, dtype=torch.int32)
    chosen = torch.randperm(rows, generator=g)[:120]
    index[chosen] = torch.randint(0, 77, (120,), generator=g, dtype=torch.int32)
    want = tokens.clone()
    want[chosen] = source[index[chosen].long()]
    word = ops.new_error_word(DEV)
    got = tokens.to(DEV)
    ops.take_tokens(got, source.to(DEV), index.to(DEV), word)
    ops.raise_on_error_word(word)
    assert torch.equal(got.cpu(), want)
    index[5] = 77
    got = tokens.to(DEV)
    ops.take_tokens(got, source.to(DEV), index.to(DEV), word)
    assert int(got[5]) == int(tokens[5])
    with pytest.raises(ops.KernelError, match="token id outside"):
        ops.raise_on_error_word(word)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 100, 1023, 5120, 16400])
def test_add_rmsnorm(dtype, width):
    g = torch.Generator().manual_seed(width)
    rows = 7
    residual = torch.randn(rows, width, generator=g) * 3
    delta = torch.randn(rows, width, generator=g)
    weight = 1 + 0.1 * torch.randn(width, generator=g)
    eps = 3e-5
    res_d = residual.to(DEV)
    out = torch.empty(rows, width, device=DEV, dtype=dtype)
    ops.add_rmsnorm(res_d, delta.to(DEV, dtype), weight.to(DEV), eps, out)
    summed = residual.double() + rounded(delta, dtype)
    assert torch.allclose(res_d.cpu().double(), summed, atol=1e-6)        # the 32-bit sum is stored back
    close(out, pm.plain_rms_norm(summed, weight.double(), eps), dtype, "add+norm")
    # no delta; picked rows; the residual stays untouched
    before = res_d.clone()
    pick = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, width, device=DEV, dtype=dtype)
    ops.add_rmsnorm(res_d, None, weight.to(DEV), eps, out2, row_index=pick, write_residual=False)
    assert torch.equal(res_d, before)
    close(out2, pm.plain_rms_norm(before.cpu().double()[pick.cpu().long()], weight.double(), eps), dtype, "picked rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,parts,rows", [(4096, 9, 3), (4096, 9, 320), (2560, 16, 8), (2560, 17, 8), (264, 1, 64),
                                              (5128, 0, 37), (8192, 3, 2)])
def test_add_rmsnorm_of_few_and_of_many_rows(dtype, width, parts, rows):
    """Residual, pending sum and up to 17 partial sums are added in that order, for few rows and for many,
    at widths that take the vector kernel and widths that do not."""
    g = torch.Generator().manual_seed(width + parts + rows)
    residual = torch.randn(rows, width, generator=g) * 2
    weight = 1 + 0.1 * torch.randn(width, generator=g)
    eps = 1e-6
    res_d = residual.to(DEV)
    out = torch.full((rows, width), float("nan"), device=DEV, dtype=dtype)
    if parts:
        pieces = torch.randn(parts, rows, width, generator=g)
        ops.add_rmsnorm(res_d, pieces.to(DEV), weight.to(DEV), eps, out)
        summed = residual.double() + pieces.double().sum(0)
    else:
        delta = torch.randn(rows, width, generator=g)
        ops.add_rmsnorm(res_d, delta.to(DEV, dtype), weight.to(DEV), eps, out)
        summed = residual.double() + rounded(delta, dtype)
    assert torch.allclose(res_d.cpu().double(), summed, atol=1e-5)
    close(out, pm.plain_rms_norm(summed, weight.double(), eps), dtype, "add+norm")
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.full((2, width), float("nan"), device=DEV, dtype=dtype)
    before = res_d.clone()
    ops.add_rmsnorm(res_d, None, weight.to(DEV), eps, out2, row_index=pick, write_residual=False)
    assert torch.equal(res_d, before)
    close(out2, pm.plain_rms_norm(summed[pick.cpu().long()], weight.double(), eps), dtype, "picked rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_and_rope_take_partial_sums(dtype):
    """A product cut along K hands its consumer float partial sums; they are added in order."""
    g = torch.Generator().manual_seed(2)
    rows, width, parts = 5, 200, 3
    residual, weight = torch.randn(rows, width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    pieces = torch.randn(parts, rows, width, generator=g)
    res_d = residual.to(DEV)
    out = torch.empty(rows, width, device=DEV, dtype=dtype)
    ops.add_rmsnorm(res_d, pieces.to(DEV), weight.to(DEV), 1e-6, out)
    summed = residual.double() + pieces.double().sum(0)
    assert torch.allclose(res_d.cpu().double(), summed, atol=1e-5)
    close(out, pm.plain_rms_norm(summed, weight.double(), 1e-6), dtype, "norm of partial sums")
    n_q, n_kv, d = 3, 1, 32
    qkv = torch.randn(parts, rows, (n_q + 2 * n_kv) * d, generator=g)
    positions = torch.arange(rows, dtype=torch.int32)
    inv = pm.plain_inverse_frequencies(1e4, d)
    k_pool = torch.zeros(2, n_kv, 8, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(rows, n_q, d, device=DEV, dtype=dtype)
    word = ops.new_error_word(DEV)
    ops.qk_norm_rope_kv(qkv.to(DEV), q_out, k_pool, v_pool, positions.to(DEV), positions.to(DEV), None, None, 0.0,
                        inv.to(DEV), d, False, n_q, n_kv, d, word)
    ops.raise_on_error_word(word)
    total = qkv.double().sum(0)
    close(q_out, pm.plain_rope_neox(total[:, :n_q * d].view(rows, n_q, d), positions, inv), dtype, "q of partial sums")
    close(v_pool[0, 0, :rows], total[:, (n_q + n_kv) * d:], dtype, "v of partial sums")


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_and_bias(dtype):
    g = torch.Generator().manual_seed(1)
    gate_up = torch.randn(5, 2 * 200, generator=g) * 4
    out = torch.empty(5, 200, device=DEV, dtype=dtype)
    ops.gated_mul(gate_up.to(DEV, dtype), out)
    seen = rounded(gate_up, dtype)
    close(out, pm.plain_silu_mul(seen[:, :200], seen[:, 200:]), dtype, "silu*mul")
    ops.gated_mul(gate_up.to(DEV, dtype), out, "gelu_tanh")
    g_, u_ = seen[:, :200], seen[:, 200:]
    close(out, 0.5 * g_ * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g_ + 0.044715 * g_ ** 3))) * u_, dtype, "gelu*mul")
    values = torch.randn(4, 77, generator=g)
    bias = torch.randn(77, generator=g)
    v = values.to(DEV, dtype)
    ops.add_bias(v, bias.to(DEV))
    close(v, rounded(values, dtype) + bias.double(), dtype, "bias")


@pytest.mark.parametrize("m,n,k", [(1, 331, 72), (3, 64, 1000), (65, 130, 257), (200, 17, 48)])
def test_gemm_f32_is_true_32_bit(m, n, k):
    g = torch.Generator().manual_seed(m * n)
    x, w, b = torch.randn(m, k, generator=g), torch.randn(n, k, generator=g), torch.randn(n, generator=g)
    out = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV))
    want = pm.plain_linear(x.double(), w.double(), b.double())
    err = float((out.cpu().double() - want).abs().max() / want.abs().max())
    assert err < 3e-6, err                                # a TF32 product would be near 1e-3
    # a row's result does not depend on the rows beside it
    alone = ops.linear(x[m - 1:].contiguous().to(DEV), w.to(DEV), b.to(DEV))
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,rot,inter", [(4, 2, 16, 16, False), (5, 1, 48, 48, False), (3, 3, 128, 64, False),
                                                  (2, 1, 80, 80, True), (8, 2, 256, 256, False)])
def test_qk_norm_rope_kv(dtype, n_q, n_kv, d, rot, inter):
    g = torch.Generator().manual_seed(d + n_q)
    rows, page, pages = 9, 8, 6
    qkv = torch.randn(rows, (n_q + 2 * n_kv) * d, generator=g)
    qn, kn = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.tensor([0, 1, 2, 50, 51, 7, 8, 1000, 3], dtype=torch.int32)
    slots = torch.tensor([5, 6, 7, 40, 41, 16, 17, 0, 30], dtype=torch.int32)
    theta, eps = 50000.0, 1e-5
    inv = pm.plain_inverse_frequencies(theta, rot)
    k_pool = torch.zeros(pages, n_kv, page, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(rows, n_q, d, device=DEV, dtype=dtype)
    word = ops.new_error_word(DEV)
    ops.qk_norm_rope_kv(qkv.to(DEV, dtype), q_out, k_pool, v_pool, positions.to(DEV), slots.to(DEV), qn.to(DEV),
                        kn.to(DEV), eps, inv.to(DEV), rot, inter, n_q, n_kv, d, word)
    ops.raise_on_error_word(word)
    seen = rounded(qkv, dtype)
    q = pm.plain_rms_norm(seen[:, :n_q * d].view(rows, n_q, d), qn.double(), eps)
    k = pm.plain_rms_norm(seen[:, n_q * d:(n_q + n_kv) * d].view(rows, n_kv, d), kn.double(), eps)
    v = seen[:, (n_q + n_kv) * d:].view(rows, n_kv, d)

    def rotate(x):
        if not inter:
            out = x.clone()
            out[..., :rot] = pm.plain_rope_neox(x[..., :rot].contiguous(), positions, inv)
            return out
        # interleaved pairs (2i, 2i+1): the same rotation after a permutation (rotary.rs:223-226)
        perm = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2)])
        out = x.clone()
        out[..., perm] = pm.plain_rope_neox(x[..., perm].contiguous(), positions, inv)
        return out

    close(q_out, rotate(q), dtype, "q")
    k_want, v_want = rotate(k), v
    for r in range(rows):
        pg, off = int(slots[r]) // page, int(slots[r]) % page
        close(k_pool[pg, :, off], k_want[r], dtype, f"k row {r}")
        close(v_pool[pg, :, off], v_want[r], dtype, f"v row {r}")
    written = {(int(s) // page, int(s) % page) for s in slots}
    for pg in range(pages):
        for off in range(page):
            if (pg, off) not in written:
                assert float(k_pool[pg, :, off].abs().max()) == 0.0
    # a slot outside the pool is skipped and flagged
    ops.qk_norm_rope_kv(qkv.to(DEV, dtype), q_out, k_pool, v_pool, positions.to(DEV),
                        torch.full((rows,), pages * page, dtype=torch.int32, device=DEV), qn.to(DEV), kn.to(DEV), eps,
                        inv.to(DEV), rot, inter, n_q, n_kv, d, word)
    with pytest.raises(ops.KernelError, match="cache slot"):
        ops.raise_on_error_word(word)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("use_parts,n_q,n_kv", [(False, 6, 2), (True, 6, 2), (False, 32, 8), (False, 64, 8), (False, 5, 5)])
def test_qk_norm_rope_kv_many_rows_of_128(dtype, use_parts, n_q, n_kv):
    """Portions of 256 rows and more with head_dim 128 take a kernel that keeps a head in
    registers: against the plain formulas, and bit for bit against the kernel that the same rows
    take when they come a few at a time (a token's cache entry must not depend on the step it
    came in)."""
    g = torch.Generator().manual_seed(5)
    rows, d, page = 291, 128, 16        # 10, 48, 80 or 15 heads a row: less than a pass of 16, three passes, five, one
    pages = -(-rows // page) + 2
    width = (n_q + 2 * n_kv) * d
    qkv = torch.randn(rows, width, generator=g)
    qn, kn = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    positions = torch.randint(0, 5000, (rows,), generator=g).to(torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:rows].to(torch.int32)
    inv = pm.plain_inverse_frequencies(1e6, d)
    word = ops.new_error_word(DEV)
    if use_parts:
        parts = torch.randn(3, rows, width, generator=g)
        source, seen = parts.to(DEV), parts.double().sum(0)
    else:
        source, seen = qkv.to(DEV, dtype), rounded(qkv, dtype)

    def run(lo, hi, table=False):
        k_pool = torch.zeros(pages, n_kv, page, d, device=DEV, dtype=dtype)
        v_pool = torch.zeros_like(k_pool)
        q_out = torch.zeros(hi - lo, n_q, d, device=DEV, dtype=dtype)
        src = source[:, lo:hi].contiguous() if use_parts else source[lo:hi]
        cos_sin = ops.rope_table(positions[lo:hi].to(DEV), inv.to(DEV), d) if table else None
        ops.qk_norm_rope_kv(src, q_out, k_pool, v_pool, positions[lo:hi].to(DEV), slots[lo:hi].to(DEV), qn.to(DEV),
                            kn.to(DEV), 1e-6, inv.to(DEV), d, False, n_q, n_kv, d, word, cos_sin=cos_sin)
        return q_out, k_pool, v_pool

    q_out, k_pool, v_pool = run(0, rows)
    ops.raise_on_error_word(word)
    q = pm.plain_rope_neox(pm.plain_rms_norm(seen[:, :n_q * d].view(rows, n_q, d), qn.double(), 1e-6), positions, inv)
    k = pm.plain_rope_neox(pm.plain_rms_norm(seen[:, n_q * d:(n_q + n_kv) * d].view(rows, n_kv, d), kn.double(), 1e-6),
                           positions, inv)
    v = seen[:, (n_q + n_kv) * d:].view(rows, n_kv, d)
    close(q_out, q, dtype, "q")
    close(k_pool.cpu()[slots.long() // page, :, slots.long() % page], k, dtype, "k")
    close(v_pool.cpu()[slots.long() // page, :, slots.long() % page], v, dtype, "v")
    # with the cosines and sines computed once for all rows (as the step executor does): the same bits
    q_table, k_table, v_table = run(0, rows, table=True)
    assert torch.equal(q_table, q_out) and torch.equal(k_table, k_pool) and torch.equal(v_table, v_pool)
    table = ops.rope_table(positions.to(DEV), inv.to(DEV), d).cpu().double()
    angle = positions.double()[:, None] * inv.double()[None, :]
    assert float((table[:, :d // 2] - torch.cos(angle)).abs().max()) < 1e-3      # float32 angles of up to 5,000
    # the same rows, 37 at a time, through the kernel for few rows
    for lo in range(0, rows, 37):
        hi = min(rows, lo + 37)
        q_few, k_few, v_few = run(lo, hi)
        assert torch.equal(q_few, q_out[lo:hi])
        idx = slots[lo:hi].long()
        assert torch.equal(k_few[idx // page, :, idx % page], k_pool[idx // page, :, idx % page])
        assert torch.equal(v_few[idx // page, :, idx % page], v_pool[idx // page, :, idx % page])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,n_q,n_kv,d,rot", [(5, 3, 1, 32, 32), (150, 6, 2, 64, 48)])
def test_rope_from_a_table_of_angles(dtype, rows, n_q, n_kv, d, rot):
    """The kernel may be given an angle per (row, pair) instead of frequencies: another
    position encoding needs no kernel of its own.  Few rows and many rows take different
    ways through the kernel."""
    g = torch.Generator().manual_seed(rows + d)
    page = 8
    pages = -(-rows // page) + 1
    qkv = torch.randn(rows, (n_q + 2 * n_kv) * d, generator=g)
    qn, kn = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    angles = (torch.rand(rows, rot // 2, generator=g) * 12 - 6).float()
    slots = torch.randperm(pages * page, generator=g)[:rows].to(torch.int32)
    positions = torch.arange(rows, dtype=torch.int32)
    k_pool = torch.zeros(pages, n_kv, page, d, device=DEV, dtype=dtype)
    v_pool = torch.zeros_like(k_pool)
    q_out = torch.empty(rows, n_q, d, device=DEV, dtype=dtype)
    word = ops.new_error_word(DEV)
    ops.qk_norm_rope_kv(qkv.to(DEV, dtype), q_out, k_pool, v_pool, positions.to(DEV), slots.to(DEV), qn.to(DEV),
                        kn.to(DEV), 1e-6, None, rot, False, n_q, n_kv, d, word, angles=angles.to(DEV))
    ops.raise_on_error_word(word)
    seen = rounded(qkv, dtype)
    cos, sin = torch.cos(angles.double())[:, None, :], torch.sin(angles.double())[:, None, :]

    def rotate(x):
        out = x.clone()
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = a * cos - b * sin, b * cos + a * sin
        return out

    q = rotate(pm.plain_rms_norm(seen[:, :n_q * d].view(rows, n_q, d), qn.double(), 1e-6))
    k = rotate(pm.plain_rms_norm(seen[:, n_q * d:(n_q + n_kv) * d].view(rows, n_kv, d), kn.double(), 1e-6))
    close(q_out, q, dtype, "q from angles")
    got_k = k_pool.cpu()[slots.long() // page, :, slots.long() % page]
    close(got_k, k, dtype, "k from angles")


def paged_case(dtype, n_q, n_kv, d, page, lengths, rows_per_request, window, seed, boost=None):
    """Requests with their keys scattered over shuffled pages; the last ``rows`` positions of
    each request are the step's rows."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    k_pool = torch.randn(total_pages, n_kv, page, d, generator=g)       # stale values everywhere
    v_pool = torch.randn(total_pages, n_kv, page, d, generator=g)
    stride = max(-(-n // page) for n in lengths) + 1
    table = torch.full((len(lengths), stride), -1, dtype=torch.int32)
    ks, vs, qs, positions, row_request = [], [], [], [], []
    for r, (n, rows) in enumerate(zip(lengths, rows_per_request)):
        k, v = torch.randn(n, n_kv, d, generator=g), torch.randn(n, n_kv, d, generator=g)
        q = torch.randn(rows, n_q, d, generator=g)
        if boost is not None and n > boost[0]:
            # one far key stands out for the last row: its score dominates the softmax
            k[boost[0]] = q[-1, ::n_q // n_kv] * boost[1]
        for j in range(-(-n // page)):
            pg = order.pop()
            table[r, j] = pg
            chunk = slice(j * page, min(n, (j + 1) * page))
            k_pool[pg, :, :chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            v_pool[pg, :, :chunk.stop - chunk.start] = v[chunk].transpose(0, 1)
        ks.append(k); vs.append(v); qs.append(q)
        positions += list(range(n - rows, n))
        row_request += [r] * rows
    return dict(k_pool=k_pool.to(DEV, dtype), v_pool=v_pool.to(DEV, dtype), table=table.to(DEV),
                q=torch.cat(qs).to(DEV, dtype), positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                row_request=torch.tensor(row_request, dtype=torch.int32, device=DEV), ks=ks, vs=vs, qs=qs,
                lengths=lengths, rows=rows_per_request, window=window, dtype=dtype)


def expected_attention(case, scale):
    outs = []
    for k, v, q, n, rows in zip(case["ks"], case["vs"], case["qs"], case["lengths"], case["rows"]):
        outs.append(pm.plain_attention(rounded(q, case["dtype"]), rounded(k, case["dtype"]), rounded(v, case["dtype"]),
                                       scale, window=case["window"], first_position=n - rows))
    return torch.cat(outs)


def run_attention(case, scale, split_size):
    q = case["q"]
    rows, n_q, d = q.shape
    out = torch.full_like(q, float("nan"))
    word = ops.new_error_word(DEV)
    max_splits, acc, ml = 1, None, None
    if split_size:
        pos = case["positions"].cpu()
        begin = torch.clamp(pos + 1 - case["window"], min=0) if case["window"] else torch.zeros_like(pos)
        max_splits = int((pos // split_size - begin // split_size + 1).max())
        a, m = ops.attention_scratch_sizes(rows, n_q, d, max_splits)
        acc = torch.full((a,), float("nan"), device=DEV)
        ml = torch.full((m,), float("nan"), device=DEV)
    ops.paged_attention(q, case["k_pool"], case["v_pool"], out, case["positions"], case["row_request"], case["table"],
                        scale=scale, window=case["window"] or 0, split_size=split_size, max_splits=max_splits,
                        scratch_acc=acc, scratch_ml=ml, error_word=word)
    ops.raise_on_error_word(word)
    return out


def run_decode(case, scale, counters, max_keys=None):
    q = case["q"]
    rows, n_q, d = q.shape
    n_kv = case["k_pool"].shape[1]
    splits = ops.decode_splits(rows, n_kv, max_keys)
    out = torch.full_like(q, float("nan"))
    word = ops.new_error_word(DEV)
    acc = torch.full((rows * n_q * splits * d,), float("nan"), device=DEV)
    ml = torch.full((rows * n_q * splits * 2,), float("nan"), device=DEV)
    ops.decode_attention(q, case["k_pool"], case["v_pool"], out, case["positions"], case["row_request"], case["table"],
                         scale=scale, window=case["window"] or 0, scratch_acc=acc, scratch_ml=ml, counters=counters,
                         error_word=word, max_keys=max_keys)
    ops.raise_on_error_word(word)
    return out


@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(8, 2, 64, 16, None), (16, 1, 128, 8, 300), (6, 3, 128, 32, None),
                                                    (4, 4, 128, 16, 70), (32, 8, 128, 16, None)])
@pytest.mark.parametrize("lengths", [(1, 129, 700, 64, 257, 1000), (3000,), tuple(range(60, 100))])
def test_decode_attention_of_single_tokens(n_q, n_kv, d, page, window, lengths):
    """The tensor-core kernel for decoded tokens: one row per request, contexts from 1 to 3,000
    keys, 1 to 40 rows (so from 55 blocks per (row, kv head) down to one), twice in a row with
    the same counters, which are zero again afterwards."""
    assert ops.decode_attention_takes(torch.bfloat16, n_q, n_kv, d)
    assert not ops.decode_attention_takes(torch.float32, n_q, n_kv, d)
    assert not ops.decode_attention_takes(torch.bfloat16, n_q, n_kv, 48)
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, lengths, (1,) * len(lengths), window, seed=d + len(lengths))
    scale = 1.0 / math.sqrt(d)
    want = expected_attention(case, scale)
    counters = torch.zeros(len(lengths) * n_kv, dtype=torch.int32, device=DEV)
    first = run_decode(case, scale, counters)
    assert int(counters.abs().sum()) == 0
    second = run_decode(case, scale, counters)
    assert int(counters.abs().sum()) == 0
    assert torch.equal(first, second)
    close(first, want, torch.bfloat16, "decode attention")


@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(32, 8, 128, 16, None), (12, 6, 64, 8, 500), (16, 1, 128, 32, None)])
@pytest.mark.parametrize("splits", [1, 2, 5, 13])
def test_decode_attention_with_more_blocks_than_run_at_once(n_q, n_kv, d, page, window, splits, monkeypatch):
    """Many rows of very different lengths, cut into several times more blocks than run at once: the
    same result whatever the number of blocks per row, twice in a row with the same counters, which
    are zero again afterwards."""
    rows = 1400 // (n_kv * splits) + 7
    lengths = tuple(1 + (37 * i * i + 11 * i) % 1500 for i in range(rows))
    assert rows * n_kv * splits > 3 * ops.sm_count()
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, lengths, (1,) * rows, window, seed=rows)
    scale = 1.0 / math.sqrt(d)
    monkeypatch.setattr(ops, "decode_splits", lambda *a, **k: splits)
    counters = torch.zeros(rows * n_kv, dtype=torch.int32, device=DEV)
    first = run_decode(case, scale, counters, max_keys=max(lengths))
    assert int(counters.abs().sum()) == 0
    second = run_decode(case, scale, counters, max_keys=max(lengths))
    assert int(counters.abs().sum()) == 0
    assert torch.equal(first, second)
    close(first, expected_attention(case, scale), torch.bfloat16, "decode attention, several waves of blocks")


def test_decode_attention_finds_a_far_key_and_respects_the_window_edge():
    case = paged_case(torch.bfloat16, 4, 2, 64, 16, (700, 530), (1, 1), None, seed=9, boost=(17, 3.0))
    scale = 1.0 / 8.0
    counters = torch.zeros(16, dtype=torch.int32, device=DEV)
    out = run_decode(case, scale, counters)
    close(out, expected_attention(case, scale), torch.bfloat16, "far key")
    v_far = rounded(case["vs"][0][17], torch.bfloat16)
    for h in (0, 2):
        assert float((out[0, h].double().cpu() - v_far[h // 2]).abs().max()) < 0.05
    window, n = 24, 100
    for which, visible in ((n - window - 1, False), (n - window, True)):
        case = paged_case(torch.bfloat16, 2, 1, 64, 8, (n,), (1,), window, seed=4, boost=(which, 4.0))
        out = run_decode(case, scale, counters)
        close(out, expected_attention(case, scale), torch.bfloat16, f"window edge key {which}")
        near = float((out[0, 0].double().cpu() - rounded(case["vs"][0][which, 0], torch.bfloat16)).abs().max()) < 0.05
        assert near == visible


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(4, 2, 16, 16, None), (6, 3, 32, 8, None), (5, 1, 48, 16, 37),
                                                    (8, 8, 64, 4, None), (16, 2, 128, 32, 100), (3, 1, 272, 16, None),
                                                    (6, 2, 40, 16, None), (3, 3, 18, 8, 50), (2, 1, 510, 16, None)])
@pytest.mark.parametrize("split", [0, 32, 128, 256])
def test_paged_attention(dtype, n_q, n_kv, d, page, window, split):
    lengths, rows = (1, 33, 300, 64, 257), (1, 5, 2, 64, 1)
    case = paged_case(dtype, n_q, n_kv, d, page, lengths, rows, window, seed=d + page)
    scale = 0.7 / math.sqrt(d)
    close(run_attention(case, scale, split), expected_attention(case, scale), dtype, "attention")


def tiles_of(case, tile_rows=64):
    tiles, first = [], 0
    for r, (n, rows) in enumerate(zip(case["lengths"], case["rows"])):
        for begin in range(0, rows, tile_rows):
            tiles.append([first + begin, min(tile_rows, rows - begin), r, n - rows + begin])
        first += rows
    return torch.tensor(tiles, dtype=torch.int32, device=DEV)


def run_tiled(case, scale, tensor_memory=False):
    out = torch.full_like(case["q"], float("nan"))
    word = ops.new_error_word(DEV)
    if tensor_memory:
        ops.tiled_attention_tc(case["q"], case["k_pool"], case["v_pool"], out, tiles_of(case, 128), case["table"],
                               scale=scale, window=case["window"] or 0, error_word=word)
    else:
        ops.tiled_attention(case["q"], case["k_pool"], case["v_pool"], out, tiles_of(case), case["table"], scale=scale,
                            window=case["window"] or 0, error_word=word)
    ops.raise_on_error_word(word)
    return out


@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(4, 2, 64, 16, None), (6, 3, 128, 8, None), (16, 2, 128, 32, 100),
                                                    (5, 1, 64, 16, 37), (3, 3, 128, 64, 64), (32, 8, 128, 16, None)])
def test_tcgen05_attention_of_prompt_portions(n_q, n_kv, d, page, window):
    """The tensor-memory kernel: portions of 1 to 300 rows at the end of sequences of up to 700 keys."""
    assert ops.tiled_attention_tc_takes(torch.bfloat16, n_q, n_kv, d, page)
    assert not ops.tiled_attention_tc_takes(torch.bfloat16, n_q, n_kv, d, 4)
    assert not ops.tiled_attention_tc_takes(torch.float32, n_q, n_kv, d, page)
    lengths, rows = (1, 33, 300, 64, 257, 191, 700), (1, 5, 130, 64, 70, 191, 300)
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, lengths, rows, window, seed=3 * d + page)
    scale = 0.9 / math.sqrt(d)
    close(run_tiled(case, scale, tensor_memory=True), expected_attention(case, scale), torch.bfloat16, "tcgen05 attention")


@pytest.mark.parametrize("n_q,n_kv,d,page", [(4, 2, 128, 16), (3, 1, 64, 8)])
def test_tcgen05_attention_with_maxima_that_keep_jumping(n_q, n_kv, d, page):
    """Scores thirty times as wide as usual: a row's maximum jumps by far more than 2^8 from one
    64-key block to the next, so the output in tensor memory is rescaled in many blocks, each time
    after the product of the block before has landed (the kernel computes S of the next block
    while it waits)."""
    lengths, rows = (900, 260, 1500), (300, 260, 129)
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, lengths, rows, None, seed=d + page)
    scale = 30.0 / math.sqrt(d)
    close(run_tiled(case, scale, tensor_memory=True), expected_attention(case, scale), torch.bfloat16, "jumping maxima")


def test_tcgen05_attention_finds_a_far_key_and_respects_the_window_edge():
    case = paged_case(torch.bfloat16, 4, 2, 64, 16, (700, 530), (70, 3), None, seed=9, boost=(17, 3.0))
    scale = 1.0 / 8.0
    out = run_tiled(case, scale, tensor_memory=True)
    close(out, expected_attention(case, scale), torch.bfloat16, "far key")
    v_far = rounded(case["vs"][0][17], torch.bfloat16)
    for h in (0, 2):
        assert float((out[69, h].double().cpu() - v_far[h // 2]).abs().max()) < 0.05
    window, n = 24, 100
    for which, visible in ((n - window - 1, False), (n - window, True)):
        case = paged_case(torch.bfloat16, 2, 1, 64, 8, (n,), (5,), window, seed=4, boost=(which, 4.0))
        out = run_tiled(case, scale, tensor_memory=True)
        close(out, expected_attention(case, scale), torch.bfloat16, f"window edge key {which}")
        near = float((out[4, 0].double().cpu() - rounded(case["vs"][0][which, 0], torch.bfloat16)).abs().max()) < 0.05
        assert near == visible


@pytest.mark.parametrize("n_q,n_kv,d,page,window", [(4, 2, 64, 16, None), (6, 3, 128, 8, None), (16, 2, 128, 32, 100),
                                                    (5, 1, 64, 16, 37), (3, 3, 128, 4, 64)])
def test_tiled_attention_of_prompt_portions(n_q, n_kv, d, page, window):
    """Portions of 1 to 130 rows at the end of sequences of up to 300 keys, tiles that end in
    the middle of a key block, windows that start in the middle of one."""
    assert ops.tiled_attention_takes(torch.bfloat16, n_q, n_kv, d)
    assert not ops.tiled_attention_takes(torch.float32, n_q, n_kv, d)
    assert not ops.tiled_attention_takes(torch.bfloat16, n_q, n_kv, 48)
    lengths, rows = (1, 33, 300, 64, 257, 191), (1, 5, 130, 64, 70, 191)
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, lengths, rows, window, seed=3 * d + page)
    scale = 0.9 / math.sqrt(d)
    close(run_tiled(case, scale), expected_attention(case, scale), torch.bfloat16, "tiled attention")


def test_tiled_attention_finds_a_far_key_and_respects_the_window_edge():
    n_q, n_kv, d, page = 4, 2, 64, 16
    case = paged_case(torch.bfloat16, n_q, n_kv, d, page, (700, 530), (70, 3), None, seed=9, boost=(17, 3.0))
    scale = 1.0 / math.sqrt(d)
    out = run_tiled(case, scale)
    close(out, expected_attention(case, scale), torch.bfloat16, "far key")
    v_far = rounded(case["vs"][0][17], torch.bfloat16)
    for h in (0, 2):
        assert float((out[69, h].double().cpu() - v_far[h // 2]).abs().max()) < 0.05
    window, n = 24, 100
    for which, visible in ((n - window - 1, False), (n - window, True)):
        case = paged_case(torch.bfloat16, 2, 1, 64, 8, (n,), (5,), window, seed=4, boost=(which, 4.0))
        out = run_tiled(case, 1.0 / 8.0)
        close(out, expected_attention(case, 1.0 / 8.0), torch.bfloat16, f"window edge key {which}")
        near = float((out[4, 0].double().cpu() - rounded(case["vs"][0][which, 0], torch.bfloat16)).abs().max()) < 0.05
        assert near == visible


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("split", [0, 128])
def test_a_far_key_among_hundreds_is_found(dtype, split):
    """One key far back gets a score that dominates; leaving it out, or reading a stale page
    in its place, would change the output completely."""
    n_q, n_kv, d, page = 4, 2, 64, 16
    case = paged_case(dtype, n_q, n_kv, d, page, (700, 530), (1, 3), None, seed=9, boost=(17, 3.0))
    scale = 1.0 / math.sqrt(d)
    out = run_attention(case, scale, split)
    close(out, expected_attention(case, scale), dtype, "far key")
    # the last row of the first request is, within rounding, the boosted key's value
    v_far = rounded(case["vs"][0][17], dtype)               # [n_kv, d]
    got = out[0].double().cpu()                             # row 0 = request 0's only row, [n_q, d]
    for h in (0, 2):                                        # the query heads the key was aligned with
        assert float((got[h] - v_far[h // 2]).abs().max()) < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edge(dtype):
    """The key just outside the window is boosted: it must not be seen; the one just inside is."""
    n_q, n_kv, d, page, window = 2, 1, 32, 8, 24
    n = 100
    for which, visible in ((n - window - 1, False), (n - window, True)):
        case = paged_case(dtype, n_q, n_kv, d, page, (n,), (1,), window, seed=4, boost=(which, 4.0))
        out = run_attention(case, 1.0 / math.sqrt(d), 0)
        close(out, expected_attention(case, 1.0 / math.sqrt(d)), dtype, f"window edge key {which}")
        near = float((out[0, 0].double().cpu() - rounded(case["vs"][0][which, 0], dtype)).abs().max()) < 0.05
        assert near == visible


def test_attention_refuses_sizes_it_cannot_take():
    case = paged_case(torch.float32, 4, 2, 16, 16, (5,), (1,), None, seed=0)
    bad_q = torch.zeros(1, 4, 24, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.paged_attention(bad_q, case["k_pool"], case["v_pool"], torch.empty_like(bad_q), case["positions"],
                            case["row_request"], case["table"], scale=1.0, window=0, split_size=0, max_splits=1,
                            scratch_acc=None, scratch_ml=None, error_word=ops.new_error_word(DEV))
    pool = torch.zeros(4, 1, 16, 520, device=DEV)
    q = torch.zeros(1, 2, 520, device=DEV)
    with pytest.raises(ops.KernelError, match="at most 512"):
        ops.paged_attention(q, pool, pool, torch.empty_like(q), case["positions"], case["row_request"], case["table"],
                            scale=1.0, window=0, split_size=0, max_splits=1, scratch_acc=None, scratch_ml=None,
                            error_word=ops.new_error_word(DEV))
    pool = torch.zeros(4, 1, 16, 16, device=DEV)
    q = torch.zeros(1, 40, 16, device=DEV)
    with pytest.raises(ops.KernelError, match="exceed 32"):
        ops.paged_attention(q, pool, pool, torch.empty_like(q), case["positions"], case["row_request"], case["table"],
                            scale=1.0, window=0, split_size=0, max_splits=1, scratch_acc=None, scratch_ml=None,
                            error_word=ops.new_error_word(DEV))


def test_sampling_kernel():
    g = torch.Generator().manual_seed(3)
    vocab = 1531
    logits = torch.randn(6, vocab, generator=g) * 3
    logits[2, 100] = logits[2, 900] = 50.0                 # equal maxima: the lowest index wins
    picked = ops.sample(logits.to(DEV), None, None).cpu()
    assert picked.tolist() == [pm.plain_argmax(row) for row in logits]
    assert picked[2] == 100
    temperature = torch.tensor([0.7, 1.0, 0.0, 1.5, 0.3, 1.0])
    for trial in range(20):
        u = torch.rand(6, generator=g)
        got = ops.sample(logits.to(DEV), temperature.to(DEV), u.to(DEV)).cpu().tolist()
        for r in range(6):
            if temperature[r] <= 0:
                assert got[r] == pm.plain_argmax(logits[r])
                continue
            want = pm.plain_temperature_sample(logits[r], float(temperature[r]), float(u[r]))
            if got[r] != want:
                # only a tie of the running sum at 32-bit rounding may move the pick by one place
                p = torch.softmax(logits[r].double() / float(temperature[r]), 0)
                edge = float(torch.cumsum(p, 0)[min(got[r], want)])
                assert abs(got[r] - want) == 1 and abs(edge - float(u[r])) < 1e-5, (r, got[r], want)
    # u at the ends
    ends = ops.sample(logits[:1].to(DEV), torch.tensor([1.0], device=DEV), torch.tensor([0.0], device=DEV))
    assert int(ends[0]) == 0
    last = ops.sample(logits[:1].to(DEV), torch.tensor([1.0], device=DEV), torch.tensor([0.99999994], device=DEV))
    assert int(last[0]) >= vocab - 50


def plain_filtered_pick(kept, u):
    """The reference's walk over the kept items in sorted order (model_executor.rs:532-555), in 64-bit;
    also how far u * mass lies from the nearest edge between two items, as a fraction of the mass."""
    tokens, masses = list(kept), list(kept.values())
    total = sum(masses)
    target, running, pick, gap = u * total, 0.0, tokens[-1], 1.0
    found = False
    for token, mass in zip(tokens, masses):
        running += mass
        gap = min(gap, abs(running - target) / total)
        if not found and running > target:
            pick, found = token, True
    return pick, tokens, gap


@pytest.mark.parametrize("vocab", [1531, 20011])
def test_sampling_with_top_k_top_p_and_min_p(vocab):
    """The kernel that samples with cuts against the reference's algorithm: peaked and flat rows, equal
    logits at the edge of a cut (index order decides), cuts alone and together, u at both ends."""
    g = torch.Generator().manual_seed(vocab)
    rows = 8
    logits = torch.randn(rows, vocab, generator=g) * 4
    logits[1] = torch.randn(vocab, generator=g) * 0.01                     # nearly flat
    logits[2] = 0.0                                                        # all equal: index order only
    logits[3, [5, 77, 300, 900]] = 9.0                                     # four equal maxima
    logits[4, [10, 20, 30]] = logits[4].max() - 1.0                        # equal values below the maximum
    logits[5] = torch.round(logits[5])                                     # many ties everywhere
    cases = [dict(top_k=1), dict(top_k=3), dict(top_k=50), dict(top_p=0.9), dict(top_p=1e-6), dict(top_p=0.3),
             dict(min_p=0.5), dict(min_p=0.01), dict(top_k=40, top_p=0.83, min_p=0.02), dict(top_k=vocab - 1),
             dict(top_k=2, top_p=0.999)]
    temperature = torch.tensor([0.7, 1.0, 1.0, 0.5, 1.3, 2.0, 0.9, 1.0])
    logits_d = logits.to(DEV)
    out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    for case in cases:
        k = torch.full((rows,), case.get("top_k", 0), dtype=torch.int32)
        tp = torch.full((rows,), case.get("top_p", 1.0))
        mp = torch.full((rows,), case.get("min_p", 0.0))
        kept_of = [pm.plain_filtered_distribution(logits[r], float(temperature[r]), case.get("top_k"), case.get("top_p"),
                                                  case.get("min_p")) for r in range(rows)]
        for trial in range(6 if vocab < 5000 else 3):
            u = torch.rand(rows, generator=g)
            if trial == 0:
                u[:] = 0.0
            if trial == 1:
                u[:] = 0.99999994
            out.fill_(-1)
            ops.sample_filtered(logits_d, None, temperature.to(DEV), k.to(DEV), tp.to(DEV), mp.to(DEV), u.to(DEV), out)
            got = out.cpu().tolist()
            for r in range(rows):
                want, kept, gap = plain_filtered_pick(kept_of[r], float(u[r]))
                if got[r] != want:
                    # The kernel has 32-bit exponentials, the oracle 64-bit ones.  That may move a u within
                    # rounding of an edge between two items to the other item, and it may order two items
                    # of nearly equal probability the other way round; nothing else.
                    scaled = logits[r].double() / float(temperature[r])
                    p_got, p_want = math.exp(float(scaled[got[r]] - scaled.max())), math.exp(float(scaled[want] - scaled.max()))
                    nearly_equal = abs(p_got - p_want) <= 1e-5 * p_want
                    assert gap < 1e-5 or float(u[r]) > 0.9999 or nearly_equal, (case, r, got[r], want, gap)
                    p_last = math.exp(float(scaled[kept[-1]] - scaled.max()))
                    assert got[r] in kept or abs(p_got - p_last) <= 1e-5 * p_last, (case, r, got[r])
    # only the rows that are named are written
    out.fill_(-1)
    index = torch.tensor([6, 2], dtype=torch.int32, device=DEV)
    ones = torch.ones(rows)
    ops.sample_filtered(logits_d, index, temperature.to(DEV), torch.full((rows,), 5, dtype=torch.int32, device=DEV),
                        ones.to(DEV), torch.zeros(rows, device=DEV), torch.full((rows,), 0.5, device=DEV), out)
    got = out.cpu().tolist()
    assert [i for i, t in enumerate(got) if t >= 0] == [2, 6]
    assert got[2] == 2                                                     # five equal items, u = 0.5: the third by index


def test_penalties_from_counts_on_the_device():
    """Counts of seen tokens per request (prompt counted once, sampled tokens as they are chosen) and the
    reference's penalties applied from them, against the plain implementation."""
    g = torch.Generator().manual_seed(5)
    vocab, rows = 777, 4
    counts = torch.zeros(3, vocab, dtype=torch.int32, device=DEV)
    prompts = {0: [5, 5, 9, 700, 5], 2: [1, 2, 3, 2]}
    for table_row, prompt in prompts.items():
        ops.count_tokens(counts[table_row], torch.tensor(prompt, dtype=torch.int32, device=DEV))
    index = torch.tensor([2, -1, 0, -1], dtype=torch.int32, device=DEV)       # logits row -> row of counts
    picked = torch.tensor([3, 8, 776, 5], dtype=torch.int32, device=DEV)
    ops.count_picked(counts, index, picked)
    seen = {0: prompts[2] + [3], 2: prompts[0] + [776]}                       # by logits row
    want_counts = torch.zeros(3, vocab, dtype=torch.int32)
    for t in prompts[0] + [776]:
        want_counts[0, t] += 1
    for t in prompts[2] + [3]:
        want_counts[2, t] += 1
    assert torch.equal(counts.cpu(), want_counts)
    logits = torch.randn(rows, vocab, generator=g) * 3
    presence = torch.tensor([0.25, 9.0, -0.5, 9.0])
    frequency = torch.tensor([0.5, 9.0, 0.3, 9.0])
    repetition = torch.tensor([2.0, 9.0, 1.0, 9.0])
    got = logits.to(DEV)
    ops.apply_penalties(got, counts, index, presence.to(DEV), frequency.to(DEV), repetition.to(DEV))
    for r in range(rows):
        if r in seen:
            want = pm.plain_apply_penalties(logits[r], seen[r], frequency=float(frequency[r]), presence=float(presence[r]),
                                            repetition=float(repetition[r]))
        else:
            want = logits[r]
        assert torch.allclose(got[r].cpu().double(), want.double(), atol=1e-6), r
