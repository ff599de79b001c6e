"""Each kernel alone against a plain torch reference in 64-bit, at sizes other than the engine's.
Inputs are built so that faults would show: a far key that dominates, a window's edge, scrambled
pages, widths and vocabularies that are no power of two."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from lia_rs_b200.kernels import ops as o
    return o


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.6e-2       # bfloat16: 2 units of 2^-8 relative on O(1) values


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_scales_rows_and_flags_bad_ids(dtype):
    table = torch.randn(301, 72, device=DEV).to(dtype)
    tokens = torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embedding(tokens, table, out, 12.0, flag)
    assert torch.equal(out, table[tokens.long()].float() * 12.0) and flag.item() == 0
    ops().embedding(torch.tensor([3, 301], dtype=torch.int32, device=DEV), table, out[:2], 1.0, flag)
    assert flag.item() == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("w_dtype", DTYPES)
@pytest.mark.parametrize("hidden", [48, 1000, 2048, 4100])
def test_rmsnorm(hidden, w_dtype, out_dtype):
    x = torch.randn(7, hidden, device=DEV) * 3
    w = (torch.rand(hidden, device=DEV) + 0.5).to(w_dtype)
    out = torch.empty(7, hidden, device=DEV, dtype=out_dtype)
    ops().rmsnorm(x, w, out, 1e-5, 0.5)
    xd = x.double()
    want = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * w.double() * 0.5
    assert float((out.double() - want).abs().max()) <= tol(out_dtype) * float(want.abs().max())
    rows = torch.tensor([6, -1, 0], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, hidden, device=DEV, dtype=out_dtype)
    ops().rmsnorm(x, w, picked, 1e-5, 0.5, rows)
    assert torch.equal(picked[0], out[6]) and torch.equal(picked[2], out[0]) and float(picked[1].abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 40, 24), (5, 130, 100), (67, 64, 257), (130, 301, 72)])
def test_gemm_simt_all_epilogues(M, N, K, dtype):
    o = ops()
    a = torch.randn(M, K, device=DEV).to(dtype)
    w = torch.randn(2 * N, K, device=DEV).to(dtype) / math.sqrt(K)
    exact = a.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    o.gemm_simt(o.GEMM_STORE, a, w[:N], out, 0.25)
    assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * max(1.0, float(exact.abs().max()))
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    o.gemm_simt(o.GEMM_ACCUM, a, w[:N], acc, 1.5)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5
    act = torch.empty(M, N, device=DEV, dtype=dtype)
    o.gemm_simt(o.GEMM_SWIGLU, a, w, act)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= tol(dtype) * max(1.0, float(want.abs().max()))
    # a row's result does not depend on the other rows of the batch
    alone = torch.empty(1, N, device=DEV)
    o.gemm_simt(o.GEMM_STORE, a[M - 1:M].contiguous(), w[:N], alone, 0.25)
    assert torch.equal(alone[0], out[M - 1])


def paged(values, page_size, num_pages, order):
    """Scatter [T, heads, d] into pages in the given physical order; returns pages and the table."""
    T = values.shape[0]
    pages = torch.zeros(num_pages, page_size, *values.shape[1:], dtype=values.dtype, device=DEV)
    blocks = (T + page_size - 1) // page_size
    table = torch.full((blocks,), -1, dtype=torch.int32)
    for b in range(blocks):
        table[b] = order[b]
        chunk = values[b * page_size:(b + 1) * page_size]
        pages[order[b], :chunk.shape[0]] = chunk
    return pages, table


def reference_attention(q, k, v, positions, window, scale):
    out = torch.zeros_like(q, dtype=torch.float64)
    g = q.shape[1] // k.shape[1]
    for t, pos in enumerate(positions):
        first = 0 if not window else max(0, pos - window + 1)
        for h in range(q.shape[1]):
            s = (k[first:pos + 1, h // g].double() @ q[t, h].double()) * scale
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[first:pos + 1, h // g].double()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,nq,nkv,page_size,window", [(16, 4, 2, 8, None), (48, 6, 3, 4, 21), (128, 8, 1, 16, None),
                                                       (80, 5, 5, 32, 100), (256, 2, 1, 16, None)])
def test_attention_generic_far_key_window_edge_and_scrambled_pages(d, nq, nkv, page_size, window, dtype):
    torch.manual_seed(d)
    T = 333
    k = torch.randn(T, nkv, d, device=DEV) * 0.3
    v = torch.randn(T, nkv, d, device=DEV)
    positions = [0, 1, page_size - 1, page_size, 2 * page_size + 1, 200, 331, 332]
    q = torch.randn(len(positions), nq, d, device=DEV) * 0.3
    # one far key stands out for the last query: key 5 (or the window's first key) carries the score
    far = 5 if not window else 332 - window + 1
    k[far, :, :] = 0
    k[far, :, 0] = 6.0
    q[-1, :, 0] = 5.0 * math.sqrt(d)
    # and the key just outside the window would dominate if it were seen
    if window:
        k[far - 1, :, 1] = 50.0
        q[-1, :, 1] = 5.0 * math.sqrt(d)
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    num_pages = 2 * ((T + page_size - 1) // page_size) + 3
    order = np.random.default_rng(0).permutation(num_pages)[:(T + page_size - 1) // page_size]
    kp, table = paged(k, page_size, num_pages, order)
    vp, _ = paged(v, page_size, num_pages, order)
    bt = torch.full((3, table.numel() + 2), -1, dtype=torch.int32)
    bt[1, :table.numel()] = table                                        # the request sits in slot 1
    out = torch.empty_like(q)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots = torch.ones(len(positions), dtype=torch.int32, device=DEV)
    slots[3] = -1                                                        # padding row: left alone
    out[3] = 7.0
    scale = 1 / math.sqrt(d)
    ops().attention_generic(q.view(-1, nq * d), kp, vp, pos, slots, bt.to(DEV), out.view(-1, nq * d), nq, nkv, d,
                            window, scale)
    want = reference_attention(q, k, v, positions, window, scale)
    keep = [i for i in range(len(positions)) if i != 3]
    error = float((out.double()[keep] - want[keep]).abs().max())
    assert error <= tol(dtype) * max(1.0, float(want.abs().max())), error
    assert float((out[3].float() - 7.0).abs().max()) == 0
    # the last query's output is the far key's value, almost alone
    assert float((out[-1, 0].double() - v[far, 0].double()).abs().max()) < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,rotary_dim", [(16, 16), (48, 48), (64, 32), (128, 128), (32, 0)])
def test_rope_kv_write(d, rotary_dim, dtype):
    nq, nkv, page_size, theta = 3, 2, 4, 50000.0
    positions = [0, 1, 3, 4, 7, 8, 1000, 30000]
    n = len(positions)
    qkv = torch.randn(n, (nq + 2 * nkv) * d, device=DEV)
    blocks = max(positions) // page_size + 1
    table = torch.full((2, blocks), -1, dtype=torch.int32)
    for i, pos in enumerate(positions):
        if table[1, pos // page_size] < 0:
            table[1, pos // page_size] = 10 - i                          # pages out of order
    kp = torch.zeros(12, page_size, nkv, d, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    q_out = torch.zeros(n, nq * d, device=DEV, dtype=dtype)
    inv = None
    if rotary_dim:
        inv = (1.0 / theta ** (2.0 * torch.arange(rotary_dim // 2, dtype=torch.float64) / rotary_dim)).float().to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().rope_kv_write(qkv, torch.tensor(positions, dtype=torch.int32, device=DEV),
                        torch.ones(n, dtype=torch.int32, device=DEV), table.to(DEV), q_out, kp, vp, nq, nkv, d,
                        rotary_dim, inv, True, flag)
    assert flag.item() == 0
    x = qkv.double().view(n, nq + 2 * nkv, d)
    rotated = x.clone()
    if rotary_dim:
        half = rotary_dim // 2
        angle = torch.tensor(positions, dtype=torch.float64, device=DEV)[:, None] * inv.double()[None, :]
        c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        a, b = x[..., :half], x[..., half:rotary_dim]
        rotated[..., :half] = a * c - b * s
        rotated[..., half:rotary_dim] = b * c + a * s
    limit = 1e-5 * 4 if dtype == torch.float32 else 2.0 ** -8 * 4
    # 32-bit angles: at position 30000 the product pos * inv_freq is rounded to 2^-24 relative
    limit += 30000 * 2.0 ** -23 * 4
    assert float((q_out.double().view(n, nq, d) - rotated[:, :nq]).abs().max()) < limit
    for i, pos in enumerate(positions):
        page = int(table[1, pos // page_size])
        assert float((kp[page, pos % page_size].double() - rotated[i, nq:nq + nkv]).abs().max()) < limit
        assert float((vp[page, pos % page_size].double() - x[i, nq + nkv:]).abs().max()) < limit
    # a position whose block has no page raises the flag and writes nothing
    ops().rope_kv_write(qkv[:1], torch.tensor([8 * page_size], dtype=torch.int32, device=DEV),
                        torch.zeros(1, dtype=torch.int32, device=DEV), table.to(DEV), q_out[:1], kp, vp, nq, nkv, d,
                        rotary_dim, inv, True, flag)
    assert flag.item() == 2


def test_select_tokens_greedy_ties_and_gumbel_matches_the_host_rule():
    from lia_rs_b200.sampling import RequestSampler, Sampling
    vocab = 73448 // 8 + 3
    logits = torch.randn(6, vocab, device=DEV)
    logits[0, [5, 900, 4000]] = 9.0                   # equal maxima: the largest id wins
    logits[1, vocab - 1] = 11.0
    logits[2, 0] = 11.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops().select_tokens(logits, out)
    assert out.tolist()[:3] == [4000, vocab - 1, 0]
    assert out.tolist() == [RequestSampler(Sampling()).sample(row, 0) for row in logits.cpu().numpy()]
    temperature = torch.tensor([0.7, 1.0, 0.0, 1.5, 0.3, 1.0], device=DEV)
    seeds = torch.tensor([1, 2, 3, 2 ** 40 + 5, 5, 6], dtype=torch.int64, device=DEV)
    positions = torch.tensor([0, 17, 5, 123456, 9, 2 ** 33], dtype=torch.int64, device=DEV)
    ops().select_tokens(logits, out, temperature, seeds, positions)
    host = []
    for i, row in enumerate(logits.cpu().numpy()):
        s = Sampling(temperature=float(temperature[i]), seed=int(seeds[i]), sampler="murmur3_gumbel")
        host.append(RequestSampler(s).sample(row, int(positions[i])))
    assert out.tolist() == host
    # frequencies follow softmax(logits / T)
    small = torch.tensor([[0.0, math.log(2.0), math.log(5.0)]], device=DEV).repeat(4000, 1).contiguous()
    picks = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops().select_tokens(small, picks, torch.ones(4000, device=DEV), torch.full((4000,), 9, dtype=torch.int64, device=DEV),
                        torch.arange(4000, dtype=torch.int64, device=DEV))
    freq = torch.bincount(picks.long(), minlength=3).double() / 4000
    assert torch.allclose(freq.cpu(), torch.tensor([1 / 8, 2 / 8, 5 / 8], dtype=torch.float64), atol=0.03)


@pytest.mark.parametrize("rows,vocab,k", [(1, 300, 1), (3, 300, 20), (8, 73448, 20), (5, 5000, 32), (9, 2049, 7), (2, 40, 32)])
def test_select_candidates_are_the_best_of_every_row_in_the_sampling_rules_order(rows, vocab, k):
    """The best k logits of a row, larger logit first and among equal ones the larger id; minus infinity is no
    candidate; NaN and infinities are counted."""
    import numpy as np
    torch.manual_seed(rows + vocab + k)
    logits = torch.randn(rows, vocab, device=DEV)
    logits[:, ::7] = logits[:, 3:4]                       # many equal values, across the ranges a row is cut into
    logits[0, : vocab // 2] = float("-inf")
    if rows > 1:
        logits[1, 5:] = float("-inf")                     # fewer candidates than asked for
    values = torch.empty(rows, k, device=DEV)
    ids = torch.empty(rows, k, dtype=torch.int32, device=DEV)
    odd = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().select_candidates(logits, k, values, ids, odd)
    host = logits.cpu().numpy()
    for r in range(rows):
        finite = np.nonzero(~np.isneginf(host[r]))[0]
        order = np.lexsort((-finite, -host[r][finite].astype(np.float64)))
        want = finite[order][:k]
        got = ids[r].cpu().numpy()
        assert list(got[:want.size]) == list(want), r
        assert (got[want.size:] == -1).all()
        assert np.array_equal(values[r].cpu().numpy()[:want.size], host[r][want])
    assert odd.item() == int(np.isinf(host).sum())
    # with temperatures: also each row's largest logit and its whole softmax mass in 64-bit
    temperature = torch.tensor([0.0 if r == 2 else 0.3 + 0.45 * r for r in range(rows)], dtype=torch.float64, device=DEV)
    mass = torch.full((rows, 2), -1.0, dtype=torch.float64, device=DEV)
    again = torch.empty_like(ids)
    ops().select_candidates(logits, k, values, again, odd, temperature, mass)
    assert torch.equal(again, ids)
    for r in range(rows):
        finite = host[r][~np.isneginf(host[r])].astype(np.float64)
        assert mass[r, 0].item() == finite.max()
        t = temperature[r].item()
        want = np.exp((finite - finite.max()) / t).sum() if t else 0.0
        assert abs(mass[r, 1].item() - want) <= 1e-12 * max(want, 1.0), (r, mass[r, 1].item(), want)
    odd.zero_()
    ops().select_candidates(logits, k, values, ids, odd)
    logits[rows - 1, 2] = float("nan")
    ops().select_candidates(logits, k, values, ids, odd)                     # the counter adds up over calls
    assert odd.item() == int(np.isinf(host).sum()) + int((~np.isfinite(logits.cpu().numpy())).sum())


@pytest.mark.parametrize("M", [1, 8, 40, 64, 100, 300, 1000])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 200), (2560, 2048), (1000, 6144), (384, 96), (15000, 520)])
def test_gemm_tc_all_epilogues_against_64_bit(M, N, K):
    """The tcgen05 product at sizes that are no multiple of its tiles, with and without split K."""
    o = ops()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert o.gemm_tc_accepts(o.GEMM_STORE, a, w, torch.empty(M, N, device=DEV))
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    out = torch.full((M, N), 7.0, device=DEV)
    o.gemm_tc(o.GEMM_STORE, a, w[:N], out, 0.25, flag)
    assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(K / 64)
    half = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_tc(o.GEMM_STORE, a, w[:N], half, 1.0, flag)
    assert float((half.double() - exact[:, :N]).abs().max()) <= 2.0 ** -8 * scale
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    o.gemm_tc(o.GEMM_ACCUM, a, w[:N], acc, 1.5, flag)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(K / 64)
    act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_tc(o.GEMM_SWIGLU, a, w, act, 1.0, flag)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert flag.item() == 0


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 2048), (1999, 2700, 520), (4096, 1280, 1024), (2048, 6144, 2048), (777, 12288, 256),
                                   (1500, 2048, 64), (3000, 3000, 200)])
def test_gemm_tc_many_tokens_tile_widths(M, N, K):
    """Products with more tiles than SMs: the tile width is chosen to fill the rounds (160, 192, 224 tokens
    as well as 128 and 256), the last tile of tokens and of features is partial."""
    o = ops()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    out = torch.full((M, N), 7.0, device=DEV)
    o.gemm_tc(o.GEMM_STORE, a, w[:N], out, 0.25, flag)
    assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(K / 64)
    half = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_tc(o.GEMM_STORE, a, w[:N], half, 1.0, flag)
    assert float((half.double() - exact[:, :N]).abs().max()) <= 2.0 ** -8 * scale
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    o.gemm_tc(o.GEMM_ACCUM, a, w[:N], acc, 1.5, flag)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(K / 64)
    act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_tc(o.GEMM_SWIGLU, a, w, act, 1.0, flag)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert flag.item() == 0


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(40, 64), (200, 200), (2560, 2048), (1000, 6144), (384, 96), (77, 16384), (301, 7000)])
def test_gemm_skinny_all_epilogues_against_64_bit(M, N, K):
    """The few-token product: widths that are no multiple of its 16 rows, K shorter than a chunk, K that
    ends inside a group of 32, and K long enough that the ring of stages is used again."""
    o = ops()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert o.gemm_skinny_accepts(o.GEMM_STORE, a, w, torch.empty(M, N, device=DEV))
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    out = torch.full((M, N), 7.0, device=DEV)
    o.gemm_skinny(o.GEMM_STORE, a, w[:N], out, 0.25, flag)
    assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(K / 64)
    half = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_skinny(o.GEMM_STORE, a, w[:N], half, 1.0, flag)
    assert float((half.double() - exact[:, :N]).abs().max()) <= 2.0 ** -8 * scale
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    o.gemm_skinny(o.GEMM_ACCUM, a, w[:N], acc, 1.5, flag)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(K / 64)
    act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_skinny(o.GEMM_SWIGLU, a, w, act, 1.0, flag)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    # a token's result does not depend on how many other tokens are in the batch
    alone = torch.empty(1, N, device=DEV)
    o.gemm_skinny(o.GEMM_STORE, a[M - 1:M].contiguous(), w[:N], alone, 0.25, flag)
    assert torch.equal(alone[0], out[M - 1])
    torch.cuda.synchronize()
    assert flag.item() == 0
    with pytest.raises(o.KernelError, match="refuses"):
        o.gemm_skinny(o.GEMM_STORE, torch.zeros(33, K, device=DEV, dtype=torch.bfloat16), w[:N], torch.empty(33, N, device=DEV))


@pytest.mark.parametrize("M", [1, 5, 8, 9, 13, 16])
@pytest.mark.parametrize("N,K", [(40, 64), (200, 192), (2560, 2048), (1000, 6144), (384, 1024), (520, 4096), (77, 8192), (301, 7040),
                                 (6144, 2048), (24, 2112)])
def test_gemm_stream_all_epilogues_against_64_bit(M, N, K):
    """The persistent few-token product: widths that are no multiple of its 16 rows, the forms that keep the
    tokens' rows in registers (K 1,024, 2,048, 4,096, 6,144) and the one that keeps them in shared memory, K
    in one chunk and in several, more blocks than SMs so that the ring is used again; and the same product with
    the RMSNorm of its input rows done inside the kernel."""
    o = ops()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    if not o.gemm_stream_accepts(o.GEMM_STORE, a, w[:N], torch.empty(M, N, device=DEV)):
        assert K > 4096                      # the rows of a long K that has no register form leave no room for a ring
        with pytest.raises(o.KernelError, match="refuses"):
            o.gemm_stream(o.GEMM_STORE, a, w[:N], torch.empty(M, N, device=DEV), 0.25, flag)
        return
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    out = torch.full((M, N), 7.0, device=DEV)
    o.gemm_stream(o.GEMM_STORE, a, w[:N], out, 0.25, flag)
    assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(K / 64)
    half = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_stream(o.GEMM_STORE, a, w[:N], half, 1.0, flag)
    assert float((half.double() - exact[:, :N]).abs().max()) <= 2.0 ** -8 * scale
    base = torch.randn(M, N, device=DEV)
    acc = base.clone()
    o.gemm_stream(o.GEMM_ACCUM, a, w[:N], acc, 1.5, flag)
    assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(K / 64)
    act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    o.gemm_stream(o.GEMM_SWIGLU, a, w, act, 1.0, flag)
    gate, up = exact[:, :N], exact[:, N:]
    want = up * gate / (1 + torch.exp(-gate))
    assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    # a view with a row stride of its own, and a shorter ring
    wide = torch.full((M, N + 3), 7.0, device=DEV)
    o.gemm_stream(o.GEMM_STORE, a, w[:N], wide[:, 1:N + 1], 0.25, flag, stages_cap=2, early_stages=2)
    assert torch.equal(wide[:, 1:N + 1], out) and float(wide[:, 0].min()) == 7.0 and float(wide[:, N + 1:].min()) == 7.0
    # a token's result does not depend on how many other tokens are in the batch
    alone = torch.empty(1, N, device=DEV)
    o.gemm_stream(o.GEMM_STORE, a[M - 1:M].contiguous(), w[:N], alone, 0.25, flag)
    assert torch.equal(alone[0], out[M - 1])
    # the norm inside the kernel against the norm's own kernel followed by the product
    rows = torch.randn(M, K, device=DEV) * 3.0
    for weight in ((1 + 0.2 * torch.randn(K, device=DEV)).to(torch.bfloat16), 1 + 0.2 * torch.randn(K, device=DEV)):
        if not o.gemm_stream_accepts(o.GEMM_STORE, rows, w[:N], torch.empty(M, N, device=DEV), norm=True):
            assert K > 4096 or (M > 8 and K > 2048) or K % 1024
            continue
        normed = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
        o.rmsnorm(rows, weight, normed, 1e-5)
        plain = torch.empty(M, N, device=DEV)
        o.gemm_stream(o.GEMM_STORE, normed, w[:N], plain, 1.0, flag)
        fused = torch.empty(M, N, device=DEV)
        o.gemm_stream(o.GEMM_STORE, rows, w[:N], fused, 1.0, flag, norm_weight=weight, eps=1e-5)
        # the sum of squares is taken in another order than in the norm's kernel: a row may differ in the last
        # bit of some bfloat16 elements, which moves a sum of K products of size ~1/sqrt(K) by ~2^-9 at most
        assert float((fused - plain).abs().max()) < 2.0 ** -7 * scale
        want_rows = rows.double() / torch.sqrt((rows.double() ** 2).mean(dim=1, keepdim=True) + 1e-5) * weight.double()
        assert float((fused.double() - want_rows @ w[:N].double().T).abs().max()) < 2.0 ** -6 * scale * max(1.0, float(want_rows.abs().max()))
    torch.cuda.synchronize()
    assert flag.item() == 0
    with pytest.raises(o.KernelError, match="refuses"):
        o.gemm_stream(o.GEMM_STORE, torch.zeros(17, K, device=DEV, dtype=torch.bfloat16), w[:N], torch.empty(17, N, device=DEV))
    with pytest.raises(o.KernelError, match="refuses"):
        o.gemm_stream(o.GEMM_STORE, torch.zeros(M, 72, device=DEV, dtype=torch.bfloat16),
                      torch.zeros(N, 72, device=DEV, dtype=torch.bfloat16), torch.empty(M, N, device=DEV))      # K no multiple of 64


@pytest.mark.parametrize("M", [1, 16, 33, 40, 64, 100, 128, 200, 300])
@pytest.mark.parametrize("N,K", [(128, 64), (200, 200), (2560, 2048), (1000, 6144), (384, 96), (2048, 2048), (6144, 2048)])
def test_gemm_cluster_all_epilogues_against_64_bit(M, N, K):
    """The product that cuts K over a cluster: token counts that are no multiple of 16, widths that are no
    multiple of 128, K shorter than the cluster is wide, K long enough that the ring is used again."""
    o = ops()
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    exact = a.double() @ w.double().T
    scale = max(1.0, float(exact.abs().max()))
    if o.gemm_cluster_accepts(o.GEMM_STORE, a, w[:N], torch.empty(M, N, device=DEV)):
        out = torch.full((M, N), 7.0, device=DEV)
        o.gemm_cluster(o.GEMM_STORE, a, w[:N], out, 0.25, flag)
        assert float((out.double() - 0.25 * exact[:, :N]).abs().max()) < 2e-5 * scale * math.sqrt(K / 64)
        again = torch.full((M, N), 7.0, device=DEV)
        o.gemm_cluster(o.GEMM_STORE, a, w[:N], again, 0.25, flag)
        assert torch.equal(out, again)                  # the ranges are added in a fixed order
        half = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        o.gemm_cluster(o.GEMM_STORE, a, w[:N], half, 1.0, flag)
        assert float((half.double() - exact[:, :N]).abs().max()) <= 2.0 ** -8 * scale
        base = torch.randn(M, N, device=DEV)
        acc = base.clone()
        o.gemm_cluster(o.GEMM_ACCUM, a, w[:N], acc, 1.5, flag)
        assert float((acc.double() - (base.double() + 1.5 * exact[:, :N])).abs().max()) < 5e-5 * scale * math.sqrt(K / 64)
        # a view with a row stride that rules out 16-byte stores
        wide = torch.full((M, N + 3), 7.0, device=DEV)
        o.gemm_cluster(o.GEMM_STORE, a, w[:N], wide[:, 1:N + 1], 0.25, flag)
        assert torch.equal(wide[:, 1:N + 1], out) and float(wide[:, 0].min()) == 7.0 and float(wide[:, N + 1:].min()) == 7.0
    else:
        with pytest.raises(o.KernelError, match="refuses"):
            o.gemm_cluster(o.GEMM_STORE, a, w[:N], torch.empty(M, N, device=DEV), 0.25, flag)
    if o.gemm_cluster_accepts(o.GEMM_SWIGLU, a, w, torch.empty(M, N, device=DEV, dtype=torch.bfloat16)):
        act = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        o.gemm_cluster(o.GEMM_SWIGLU, a, w, act, 1.0, flag)
        gate, up = exact[:, :N], exact[:, N:]
        want = up * gate / (1 + torch.exp(-gate))
        assert float((act.double() - want).abs().max()) <= 2.0 ** -8 * max(1.0, float(want.abs().max()))
    torch.cuda.synchronize()
    assert flag.item() == 0


def test_gemm_tc_refuses_what_tma_cannot_address():
    o = ops()
    a = torch.randn(4, 100, device=DEV).to(torch.bfloat16)          # K = 100: rows of 200 bytes
    w = torch.randn(16, 100, device=DEV).to(torch.bfloat16)
    assert not o.gemm_tc_accepts(o.GEMM_STORE, a, w, torch.empty(4, 16, device=DEV))
    with pytest.raises(o.KernelError, match="refuses"):
        o.gemm_tc(o.GEMM_STORE, a, w, torch.empty(4, 16, device=DEV))


@pytest.mark.parametrize("d,nq,nkv,page_size,window,split_len", [
    (128, 16, 2, 16, None, 128), (128, 16, 2, 16, None, 4096), (64, 16, 2, 4, None, 64), (32, 3, 1, 16, 100, 64),
    (64, 40, 2, 8, None, 192), (128, 32, 2, 32, 700, 256), (32, 8, 8, 16, None, 64), (64, 6, 3, 12, None, 128),
    (128, 16, 2, 16, None, 384), (128, 16, 2, 16, None, 768), (64, 6, 3, 12, 500, 128)])
@pytest.mark.parametrize("fused", [True, False])
def test_attention_decode_split_keys(d, nq, nkv, page_size, window, split_len, fused):
    """Tensor-core decode attention: groups of up to 16 query heads per kv head, ranges of keys merged,
    a far key that dominates, the window's edge, scrambled pages, rows that are skipped."""
    torch.manual_seed(d + nq)
    T = 1500
    k = torch.randn(T, nkv, d, device=DEV) * 0.5
    v = torch.randn(T, nkv, d, device=DEV)
    positions = [0, 1, 62, 63, 64, 127, 128, 700, 1498, 1499]
    q = torch.randn(len(positions), nq, d, device=DEV) * 0.5
    far = 3 if not window else 1499 - window + 1
    k[far] = 0
    k[far, :, 0] = 6.0
    q[-1, :, 0] = 4.0 * math.sqrt(d)
    if window:
        k[far - 1, :, 1] = 50.0
        q[-1, :, 1] = 4.0 * math.sqrt(d)
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    blocks = (T + page_size - 1) // page_size
    num_pages = blocks + 5
    order = np.random.default_rng(1).permutation(num_pages)[:blocks]
    kp, table = paged(k, page_size, num_pages, order)
    vp, _ = paged(v, page_size, num_pages, order)
    bt = torch.full((2, blocks + 1), -1, dtype=torch.int32)
    bt[1, :blocks] = table
    n = len(positions)
    rows = torch.tensor([0, 1, 2, 3, -1, 5, 6, 7, 8, 9], dtype=torch.int32, device=DEV)     # row 4 is skipped
    out = torch.full((n, nq * d), 7.0, device=DEV, dtype=torch.bfloat16)
    span = min(1500, window) if window else 1500
    n_splits = (span + split_len - 1) // split_len
    partial = torch.empty(n * nq * n_splits * (d + 1), device=DEV) if n_splits > 1 else None
    scale = 1 / math.sqrt(d)
    # fused: the CTA that finishes a token last merges its ranges (counters zero before, zero after)
    counters = torch.zeros(n * nkv * ((nq // nkv + 15) // 16), dtype=torch.int32, device=DEV) if fused else None
    for _ in range(2 if fused else 1):
        out.fill_(7.0)
        ops().attention_decode(q.view(n, nq * d), kp, vp, rows, torch.tensor(positions, dtype=torch.int32, device=DEV),
                               torch.ones(n, dtype=torch.int32, device=DEV), bt.to(DEV), out, partial, nq, nkv, d, window,
                               scale, split_len, n_splits, counters)
    if fused:
        assert int(counters.abs().max()) == 0
    want = reference_attention(q, k, v, positions, window, scale)
    got = out.view(n, nq, d).double()
    keep = [i for i in range(n) if i != 4]
    error = float((got[keep] - want[keep]).abs().max())
    assert error <= 1.6e-2 * max(1.0, float(want.abs().max())), error
    assert float((out[4].float() - 7.0).abs().max()) == 0
    assert float((got[-1, 0] - v[far, 0].double()).abs().max()) < 0.05
    # the same ranges as thread-block clusters, meeting in distributed shared memory: the ranges are normalised and
    # added in the same order as through scratch memory, so the bits are the same
    if n_splits in (2, 4, 8, 16) and fused:
        fit = ops().attention_decode_cluster_splits(d, nq // nkv, n * nkv * ((nq // nkv + 15) // 16), n_splits)
        assert fit in (1, 2, 4, 8, 16) and fit <= n_splits
        if fit == n_splits:
            clustered = torch.full((n, nq * d), 7.0, device=DEV, dtype=torch.bfloat16)
            ops().attention_decode(q.view(n, nq * d), kp, vp, rows, torch.tensor(positions, dtype=torch.int32, device=DEV),
                                   torch.ones(n, dtype=torch.int32, device=DEV), bt.to(DEV), clustered, None, nq, nkv, d, window,
                                   scale, split_len, n_splits, None, cluster=True)
            assert float((clustered[4].float() - 7.0).abs().max()) == 0
            difference = float((clustered[keep].float() - out[keep].float()).abs().max())
            assert difference <= 2.0 ** -7 * max(1.0, float(want.abs().max())), difference


@pytest.mark.parametrize("kernel", ["mma.sync", "tcgen05"])
@pytest.mark.parametrize("d,nq,nkv,page_size,window", [(128, 16, 2, 16, None), (64, 16, 2, 4, None), (32, 3, 1, 16, 40),
                                                       (64, 10, 2, 8, 150), (128, 4, 4, 32, None), (32, 64, 1, 16, None),
                                                       (128, 32, 2, 16, 300), (64, 8, 2, 12, 100), (128, 2, 1, 16, 37)])
def test_attention_prefill_portions(d, nq, nkv, page_size, window, kernel):
    """Tensor-core prefill attention: portions that start and end anywhere (at 0, inside a page, one that
    continues an earlier portion), groups that do not divide 64, a far key that dominates, the window's
    edge, scrambled pages, two requests in one launch."""
    torch.manual_seed(d + nq)
    T = 700
    scale = 1 / math.sqrt(d)
    # request in slot 1: 700 tokens, this step brings [437, 700); request in slot 0: 150 tokens, whole
    ka, va = torch.randn(T, nkv, d, device=DEV) * 0.5, torch.randn(T, nkv, d, device=DEV)
    kb, vb = torch.randn(150, nkv, d, device=DEV) * 0.5, torch.randn(150, nkv, d, device=DEV)
    qa, qb = torch.randn(T - 437, nq, d, device=DEV) * 0.5, torch.randn(150, nq, d, device=DEV) * 0.5
    far = 3 if not window else 699 - window + 1
    ka[far] = 0
    ka[far, :, 0] = 6.0
    qa[-1, :, 0] = 4.0 * math.sqrt(d)
    if window:
        ka[far - 1, :, 1] = 50.0
        qa[-1, :, 1] = 4.0 * math.sqrt(d)
    bf = lambda x: x.to(torch.bfloat16)
    ka, va, kb, vb, qa, qb = map(bf, (ka, va, kb, vb, qa, qb))
    blocks_a, blocks_b = (T + page_size - 1) // page_size, (150 + page_size - 1) // page_size
    num_pages = blocks_a + blocks_b + 4
    order = np.random.default_rng(2).permutation(num_pages)
    kp = torch.zeros(num_pages, page_size, nkv, d, device=DEV, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    bt = torch.full((2, blocks_a + 1), -1, dtype=torch.int32)
    for slot, (kk, vv, blocks, base) in enumerate([(kb, vb, blocks_b, 0), (ka, va, blocks_a, blocks_b)]):
        for b in range(blocks):
            page = int(order[base + b])
            bt[slot, b] = page
            chunk = slice(b * page_size, min((b + 1) * page_size, kk.shape[0]))
            kp[page, :chunk.stop - chunk.start] = kk[chunk]
            vp[page, :chunk.stop - chunk.start] = vv[chunk]
    q = torch.cat([qb, qa]).contiguous()
    n = q.shape[0]
    slots = torch.tensor([0] * 150 + [1] * (T - 437), dtype=torch.int32, device=DEV)
    segments = torch.tensor([[0, 0, 150], [150, 437, T - 437]], dtype=torch.int32, device=DEV)
    tc = kernel == "tcgen05"
    per_tile = ops().attention_prefill_tc_tokens_per_tile(nq // nkv, d) if tc else ops().attention_prefill_tokens_per_tile(nq // nkv)
    if tc and per_tile == 0:
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 and group sizes that divide 128")
    tiles = (150 + per_tile - 1) // per_tile + (T - 437 + per_tile - 1) // per_tile
    out = torch.zeros(n, nq * d, device=DEV, dtype=torch.bfloat16)
    if tc:
        flag = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops().attention_prefill_tc(q.view(n, nq * d), kp, vp, segments, 2, tiles, slots, bt.to(DEV), out, nq, nkv, d,
                                   window, scale, flag)
        torch.cuda.synchronize()
        assert flag.item() == 0
    else:
        ops().attention_prefill(q.view(n, nq * d), kp, vp, segments, 2, tiles, slots, bt.to(DEV), out, nq, nkv, d,
                                window, scale)
    want_b = reference_attention(qb, kb, vb, list(range(150)), window, scale)
    want_a = reference_attention(qa, ka, va, list(range(437, T)), window, scale)
    got = out.view(n, nq, d).double()
    limit = 1.6e-2 * max(1.0, float(want_a.abs().max()), float(want_b.abs().max()))
    assert float((got[:150] - want_b).abs().max()) <= limit
    assert float((got[150:] - want_a).abs().max()) <= limit
    assert float((got[-1, 0] - va[far, 0].double()).abs().max()) < 0.05
    if tc:
        # the keys of every CTA cut into ranges that are merged afterwards: 7 is more than the tiles of either request,
        # so some ranges are empty; the scratch starts as NaN, so a word that is read without having been written shows
        for splits in (2, 3, 7):
            partial = torch.full((ops().attention_prefill_tc_partial_floats(n, nq, d, splits),), float("nan"), device=DEV)
            cut = torch.zeros(n, nq * d, device=DEV, dtype=torch.bfloat16)
            ops().attention_prefill_tc(q.view(n, nq * d), kp, vp, segments, 2, tiles, slots, bt.to(DEV), cut, nq, nkv, d,
                                       window, scale, flag, splits=splits, partial=partial)
            torch.cuda.synchronize()
            assert flag.item() == 0
            got = cut.view(n, nq, d).double()
            assert float((got[:150] - want_b).abs().max()) <= limit, splits
            assert float((got[150:] - want_a).abs().max()) <= limit, splits
            assert float((got[-1, 0] - va[far, 0].double()).abs().max()) < 0.05
        with pytest.raises(Exception):
            ops().attention_prefill_tc(q.view(n, nq * d), kp, vp, segments, 2, tiles, slots, bt.to(DEV), cut, nq, nkv, d,
                                       window, scale, flag, splits=2, partial=partial[:16])


@pytest.mark.parametrize("d,nq,nkv,page_size,window,rotary_dim,n_splits", [
    (128, 16, 2, 16, None, 128, 5), (64, 12, 3, 8, None, 64, 1), (32, 3, 1, 16, 50, 16, 3), (128, 4, 4, 32, 300, 0, 2),
    (64, 32, 2, 4, None, 32, 7), (128, 16, 2, 16, None, 128, 16), (128, 16, 2, 16, None, 128, 8), (64, 32, 2, 4, None, 32, 4),
    (32, 3, 1, 16, 50, 16, 2), (64, 8, 2, 8, 100, 64, 4)])
def test_attention_decode_with_rotary_and_append(d, nq, nkv, page_size, window, rotary_dim, n_splits):
    """The decode attention kernel that also encodes positions and appends the token's key and value,
    against the two separate kernels: the same pages afterwards, the same output (each token at another
    position, one at position 0, one at a page's first slot, one at its last)."""
    o = ops()
    torch.manual_seed(d + nq + rotary_dim)
    positions = [0, 1, page_size - 1, page_size, 63, 64, 65, 200, 333]
    n = len(positions)
    T = 340
    k_old = (torch.randn(n, T, nkv, d, device=DEV) * 0.5).to(torch.bfloat16)
    v_old = torch.randn(n, T, nkv, d, device=DEV).to(torch.bfloat16)
    blocks = (T + page_size - 1) // page_size
    num_pages = n * blocks + 3
    order = np.random.default_rng(3).permutation(num_pages)
    kp = torch.zeros(num_pages, page_size, nkv, d, device=DEV, dtype=torch.bfloat16)
    vp = torch.zeros_like(kp)
    bt = torch.full((n, blocks + 1), -1, dtype=torch.int32)
    for r in range(n):
        pages_k, table = paged(k_old[r], page_size, num_pages, order[r * blocks:(r + 1) * blocks])
        pages_v, _ = paged(v_old[r], page_size, num_pages, order[r * blocks:(r + 1) * blocks])
        used = table.long()
        kp[used] = pages_k[used]
        vp[used] = pages_v[used]
        bt[r, :blocks] = table
    bt = bt.to(DEV)
    qkv = torch.randn(n, (nq + 2 * nkv) * d, device=DEV)
    pos = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    rows = torch.arange(n, dtype=torch.int32, device=DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / max(rotary_dim, 1)))).float().to(DEV) if rotary_dim else None
    scale = 1 / math.sqrt(d)

    def scratch():
        partial = torch.empty(n * nq * n_splits * (d + 1), device=DEV) if n_splits > 1 else None
        counters = torch.zeros(n * nkv, dtype=torch.int32, device=DEV) if n_splits > 1 else None
        return partial, counters

    # separately
    k1, v1 = kp.clone(), vp.clone()
    q1 = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
    o.rope_kv_write(qkv, pos, slots, bt, q1, k1, v1, nq, nkv, d, rotary_dim, inv)
    out1 = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
    partial, counters = scratch()
    o.attention_decode(q1, k1, v1, rows, pos, slots, bt, out1, partial, nq, nkv, d, window, scale, 0, n_splits, counters)
    # in one kernel
    k2, v2 = kp.clone(), vp.clone()
    out2 = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
    partial, counters = scratch()
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.attention_decode(None, k2, v2, rows, pos, slots, bt, out2, partial, nq, nkv, d, window, scale, 0, n_splits, counters,
                       qkv=qkv, inv_freq=inv, rotary_dim=rotary_dim, write_kv=True, error_flag=flag)
    torch.cuda.synchronize()
    assert flag.item() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.equal(out1, out2)
    # and with the ranges of a token as a cluster (ranges beyond a short context have no keys and still take part)
    if n_splits in (2, 4, 8, 16) and o.attention_decode_cluster_splits(d, nq // nkv, n * nkv, n_splits) == n_splits:
        k3, v3 = kp.clone(), vp.clone()
        out3 = torch.empty(n, nq * d, device=DEV, dtype=torch.bfloat16)
        o.attention_decode(None, k3, v3, rows, pos, slots, bt, out3, None, nq, nkv, d, window, scale, 0, n_splits, None,
                           qkv=qkv, inv_freq=inv, rotary_dim=rotary_dim, write_kv=True, error_flag=flag, cluster=True)
        torch.cuda.synchronize()
        assert flag.item() == 0
        assert torch.equal(k1, k3) and torch.equal(v1, v3)
        assert float((out3.float() - out1.float()).abs().max()) <= 2.0 ** -7 * max(1.0, float(out1.float().abs().max()))
