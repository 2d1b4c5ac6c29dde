"""Each CUDA kernel alone against a plain float32 formula, at sizes other than the engine's tiny models:
widths and vocabularies that are no power of two, head sizes in steps of 16, odd group sizes, shuffled
page tables, windows, and inputs built so that a single wrong key, page or row shows."""
import math

import pytest
import torch

from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev():
    return torch.device("cuda:0")


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(dev())


@pytest.mark.parametrize("table_dtype,out_dtype", [("float32", "float32"), ("bfloat16", "float32"), ("bfloat16", "bfloat16")])
def test_embedding(table_dtype, out_dtype):
    from zedinfer_b200 import ops
    table = rand(1003, 136, dtype=DT[table_dtype])
    ids = torch.tensor([0, 1002, 17, 17, 500, 999, 3], dtype=torch.int32, device=dev())
    out = torch.empty(7, 136, dtype=DT[out_dtype], device=dev())
    ops.embedding(table, ids, out)
    assert torch.equal(out.float(), table[ids.long()].to(DT[out_dtype]).float())


@pytest.mark.parametrize("hidden", [48, 1000, 1536, 5120])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_and_fused_add(hidden, dtype):
    from zedinfer_b200 import ops
    t = DT[dtype]
    rows, eps = 9, 1e-5
    res = rand(rows, hidden, scale=3.0)
    delta = rand(rows, hidden, dtype=t, seed=1)
    w = (1 + rand(hidden, scale=0.1, seed=2)).to(t)
    out = torch.empty(rows, hidden, dtype=t, device=dev())
    res2 = res.clone()
    ops.add_rmsnorm(res2, delta, w, eps, out)
    ref_res = res + delta.float()
    ref = P.rms_norm(ref_res.cpu(), w.float().cpu(), eps)
    assert torch.allclose(res2.cpu(), ref_res.cpu(), atol=0, rtol=0)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)
    # rows picked by index, residual untouched
    idx = torch.tensor([8, 0, 3], dtype=torch.int32, device=dev())
    out3 = torch.empty(3, hidden, dtype=t, device=dev())
    res3 = res.clone()
    ops.add_rmsnorm(res3, delta, w, eps, out3, row_idx=idx, write_residual=False)
    assert torch.equal(res3, res)
    assert torch.allclose(out3.float().cpu(), ref[idx.long().cpu()], atol=tol, rtol=tol)
    # plain norm
    x = rand(rows, hidden, dtype=t, seed=4)
    out4 = torch.empty_like(x)
    ops.rmsnorm(x, w, eps, out4)
    assert torch.allclose(out4.float().cpu(), P.rms_norm(x.float().cpu(), w.float().cpu(), eps), atol=tol, rtol=tol)


@pytest.mark.parametrize("types", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                   ("float32", "bfloat16", "float32")])
def test_add(types):
    from zedinfer_b200 import ops
    a = rand(7, 1003, dtype=DT[types[0]], scale=3.0)
    b = rand(7, 1003, dtype=DT[types[1]], seed=1)
    out = torch.empty(7, 1003, dtype=DT[types[2]], device=dev())
    ops.add(a, b, out)
    assert torch.equal(out, (a.float() + b.float()).to(DT[types[2]]))
    with pytest.raises(ops.KernelError, match="shapes"):
        ops.add(a, b[:3].contiguous(), out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,inter", [(5, 176), (3, 8960), (1, 7)])
def test_silu_mul(dtype, rows, inter):
    from zedinfer_b200 import ops
    t = DT[dtype]
    gu = rand(rows, 2 * inter, dtype=t, scale=3.0)
    out = torch.empty(rows, inter, dtype=t, device=dev())
    ops.silu_mul(gu, out)
    ref = P.swiglu(gu[:, :inter].float().cpu(), gu[:, inter:].float().cpu())
    tol = 1e-6 if dtype == "float32" else 2e-2
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("m,n,k", [(1, 1000, 96), (7, 130, 1536), (64, 257, 100), (130, 64, 33), (2, 5, 3)])
@pytest.mark.parametrize("types", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "bfloat16"),
                                   ("bfloat16", "float32", "bfloat16"), ("bfloat16", "bfloat16", "float32")])
def test_gemm_simt(m, n, k, types):
    from zedinfer_b200 import ops
    ta, tw, tc = (DT[x] for x in types)
    a, w, b = rand(m, k, dtype=ta), rand(n, k, dtype=tw, seed=1), rand(n, dtype=tw, seed=2)
    out = torch.empty(m, n, dtype=tc, device=dev())
    ops.gemm_nt(a, w, b, out)
    ref = (a.double().cpu() @ w.double().cpu().t() + b.double().cpu()).float()
    tol = 1e-4 if tc == torch.float32 else 0.1
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=1e-2 if tc == torch.bfloat16 else 1e-5)
    # a row's result does not depend on what else is in the batch
    if m > 1:
        out1 = torch.empty(1, n, dtype=tc, device=dev())
        ops.gemm_nt(a[m - 1:m], w, b, out1)
        assert torch.equal(out1[0], out[m - 1])


@pytest.mark.parametrize("m,n,k", [(1, 1000, 96), (8, 2048, 1536), (64, 1536, 8960), (300, 130, 64)])
def test_linear_bf16(m, n, k):
    from zedinfer_b200 import ops
    a, w, b = rand(m, k, dtype=torch.bfloat16), rand(n, k, dtype=torch.bfloat16, seed=1, scale=0.05), \
        rand(n, dtype=torch.bfloat16, seed=2)
    ref = (a.double().cpu() @ w.double().cpu().t() + b.double().cpu()).float()
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.empty(m, n, dtype=out_dtype, device=dev())
        ops.linear(a, w, b, out)
        assert torch.allclose(out.float().cpu(), ref, atol=0.05, rtol=2e-2)


def build_cache(n_req, lens, nkv, hd, ps, dtype, seed=0, n_calls=2, call=1):
    """A pool with shuffled pages holding random k, v for each request; returns what the kernels need."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-l // ps) for l in lens]
    total = sum(blocks) + 3
    perm = torch.randperm(total, generator=g).tolist()
    pool = torch.full((total + 1, n_calls, 2, nkv, ps, hd), 1000.0).to(dtype).to(dev())   # stale pages hold junk
    width = max(blocks) + 1
    tables = torch.full((n_req, width), -1, dtype=torch.int32)
    ks, vs = [], []
    it = iter(perm)
    for r, l in enumerate(lens):
        k = torch.randn(l, nkv, hd, generator=g)
        v = torch.randn(l, nkv, hd, generator=g)
        ks.append(k.to(dtype).float()), vs.append(v.to(dtype).float())
        for b in range(blocks[r]):
            page = next(it)
            tables[r, b] = page
            n = min(ps, l - b * ps)
            pool[page, call, 0, :, :n] = k[b * ps:b * ps + n].transpose(0, 1).to(dtype).to(dev())
            pool[page, call, 1, :, :n] = v[b * ps:b * ps + n].transpose(0, 1).to(dtype).to(dev())
    view = pool[:, call]
    return pool, view, tables.to(dev()), ks, vs, pool.stride(0), pool.stride(2)


def release_behind_window(tables, first_positions, window, ps, junk_page):
    """What the engine shows the kernels once a window has passed a page and the page was given back: the entry
    points at the scratch page, here ``junk_page`` (the pool's last page, which no request owns and which holds
    1000.0 like every stale page).  ``first_positions[r]``: the earliest query position of row r in the step."""
    t = tables.clone()
    for r, p0 in enumerate(first_positions):
        t[r, :max(0, p0 - window + 1) // ps] = junk_page
    return t


def plain_attention_rows(q, k, v, positions, scale, window):
    """q [n, nh, hd] at the given positions of a sequence whose k, v are [L, nkv, hd]."""
    out = torch.zeros_like(q)
    nh, nkv = q.shape[1], k.shape[1]
    pos = torch.tensor(list(positions))
    keys = torch.arange(k.shape[0])
    seen = keys[None, :] <= pos[:, None]
    if window:
        seen &= keys[None, :] > pos[:, None] - window
    for h in range(nh):
        kvh = h // (nh // nkv)
        s = (q[:, h] @ k[:, kvh].t()) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=1) @ v[:, kvh]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(4, 2, 16, 4, None), (3, 1, 32, 8, None), (6, 3, 48, 16, 24),
                                                  (12, 2, 128, 16, None), (7, 7, 64, 32, 100), (5, 1, 256, 16, None),
                                                  (14, 2, 80, 16, None)])
def test_paged_attention_generic(dtype, nh, nkv, hd, ps, window):
    from zedinfer_b200 import ops
    t = DT[dtype]
    lens = [37, 300, 5]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(3, lens, nkv, hd, ps, t)
    # queries: the last 3 positions of request 0 (a chunk), one decode token of request 1, all of request 2
    spec = [(0, [34, 35, 36]), (1, [299]), (2, [0, 1, 2, 3, 4])]
    g = torch.Generator().manual_seed(3)
    qs, seg, pos = [], [], []
    for r, ps_list in spec:
        for p in ps_list:
            qs.append(torch.randn(nh, hd, generator=g))
            seg.append(r), pos.append(p)
    q = torch.stack(qs)
    # one far key stands out: scale a key of request 1 and point the decode query at it
    far = 2 if not window else 299 - window + 1
    q[3, :, :] = ks[1][far, 0][None, :] * 3.0
    qd = q.to(t).to(dev())
    out = torch.empty(len(seg), nh * hd, dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    ops.paged_attention(qd, view, out, tables, torch.tensor(seg, dtype=torch.int32, device=dev()),
                        torch.tensor(pos, dtype=torch.int32, device=dev()), nh, nkv, hd, ps, page_stride, kv_stride,
                        window, scale)
    got = out.float().cpu().view(len(seg), nh, hd)
    qf = qd.float().cpu()
    i = 0
    for r, ps_list in spec:
        ref = plain_attention_rows(qf[i:i + len(ps_list)], ks[r], vs[r], ps_list, scale, window)
        tol = 2e-5 if dtype == "float32" else 2e-2
        assert torch.allclose(got[i:i + len(ps_list)], ref, atol=tol, rtol=tol), (r, float((got[i:i + len(ps_list)] - ref).abs().max()))
        i += len(ps_list)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 4), (12, 2, 128, 16), (3, 1, 48, 8)])
def test_rope_append(dtype, nh, nkv, hd, ps):
    from zedinfer_b200 import ops
    t = DT[dtype]
    theta = 10000.0
    # two requests: one appends a chunk at positions 5..10, the other a single token at position 21
    seg = [0] * 6 + [1]
    pos = list(range(5, 11)) + [21]
    n = len(seg)
    pool = torch.zeros((9, 3, 2, nkv, ps, hd), dtype=t, device=dev())
    tables = torch.tensor([[4, 7, 1, 0, 0, 0], [2, 8, 5, 3, 6, 0]][:2], dtype=torch.int32, device=dev())
    qkv = rand(n, (nh + 2 * nkv) * hd + 8, dtype=t)[:, :(nh + 2 * nkv) * hd]      # rows with a stride
    q_out = torch.empty(n, nh, hd, dtype=t, device=dev())
    expo = torch.arange(0, hd, 2, dtype=torch.float32) / float(hd)
    inv = (1.0 / torch.pow(torch.tensor(theta), expo)).to(dev())
    call = 1
    ops.rope_append(qkv, q_out, pool[:, call], tables, torch.tensor(seg, dtype=torch.int32, device=dev()),
                    torch.tensor(pos, dtype=torch.int32, device=dev()), inv, nh, nkv, hd, ps, pool.stride(0),
                    pool.stride(2))
    x = qkv.float().cpu()
    qr = P.rope(x[:, :nh * hd].reshape(n, nh, hd), torch.tensor(pos), theta)
    kr = P.rope(x[:, nh * hd:(nh + nkv) * hd].reshape(n, nkv, hd), torch.tensor(pos), theta)
    v = x[:, (nh + nkv) * hd:].reshape(n, nkv, hd)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert torch.allclose(q_out.float().cpu(), qr, atol=tol, rtol=tol)
    tab = tables.cpu()
    touched = torch.zeros(pool.shape, dtype=torch.bool)
    for i in range(n):
        page, off = int(tab[seg[i], pos[i] // ps]), pos[i] % ps
        assert torch.allclose(pool[page, call, 0, :, off].float().cpu(), kr[i], atol=tol, rtol=tol)
        assert torch.equal(pool[page, call, 1, :, off].float().cpu(), v[i].to(t).float())
        touched[page, call, :, :, off] = True
    assert float(pool.float().cpu()[~touched].abs().max()) == 0.0          # nothing else was written
    # the same with the step's table of angles in place of a sincosf per layer: bit for bit what the kernel above wrote
    cs = torch.empty(n, hd, dtype=torch.float32, device=dev())
    pos_d = torch.tensor(pos, dtype=torch.int32, device=dev())
    ops.rope_table(pos_d, inv, cs)
    pool2, q2 = torch.zeros_like(pool), torch.empty_like(q_out)
    ops.rope_append(qkv, q2, pool2[:, call], tables, torch.tensor(seg, dtype=torch.int32, device=dev()), pos_d, inv, nh, nkv,
                    hd, ps, pool2.stride(0), pool2.stride(2), cs=cs)
    assert torch.equal(q2, q_out) and torch.equal(pool2, pool)
    q3 = torch.empty_like(q_out)                                          # a layer that writes no keys or values
    ops.rope_append(qkv, q3, None, tables, torch.tensor(seg, dtype=torch.int32, device=dev()), pos_d, inv, nh, nkv, hd, ps,
                    0, 0, write_kv=False, cs=cs)
    assert torch.equal(q3, q_out)


def test_argmax_ties_and_rows():
    from zedinfer_b200 import ops
    logits = torch.randn(5, 151937)
    logits[1, 70000] = 50.0
    logits[1, 90000] = 50.0         # tie: the lower index wins
    logits[2, 0] = 60.0
    logits[3, 151936] = 60.0
    logits[4] = -1.0                # all equal
    out = torch.empty(5, dtype=torch.int32, device=dev())
    ops.argmax(logits.to(dev()), out)
    exp = [P.greedy(logits[i]) for i in range(5)]
    assert out.cpu().tolist() == exp
    assert exp[1] == 70000 and exp[4] == 0


@pytest.mark.parametrize("vocab", [777, 151936])
def test_sample_matches_plain_distribution(vocab):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(1)
    cases = [(0.7, 0, 1.0), (1.0, 5, 1.0), (1.3, 0, 0.6), (0.5, 20, 0.9), (0.0, 0, 1.0)]
    rows = len(cases)
    logits = torch.randn(rows, vocab, generator=g) * 3.0
    temp = torch.tensor([c[0] for c in cases])
    top_k = torch.tensor([c[1] for c in cases], dtype=torch.int32)
    top_p = torch.tensor([c[2] for c in cases])
    dl = logits.to(dev())
    for u in (0.0, 0.123, 0.5, 0.77, 0.999):
        uni = torch.full((rows,), u)
        out = torch.empty(rows, dtype=torch.int32, device=dev())
        ops.sample(dl, out, temp.to(dev()), top_k.to(dev()), top_p.to(dev()), uni.to(dev()))
        got = out.cpu().tolist()
        for r, (t, k, p) in enumerate(cases):
            if t <= 0:
                assert got[r] == P.greedy(logits[r])
                continue
            dist = P.sampling_distribution(logits[r], t, k, p)
            assert dist[got[r]] > 0, f"row {r}: token {got[r]} is outside the kept set"
            # the running sum just before and at the chosen token brackets u (up to rounding of the sums)
            cum = torch.cumsum(dist.double(), 0)
            lo = float(cum[got[r]] - dist[got[r]].double())
            hi = float(cum[got[r]])
            assert lo - 1e-4 <= u <= hi + 1e-4, (r, u, lo, hi)


@pytest.mark.parametrize("vocab", [3000, 151936])
def test_sample_with_few_likely_tokens(vocab):
    """Logits as a language model gives them: a few likely tokens and a long tail (probability ~ rank^-1.5, ranks
    dealt at random over the vocabulary).  top-p then keeps tens of tokens, top-k a few, a large k thousands."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(7)
    cases = [(0.8, 0, 0.9), (1.0, 0, 0.5), (0.7, 40, 0.95), (1.0, 2500, 0.99), (1.2, 2500, 1.0), (0.9, 0, 0.999), (1.0, 7, 1.0)]
    rows = len(cases)
    rank = torch.stack([torch.randperm(vocab, generator=g) for _ in range(rows)]).float() + 1.0
    logits = -1.5 * torch.log(rank) + 0.01 * torch.randn(rows, vocab, generator=g)
    temp = torch.tensor([c[0] for c in cases]).to(dev())
    top_k = torch.tensor([c[1] for c in cases], dtype=torch.int32).to(dev())
    top_p = torch.tensor([c[2] for c in cases]).to(dev())
    dl = logits.to(dev())
    dists = [P.sampling_distribution(logits[r], *cases[r]) for r in range(rows)]
    assert int((dists[0] > 0).sum()) < 500 and int((dists[3] > 0).sum()) > 300
    for u in (0.0, 0.2, 0.45, 0.71, 0.93, 0.9999):
        out = torch.empty(rows, dtype=torch.int32, device=dev())
        ops.sample(dl, out, temp, top_k, top_p, torch.full((rows,), u).to(dev()))
        got = out.cpu().tolist()
        for r in range(rows):
            dist = dists[r]
            assert dist[got[r]] > 0, f"row {r}: token {got[r]} is outside the kept set"
            cum = torch.cumsum(dist.double(), 0)
            lo, hi = float(cum[got[r]] - dist[got[r]].double()), float(cum[got[r]])
            assert lo - 1e-4 <= u <= hi + 1e-4, (r, u, lo, hi)


@pytest.mark.parametrize("vocab", [5, 8193, 40000])
def test_sample_at_the_edges_of_its_rules(vocab):
    """Ties at the k-th entry, -inf entries, k = 1, k beyond the row, a top_p that only the first entry meets,
    rows below zero throughout; every row alone gives what it gives in the batch, call after call."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(vocab)
    base = torch.randn(vocab, generator=g) * 2.0
    tied = base.clone(); tied[torch.randperm(vocab, generator=g)[:4]] = float(base.max()) + 1.0   # four equal firsts
    holes = base.clone(); holes[::2] = -math.inf
    below = -base.abs() - 3.0
    one = torch.full((vocab,), -math.inf); one[vocab - 1] = 0.5                                   # a single finite entry
    cases = [(tied, 0.9, 2, 1.0), (tied, 0.9, 0, 0.3), (holes, 1.1, 3, 1.0), (holes, 0.6, 0, 0.8), (base, 1.0, 1, 1.0),
             (base, 1.0, vocab + 7, 1.0), (base, 0.8, 0, 1e-6), (below, 1.5, 4, 0.7), (one, 1.0, 0, 0.9), (one, 0.7, 3, 1.0)]
    rows = len(cases)
    logits = torch.stack([c[0] for c in cases]).to(dev())
    temp = torch.tensor([c[1] for c in cases]).to(dev())
    top_k = torch.tensor([c[2] for c in cases], dtype=torch.int32).to(dev())
    top_p = torch.tensor([c[3] for c in cases]).to(dev())
    for u in (0.0, 0.31, 0.62, 0.97):
        uni = torch.full((rows,), u).to(dev())
        out = torch.empty(rows, dtype=torch.int32, device=dev())
        ops.sample(logits, out, temp, top_k, top_p, uni)
        got = out.cpu().tolist()
        again = torch.empty_like(out)
        ops.sample(logits, again, temp, top_k, top_p, uni)
        assert again.cpu().tolist() == got
        for r, (row, t, k, p) in enumerate(cases):
            dist = P.sampling_distribution(row, t, k, p)
            assert dist[got[r]] > 0, f"row {r}: token {got[r]} is outside the kept set"
            cum = torch.cumsum(dist.double(), 0)
            lo, hi = float(cum[got[r]] - dist[got[r]].double()), float(cum[got[r]])
            assert lo - 1e-4 <= u <= hi + 1e-4, (r, u, lo, hi)
            alone = torch.empty(1, dtype=torch.int32, device=dev())
            ops.sample(logits[r:r + 1], alone, temp[r:r + 1], top_k[r:r + 1], top_p[r:r + 1], uni[r:r + 1])
            assert int(alone[0]) == got[r]
    assert got[4] == P.greedy(base) and got[6] == P.greedy(base) and got[8] == vocab - 1 and got[9] == vocab - 1


def test_repetition_penalty():
    from zedinfer_b200 import ops
    row = torch.tensor([2.0, -1.0, 0.5, 4.0, -3.0])
    d = row.to(dev())
    ops.repetition_penalty(d, torch.tensor([0, 1, 9, 3], dtype=torch.int32, device=dev()), 2.0)
    assert torch.allclose(d.cpu(), torch.tensor([1.0, -2.0, 0.5, 2.0, -3.0]))


def test_repetition_penalty_from_a_table_of_counts():
    """Counts kept per slot: a step's chosen tokens and a list of tokens are added, and the rows' logits are penalised
    once per time the token was generated, as the loop over the generated tokens does; rows without a slot or with a
    penalty of 1 keep their logits."""
    from zedinfer_b200 import ops
    vocab, slots_n = 1311, 5
    g = torch.Generator().manual_seed(4)
    logits = torch.randn(4, vocab, generator=g) * 3.0
    logits[0, 17] = 0.0
    counts = torch.zeros(slots_n, vocab, dtype=torch.int32, device=dev())
    history = {3: [17, 5, 5, 900, 1310, 5], 0: [2, 2], 4: [7]}
    for slot, toks in history.items():
        ops.count_token_list(counts[slot], torch.tensor(toks[:-1], dtype=torch.int32, device=dev()))
    slots = torch.tensor([3, -1, 0, 4], dtype=torch.int32, device=dev())
    last = torch.tensor([history[3][-1], 11, history[0][-1], history[4][-1]], dtype=torch.int32, device=dev())
    ops.count_tokens(counts, slots, last)
    exp_counts = torch.zeros(slots_n, vocab, dtype=torch.int32)
    for slot, toks in history.items():
        for t in toks:
            exp_counts[slot, t] += 1
    assert torch.equal(counts.cpu(), exp_counts)
    penalty = torch.tensor([1.7, 2.0, 0.6, 1.0], dtype=torch.float32, device=dev())
    d = logits.to(dev())
    ops.penalty_rows(d, counts, slots, penalty)
    exp = logits.clone()
    for row, (slot, pen) in enumerate(((3, 1.7), (None, 2.0), (0, 0.6), (4, 1.0))):
        if slot is None:
            continue
        for t in history[slot]:
            exp[row, t] = exp[row, t] / pen if exp[row, t] > 0 else exp[row, t] * pen
    assert torch.equal(d.cpu(), exp)
    assert float(d[0, 17]) == 0.0


# ---- tensor-core attention (bfloat16, head_dim 64 / 128) -------------------------------------------------
@pytest.mark.parametrize("kernel", ["cp_async", "tma"])
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (7, 1, 64, 4, None), (20, 1, 128, 16, None),
                                                  (4, 4, 64, 24, None), (12, 2, 128, 16, 300), (6, 3, 64, 8, 70),
                                                  (28, 4, 128, 32, None), (6, 2, 128, 64, 900), (3, 1, 64, 128, None)])
def test_decode_attention_mma(nh, nkv, hd, ps, window, kernel):
    from zedinfer_b200 import ops
    if kernel == "tma" and not ops.tcgen05_attention_ok(hd, ps):
        pytest.skip("page size outside what the TMA kernel takes; the engine uses the cp.async kernel there")
    t = torch.bfloat16
    lens = [1, 255, 256, 257, 700, 64, 513, 1500, 5000, 33]   # around tile edges, fewer tiles than blocks, several rounds
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=5)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(len(lens), nh, hd, generator=g)
    # a far key that must dominate: request 4 (700 keys) looks hard at key 3 (or at the window's first key)
    far = 3 if not window else 699 - window + 1
    q[4, :, :] = ks[4][far, 0][None, :] * 4.0
    qd = q.to(t).to(dev())
    n = len(lens)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev())
    seg = torch.arange(n, dtype=torch.int32, device=dev())
    out = torch.empty(n, nh * hd, dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    fn = ops.decode_attention if kernel == "cp_async" else ops.decode_attention_tma
    if window:          # pages wholly behind the window were given back: the tables show the scratch page there
        tables = release_behind_window(tables, [l - 1 for l in lens], window, ps, pool.shape[0] - 1)
    fn(qd, view, out, tables, seg, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    got = out.float().cpu().view(n, nh, hd)
    qf = qd.float().cpu()
    for r in range(n):
        ref = plain_attention_rows(qf[r:r + 1], ks[r], vs[r], [lens[r] - 1], scale, window)
        err = float((got[r:r + 1] - ref).abs().max())
        assert err < 2e-2, (r, lens[r], err)
    # the general kernel computes the same function
    out2 = torch.empty_like(out)
    ops.paged_attention(qd, view, out2, tables, seg, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    assert float((out2.float() - out.float()).abs().max()) < 2e-2


@pytest.mark.parametrize("kernel", ["mma", "tcgen05"])
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(12, 2, 128, 16, None), (3, 1, 64, 4, None), (5, 5, 128, 24, None),
                                                  (6, 2, 64, 16, 50), (12, 2, 128, 16, 130), (4, 2, 64, 128, None),
                                                  (6, 1, 128, 8, 260), (2, 1, 128, 64, None)])
def test_prefill_attention_tensor_cores(nh, nkv, hd, ps, window, kernel):
    from zedinfer_b200 import ops
    if kernel == "tcgen05" and not ops.tcgen05_attention_ok(hd, ps):
        pytest.skip("page size outside what the tcgen05 kernel takes; the engine uses the mma.sync kernel there")
    t = torch.bfloat16
    lens = [200, 70, 64, 333, 1, 1100, 1100]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=6)
    # portions: (request, first position, count).  Whole prompts, portions in mid-prompt, one decoded token, a long
    # prompt (nine key tiles: every ring of the tcgen05 kernel turns over several times) and a late portion of one.
    portions = [(0, 0, 200), (1, 60, 10), (2, 0, 64), (3, 130, 203), (4, 0, 1), (5, 0, 1100), (6, 517, 583)]
    g = torch.Generator().manual_seed(4)
    qs, pos, tiles = [], [], []
    n = 0
    rows = ops.PREFILL_TILE_ROWS
    for si, (r, p0, cnt) in enumerate(portions):
        for q0 in range(0, cnt, rows):
            tiles.append((n + q0, min(rows, cnt - q0), si))
        for i in range(cnt):
            qs.append(torch.randn(nh, hd, generator=g))
            pos.append(p0 + i)
        n += cnt
    q = torch.stack(qs)
    # the last query of request 3 looks hard at one far key (or the first key inside its window), and so does the
    # last query of the long prompt at a key of its first tile
    far = 7 if not window else 332 - window + 1
    q[200 + 10 + 64 + 202, :, :] = ks[3][far, 0][None, :] * 4.0
    far5 = 5 if not window else 1099 - window + 1
    q[200 + 10 + 64 + 203 + 1 + 1099, :, :] = ks[5][far5, 0][None, :] * 4.0
    qd = q.to(t).to(dev())
    seg_tables = torch.stack([tables[r] for r, _, _ in portions])
    if window:          # pages wholly behind the window of a portion's first query were given back
        seg_tables = release_behind_window(seg_tables, [p0 for _, p0, _ in portions], window, ps, pool.shape[0] - 1)
    out = torch.full((n, nh * hd), float("nan"), dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    fn = ops.prefill_attention if kernel == "mma" else ops.prefill_attention_tcgen05
    fn(qd, view, out, seg_tables, torch.tensor(tiles, dtype=torch.int32, device=dev()),
       torch.tensor(pos, dtype=torch.int32, device=dev()), nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    got = out.float().cpu().view(n, nh, hd)
    assert torch.isfinite(got).all()
    qf = qd.float().cpu()
    i = 0
    for r, p0, cnt in portions:
        ref = plain_attention_rows(qf[i:i + cnt], ks[r], vs[r], list(range(p0, p0 + cnt)), scale, window)
        err = float((got[i:i + cnt] - ref).abs().max())
        assert err < 2e-2, (r, p0, cnt, err)
        i += cnt


@pytest.mark.parametrize("rows,n,k", [(17, 1536, 8960), (64, 1536, 8960), (256, 896, 4864), (40, 3584, 18944)])
def test_product_as_partial_sums_folded_by_the_norm(rows, n, k):
    """A product whose result goes into the residual stream may come as float32 sums over four ranges of K; the norm
    adds them in order, rounds the sum to bfloat16 as the whole product would have been rounded, and goes on as
    with a bfloat16 branch output: residual and normed output equal those of that path up to the last bit of the
    product's rounding, and both are right against float64."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(rows + n)
    x = (torch.randn(rows, k, generator=g) * 0.5).to(torch.bfloat16).to(dev())
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev())
    wn = (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).to(dev())
    h0 = torch.randn(rows, n, generator=g).to(dev())
    parts = ops.linear_for_residual(x, w, None)
    assert parts.dim() == 3 and parts.shape == (ops.RESIDUAL_K_PARTS, rows, n) and parts.dtype == torch.float32
    h1, out1 = h0.clone(), torch.empty(rows, n, dtype=torch.bfloat16, device=dev())
    ops.add_rmsnorm(h1, parts, wn, 1e-6, out1)
    ref_delta = (x.double().cpu() @ w.double().cpu().t())
    delta_bf = ref_delta.to(torch.bfloat16).double()
    ref_h = h0.double().cpu() + delta_bf
    assert float((h1.double().cpu() - ref_h).abs().max()) <= 2.0 * float(delta_bf.abs().max()) * 2 ** -8 + 1e-5
    rstd = 1.0 / torch.sqrt((h1.double().cpu() ** 2).mean(dim=1, keepdim=True) + 1e-6)
    ref_out = (wn.double().cpu() * h1.double().cpu()) * rstd
    assert float((out1.double().cpu() - ref_out).abs().max()) < 2e-2
    # the wanted-rows form reads the same sums and leaves the residual alone
    idx = torch.tensor([rows - 1, 0, 3], dtype=torch.int32, device=dev())
    h2, out2 = h0.clone(), torch.empty(3, n, dtype=torch.bfloat16, device=dev())
    ops.add_rmsnorm(h2, parts, wn, 1e-6, out2, row_idx=idx, write_residual=False)
    assert torch.equal(h2, h0) and torch.equal(out2, out1[idx.long()])
    # few rows, a bias, or a short K: the product itself
    assert ops.linear_for_residual(x[:8].contiguous(), w, None).shape == (8, n)
    assert ops.linear_for_residual(x, w, torch.zeros(n, dtype=torch.bfloat16, device=dev())).shape == (rows, n)


@pytest.mark.parametrize("hd,window", [(128, None), (64, None), (128, 200)])
def test_prefill_attention_tcgen05_with_scores_far_apart(hd, window):
    """Scores of one row spread over hundreds of units (queries scaled up), so that most exponentials lie far
    below the smallest float32: the part of them that the kernel computes by arithmetic instead of the
    special-function unit holds its argument at -125 and must come out as nothing, not as a wrapped exponent.  A row
    whose scores are all equal and a row with two equal maxima far above the rest are among them."""
    from zedinfer_b200 import ops
    t, nh, nkv, ps, L = torch.bfloat16, 4, 2, 16, 700
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(1, [L], nkv, hd, ps, t, seed=9)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(L, nh, hd, generator=g) * 25.0                # score differences of several hundred
    q[650] = 0.0                                                  # every score equal
    q[651, :, :] = (ks[0][10, 0] + ks[0][400, 0])[None, :] * 20.0
    qd = q.to(t).to(dev())
    tiles = torch.tensor([(q0, min(128, L - q0), 0) for q0 in range(0, L, 128)], dtype=torch.int32, device=dev())
    pos = torch.arange(L, dtype=torch.int32, device=dev())
    seg_tables = tables if not window else release_behind_window(tables, [0], window, ps, pool.shape[0] - 1)
    out = torch.full((L, nh * hd), float("nan"), dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    ops.prefill_attention_tcgen05(qd, view, out, seg_tables, tiles, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    got = out.float().cpu().view(L, nh, hd)
    assert torch.isfinite(got).all()
    ref = plain_attention_rows(qd.float().cpu().view(L, nh, hd), ks[0], vs[0], list(range(L)), scale, window)
    err = (got - ref).abs().amax(dim=(1, 2))
    assert float(err.max()) < 3e-2, (int(err.argmax()), float(err.max()))


@pytest.mark.parametrize("m,nh,nkv,hd,hidden,ps,with_bias", [(8, 12, 2, 128, 1536, 16, True), (1, 3, 1, 32, 96, 8, True),
                                                             (16, 4, 4, 64, 160, 4, False), (11, 6, 3, 48, 224, 16, True)])
def test_product_with_rotation_and_append_equals_the_separate_kernels(m, nh, nkv, hd, hidden, ps, with_bias):
    """The decode q/k/v product with RoPE and the cache append in its epilogue gives the bits of product, then
    rotation kernel: q and every cache page are compared exactly."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(m + hd)
    t = torch.bfloat16
    width = (nh + 2 * nkv) * hd
    x = (torch.randn(m, hidden, generator=g) * 0.7).to(t).to(dev())
    w = (torch.randn(width, hidden, generator=g) * 0.08).to(t).to(dev())
    b = (torch.randn(width, generator=g) * 0.3).to(t).to(dev()) if with_bias else None
    positions = torch.tensor([(37 * i + 5) % 200 for i in range(m)], dtype=torch.int32, device=dev())
    blocks = 200 // ps + 1
    tables = torch.randperm(m * blocks, generator=g).to(torch.int32).view(m, blocks).to(dev())
    seg = torch.arange(m, dtype=torch.int32, device=dev())
    inv_freq = (1.0 / torch.pow(torch.tensor(10000.0), torch.arange(0, hd, 2, dtype=torch.float32) / hd)).to(dev())
    pools, qs = [], []
    for fused in (False, True):
        pool = torch.full((m * blocks + 1, 2, 2, nkv, ps, hd), 7.0, dtype=t, device=dev())
        view = pool[:, 1]
        q = torch.full((m, nh, hd), float("nan"), dtype=t, device=dev())
        if fused:
            cs = torch.empty(m, hd, dtype=torch.float32, device=dev())
            ops.rope_table(positions, inv_freq, cs)
            ops.gemm_smallm_rope(x, w, b, cs, q, view, tables, seg, positions, nh, nkv, hd, ps, pool.stride(0), pool.stride(2))
        else:
            qkv = torch.empty(m, width, dtype=t, device=dev())
            ops.gemm_smallm(x, w, b, qkv)
            ops.rope_append(qkv, q, view, tables, seg, positions, inv_freq, nh, nkv, hd, ps, pool.stride(0), pool.stride(2))
        torch.cuda.synchronize()
        pools.append(pool), qs.append(q)
    assert torch.isfinite(qs[1].float()).all()
    assert torch.equal(qs[0], qs[1])
    assert torch.equal(pools[0], pools[1])
    # and the product itself is right: rotate the float64 product on the host
    ref = x.double().cpu() @ w.double().cpu().t() + (b.double().cpu() if with_bias else 0.0)
    ref = ref.to(t).double().view(m, nh + 2 * nkv, hd)[:, :nh]
    ang = positions.cpu().double()[:, None] * inv_freq.cpu().double()[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, bb = ref[..., :hd // 2], ref[..., hd // 2:]
    want = torch.cat([a * cos - bb * sin, bb * cos + a * sin], dim=-1)
    assert float((qs[1].double().cpu() - want).abs().max()) < 3e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("requests,window", [(10, None), (20, None), (40, None), (40, 200), (150, None)])
def test_decode_attention_tma_cluster_sizes(requests, window):
    """The more (request, key/value head) pairs a step has, the fewer blocks share one pair's keys: clusters of 8,
    4, 2 and single blocks on a device of 148 SMs for 10, 20, 40 and more requests of 4 key/value heads.  Lengths
    sit around tile edges, some shorter than one tile a block; one request looks hard at a far key."""
    from zedinfer_b200 import ops
    t = torch.bfloat16
    nh, nkv, hd, ps = 8, 4, 64, 16
    base = [1, 15, 16, 17, 255, 256, 257, 700, 64, 513, 1500, 33, 2049]
    lens = [base[i % len(base)] + (i // len(base)) for i in range(requests)]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=21)
    g = torch.Generator().manual_seed(4)
    q = torch.randn(len(lens), nh, hd, generator=g)
    far = 5 if not window else 700 - window
    q[7, :, :] = ks[7][far, 0][None, :] * 4.0
    qd = q.to(t).to(dev())
    n = len(lens)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev())
    seg = torch.arange(n, dtype=torch.int32, device=dev())
    out = torch.empty(n, nh * hd, dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    ops.decode_attention_tma(qd, view, out, tables, seg, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    # token n is segment n here: without the segment array the kernel asks for its page numbers ahead of the position
    out2 = torch.full_like(out, float("nan"))
    ops.decode_attention_tma(qd, view, out2, tables, None, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    assert torch.equal(out, out2)
    got = out.float().cpu().view(n, nh, hd)
    qf = qd.float().cpu()
    for r in range(n):
        ref = plain_attention_rows(qf[r:r + 1], ks[r], vs[r], [lens[r] - 1], scale, window)
        assert float((got[r:r + 1] - ref).abs().max()) < 2e-2, (r, lens[r])


@pytest.mark.parametrize("batch", [1, 9])
@pytest.mark.parametrize("shared,window", [(False, None), (True, None), (True, 9000)])
def test_decode_attention_tma_long_context(batch, shared, window):
    """20,000 keys: every warp walks more tiles than the 32 page numbers it reads at a time, with tiles of 32 keys
    (one request: its clusters fit on the device at once) and of 16 keys (nine requests: they do not).  ``shared``:
    the call is told how long the longest context is, and several clusters share the long request's keys (sixteen
    for one request of 20,000 keys, eight inside a window of 9,000, four when nine requests are in the step) while the
    short requests of the same step keep one cluster each; a second kernel adds the parts."""
    from zedinfer_b200 import ops
    t = torch.bfloat16
    nh, nkv, hd, ps = 4, 1, 64, 16
    lens = [20000] + [300 + 7 * i for i in range(batch - 1)]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=12)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(len(lens), nh, hd, generator=g)
    q[0, :, :] = ks[0][17001, 0][None, :] * 4.0           # one far key must dominate
    qd = q.to(t).to(dev())
    n = len(lens)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev())
    seg = torch.arange(n, dtype=torch.int32, device=dev())
    out = torch.full((n, nh * hd), float("nan"), dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    ops.decode_attention_tma(qd, view, out, tables, seg, pos, nh, nkv, hd, ps, page_stride, kv_stride, window, scale,
                             max_kv_len=max(lens) if shared else 0)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    got = out.float().cpu().view(n, nh, hd)
    qf = qd.float().cpu()
    for r in range(n):
        ref = plain_attention_rows(qf[r:r + 1], ks[r], vs[r], [lens[r] - 1], scale, window)
        assert float((got[r:r + 1] - ref).abs().max()) < 2e-2, (r, lens[r])


@pytest.mark.parametrize("nkv,hd", [(1, 64), (2, 128)])
def test_decode_attention_tma_where_sharing_begins(nkv, hd):
    """Contexts on both sides of the length from which clusters share a request (and of the tile that holds it), in
    one step that is told the longest; each request's query points at one key near the end of its first quarter, which
    belongs to another cluster than the newest key as soon as the request is shared."""
    from zedinfer_b200 import ops
    t = torch.bfloat16
    nh, ps = 2 * nkv, 16
    edge = ops.decode_attention_split_from()
    lens = [edge - 17, edge - 1, edge, edge + 1, edge + 15, edge + 16, edge + 1030, 2 * edge - 1, 2 * edge + 5]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=21)
    n = len(lens)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(n, nh, hd, generator=g)
    for r, l in enumerate(lens):
        q[r, :, :] = ks[r][l // 4 - 3, 0][None, :] * 4.0
    qd = q.to(t).to(dev())
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev())
    out = torch.full((n, nh * hd), float("nan"), dtype=t, device=dev())
    scale = 1.0 / math.sqrt(hd)
    ops.decode_attention_tma(qd, view, out, tables, None, pos, nh, nkv, hd, ps, page_stride, kv_stride, None, scale,
                             max_kv_len=max(lens))
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
    got = out.float().cpu().view(n, nh, hd)
    qf = qd.float().cpu()
    for r in range(n):
        ref = plain_attention_rows(qf[r:r + 1], ks[r], vs[r], [lens[r] - 1], scale, None)
        assert float((got[r:r + 1] - ref).abs().max()) < 2e-2, (r, lens[r])


def _attention_args(nh, nkv, hd, ps, misalign=False):
    """Operands of a small step for the attention entry points: 3 requests, one token each."""
    t = torch.bfloat16
    lens = [40, 17, 100]
    pool, view, tables, ks, vs, page_stride, kv_stride = build_cache(len(lens), lens, nkv, hd, ps, t, seed=3)
    n = len(lens)
    store = torch.zeros(n * nh * hd + 8, dtype=t, device=dev())
    q = (store[1:1 + n * nh * hd] if misalign else store[:n * nh * hd]).view(n, nh, hd)     # 2 bytes off when asked
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev())
    seg = torch.arange(n, dtype=torch.int32, device=dev())
    tiles = torch.tensor([(i, 1, i) for i in range(n)], dtype=torch.int32, device=dev())
    out = torch.zeros(n, nh * hd, dtype=t, device=dev())
    return q, view, out, tables, seg, pos, tiles, page_stride, kv_stride


def test_attention_kernels_refuse_what_they_cannot_do():
    """A size that an attention entry point does not take is refused on the host with a message that names it;
    nothing is launched.  Head size 96 (the tensor-core kernels take 64 and 128), pages of 24 tokens (the TMA and
    tcgen05 forms take powers of two from 8 to 128), operands that are not 16-byte aligned, head counts that do not
    divide; the general kernel refuses a head size that is no multiple of 8."""
    from zedinfer_b200 import ops
    scale = 0.1
    q, view, out, tables, seg, pos, tiles, pst, kst = _attention_args(6, 2, 96, 16)
    for call, what in ((lambda: ops.decode_attention(q, view, out, tables, seg, pos, 6, 2, 96, 16, pst, kst, None, scale), "head_dim 64 or 128, got 96"),
                       (lambda: ops.decode_attention_tma(q, view, out, tables, seg, pos, 6, 2, 96, 16, pst, kst, None, scale), "head_dim 64 or 128, got 96"),
                       (lambda: ops.prefill_attention(q, view, out, tables, tiles, pos, 6, 2, 96, 16, pst, kst, None, scale), "head_dim 64 or 128, got 96"),
                       (lambda: ops.prefill_attention_tcgen05(q, view, out, tables, tiles, pos, 6, 2, 96, 16, pst, kst, None, scale), "head_dim 96 is not 64 or 128")):
        with pytest.raises(ops.KernelError, match=what):
            call()
    q, view, out, tables, seg, pos, tiles, pst, kst = _attention_args(4, 2, 64, 24)
    with pytest.raises(ops.KernelError, match="page size 24 is not a power of two from 8 to 128"):
        ops.decode_attention_tma(q, view, out, tables, seg, pos, 4, 2, 64, 24, pst, kst, None, scale)
    with pytest.raises(ops.KernelError, match="page size 24 is not a power of two from 8 to 128"):
        ops.prefill_attention_tcgen05(q, view, out, tables, tiles, pos, 4, 2, 64, 24, pst, kst, None, scale)
    ops.decode_attention(q, view, out, tables, seg, pos, 4, 2, 64, 24, pst, kst, None, scale)       # the cp.async form takes them
    ops.prefill_attention(q, view, out, tables, tiles, pos, 4, 2, 64, 24, pst, kst, None, scale)
    q, view, out, tables, seg, pos, tiles, pst, kst = _attention_args(4, 2, 64, 16, misalign=True)
    assert q.data_ptr() % 16 == 2
    with pytest.raises(ops.KernelError, match="16-byte aligned"):
        ops.decode_attention_tma(q, view, out, tables, seg, pos, 4, 2, 64, 16, pst, kst, None, scale)
    with pytest.raises(ops.KernelError, match="16-byte aligned"):
        ops.prefill_attention_tcgen05(q, view, out, tables, tiles, pos, 4, 2, 64, 16, pst, kst, None, scale)
    q, view, out, tables, seg, pos, tiles, pst, kst = _attention_args(5, 2, 64, 16)
    with pytest.raises(ops.KernelError, match="5 query heads cannot share 2 key/value heads"):
        ops.decode_attention_tma(q, view, out, tables, seg, pos, 5, 2, 64, 16, pst, kst, None, scale)
    with pytest.raises(ops.KernelError, match="5 heads over 2 key-value heads"):
        ops.prefill_attention_tcgen05(q, view, out, tables, tiles, pos, 5, 2, 64, 16, pst, kst, None, scale)
    q, view, out, tables, seg, pos, tiles, pst, kst = _attention_args(2, 1, 20, 16)
    with pytest.raises(ops.KernelError, match="head_dim=20 must be a multiple of 8"):
        ops.paged_attention(q, view, out, tables, seg, pos, 2, 1, 20, 16, pst, kst, None, scale)
    torch.cuda.synchronize()
    assert ops.tcgen05_status(dev()) == 0
