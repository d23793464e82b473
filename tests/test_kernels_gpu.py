"""Each kernel alone against a plain float32 restatement of the same operation,
at sizes other than the engine's (widths that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def ops():
    from tokenizer_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close_tensor_core_attention(got, want):
    """bfloat16 attention on tensor cores rounds the probabilities to bfloat16
    before they meet the values (2^-9 relative per term, so up to 2^-9 of the
    largest value in the sum), on top of the output's own rounding (2^-8)."""
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    bound = 6e-3 + 2 ** -7 * want.abs()
    assert bool((err <= bound).all()), f"max |diff| {float(err.max()):.4e} at {int(err.argmax())}"


def close(got, want, dtype):
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=2e-5, rtol=2e-5), float((got - want).abs().max())
    else:  # one rounding to bfloat16 of a value computed in float32
        assert torch.allclose(got, want, atol=1e-3, rtol=2 ** -7), float((got - want).abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = rnd(301, 70, dtype=dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 70, device=DEV)
    ops().embed(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [48, 200, 1030, 3000])
def test_rms_norm_with_pending_add_and_rows(dtype, hidden):
    x = rnd(7, hidden, seed=1, scale=3.0)
    delta = rnd(7, hidden, seed=2, dtype=dtype)
    gain = 1 + rnd(hidden, seed=3, scale=0.1)
    eps = 1e-5
    want_x = x + delta.float()
    want = want_x / torch.sqrt((want_x * want_x).mean(-1, keepdim=True) + eps) * gain
    out = torch.empty(7, hidden, dtype=dtype, device=DEV)
    x_run = x.clone()
    ops().rms_norm(x_run, gain, eps, out, delta=delta)
    assert torch.allclose(x_run, want_x, atol=1e-6)          # the sum is stored back in float32
    close(out, want, dtype)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out_rows = torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops().rms_norm(x_run, gain, eps, out_rows, rows=rows)
    close(out_rows, want[rows.long()], dtype)
    y = x.clone()
    ops().residual_add(y, delta)
    assert torch.allclose(y, want_x, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,rotary", [(5, 5, 48, 48), (6, 2, 16, 16), (3, 1, 80, 32), (14, 2, 64, 64)])
def test_rope_bias_and_cache_write(dtype, nh, nkv, d, rotary):
    o = ops()
    T, page, pages = 9, 4, 6
    theta = 1e4
    inv_freq = torch.tensor([1.0 / theta ** (i / rotary) for i in range(0, rotary, 2)],
                            dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 700)
    positions = torch.arange(700, dtype=torch.float32, device=DEV)[:, None] * inv_freq[None]
    assert torch.allclose(cos, torch.cos(positions), atol=2e-6)
    assert torch.allclose(sin, torch.sin(positions), atol=2e-6)
    qkv = rnd(T, (nh + 2 * nkv) * d, seed=4, dtype=dtype)
    bias = rnd((nh + 2 * nkv) * d, seed=5, scale=0.3)
    pos = torch.tensor([0, 1, 2, 3, 650, 651, 17, 5, 6], dtype=torch.int32, device=DEV)
    slot = torch.tensor([4, 5, 6, 7, 20, 21, 0, -1, 13], dtype=torch.int32, device=DEV)
    k_pool = torch.full((pages * page, nkv, d), 7.0, dtype=dtype, device=DEV)
    v_pool = torch.full((pages * page, nkv, d), 7.0, dtype=dtype, device=DEV)
    q_out = torch.empty(T, nh * d, dtype=dtype, device=DEV)
    o.rope_store(qkv, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, rotary)

    full = (qkv.float() + bias).view(T, nh + 2 * nkv, d)

    def rotate(x):  # x [T, heads, d]
        half = rotary // 2
        c, s = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
        x1, x2, rest = x[..., :half], x[..., half:rotary], x[..., rotary:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)

    close(q_out.view(T, nh, d), rotate(full[:, :nh]), dtype)
    k_want, v_want = rotate(full[:, nh:nh + nkv]), full[:, nh + nkv:]
    for t in range(T):
        if int(slot[t]) < 0:
            continue
        close(k_pool[int(slot[t])], k_want[t], dtype)
        close(v_pool[int(slot[t])], v_want[t], dtype)
    untouched = [s for s in range(pages * page) if s not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all()) and bool((v_pool[untouched] == 7.0).all())
    # a call that reads another layer's cache rotates q and writes no keys
    k2 = k_pool.clone()
    o.rope_store(qkv, bias, pos, None, cos, sin, q_out, None, None, nh, nkv, d, rotary)
    assert torch.equal(k2, k_pool)
    with pytest.raises(ValueError):
        o.rope_store(qkv, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, rotary + 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_gate(dtype):
    gu = rnd(5, 2 * 177, seed=6, dtype=dtype, scale=3.0)
    out = torch.empty(5, 177, dtype=dtype, device=DEV)
    ops().silu_gate(gu, out)
    g, u = gu.float()[:, :177], gu.float()[:, 177:]
    close(out, g * torch.sigmoid(g) * u, dtype)


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 130, 70), (65, 64, 17), (200, 301, 96), (2, 1000, 896)])
def test_gemm_f32_is_true_32_bit(M, N, K):
    a, w, bias = rnd(M, K, seed=7), rnd(N, K, seed=8), rnd(N, seed=9)
    out = torch.empty(M, N, device=DEV)
    ops().gemm_f32(a, w, bias, out)
    want = (a.double().cpu() @ w.double().cpu().t() + bias.double().cpu()).float()
    assert torch.allclose(out.cpu(), want, atol=1e-4 * math.sqrt(K) / 8, rtol=1e-5)
    # a row's result does not depend on the rows around it
    alone = torch.empty(1, N, device=DEV)
    ops().gemm_f32(a[M - 1:].contiguous(), w, bias, alone)
    assert torch.equal(alone[0], out[M - 1])


def paged_setup(lengths, nh, nkv, d, page, dtype, seed=10, shuffle=True):
    """Random keys and values for requests of the given lengths, scattered over
    pages in a shuffled order; returns pools, tables and the dense copies."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + page - 1) // page for n in lengths) + 3
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    k_pool = torch.full((n_pages * page, nkv, d), float("nan"), dtype=dtype)
    v_pool = torch.full((n_pages * page, nkv, d), float("nan"), dtype=dtype)
    width = max((n + page - 1) // page for n in lengths) + 1
    tables = torch.full((len(lengths), width), -1, dtype=torch.int32)
    dense = []
    for r, n in enumerate(lengths):
        k = torch.randn(n, nkv, d, generator=g).to(dtype)
        v = torch.randn(n, nkv, d, generator=g).to(dtype)
        for b in range((n + page - 1) // page):
            pg = order.pop()
            tables[r, b] = pg
            rows = slice(b * page, min(n, (b + 1) * page))
            k_pool[pg * page:pg * page + rows.stop - rows.start] = k[rows]
            v_pool[pg * page:pg * page + rows.stop - rows.start] = v[rows]
        dense.append((k.float(), v.float()))
    return k_pool.to(DEV), v_pool.to(DEV), tables.to(DEV), dense


def attention_reference(q, dense, row_req, pos, nh, nkv, window, scale):
    out = torch.zeros_like(q)
    for t in range(q.shape[0]):
        k, v = dense[row_req[t]]
        p = pos[t]
        lo = 0 if window is None else max(0, p - window)
        for h in range(nh):
            g = h // (nh // nkv)
            s = (k[lo:p + 1, g] @ q[t, h]) * scale
            out[t, h] = torch.softmax(s, 0) @ v[lo:p + 1, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 32, 24), (14, 2, 64, 16, None),
    (6, 3, 112, 4, 7), (2, 1, 256, 16, None)])
def test_paged_attention(dtype, nh, nkv, d, page, window):
    lengths = [1, 37, 130, 300]
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype)
    # rows: the last 3 positions of every request (a portion) and a few inner ones
    row_req, pos = [], []
    for r, n in enumerate(lengths):
        for p in sorted(set([max(0, n - 3), max(0, n - 2), n - 1, n // 2, min(n - 1, page - 1),
                             min(n - 1, page)])):
            row_req.append(r)
            pos.append(p)
    q = rnd(len(pos), nh, d, seed=11, dtype=dtype)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    ops().paged_attention_generic(
        q.view(len(pos), nh * d), k_pool, v_pool, out.view(len(pos), nh * d), tables,
        torch.tensor(row_req, dtype=torch.int32, device=DEV),
        torch.tensor(pos, dtype=torch.int32, device=DEV), nh, nkv, d, page, window, scale)
    want = attention_reference(q.float().cpu(), dense, row_req, pos, nh, nkv, window, scale)
    assert torch.isfinite(out.float()).all()       # unused slots (NaN) are never read
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_and_respects_the_window_edge(dtype):
    """One key among hundreds is made to stand out; the output must be its
    value.  With a window, a key exactly `window` back is seen, one further is not."""
    nh, nkv, d, page, n = 2, 1, 32, 16, 400
    k_pool, v_pool, tables, dense = paged_setup([n], nh, nkv, d, page, dtype, seed=12)
    scale = 1.0 / math.sqrt(d)
    q = rnd(1, nh, d, seed=13, dtype=dtype)
    for far in (0, 15, 16, 17, 255, 256, 399 - 25, 399 - 24, 399):
        k, v = dense[0]
        k, v = k.clone(), v.clone()
        k[far, 0] = (q[0, 0].float().cpu() * 40.0).to(dtype).float()   # score stands out for head 0
        pg, off = int(tables[0, far // page]), far % page
        k_pool2 = k_pool.clone()
        k_pool2[pg * page + off, 0] = k[far, 0].to(dtype).to(DEV)
        for window in (None, 24):
            out = torch.empty(1, nh * d, dtype=dtype, device=DEV)
            ops().paged_attention_generic(
                q.view(1, nh * d), k_pool2, v_pool, out, tables,
                torch.zeros(1, dtype=torch.int32, device=DEV),
                torch.tensor([n - 1], dtype=torch.int32, device=DEV), nh, nkv, d, page, window, scale)
            visible = window is None or far + window >= n - 1
            got = out.view(nh, d)[0].float().cpu()
            if visible:
                close(got, v[far, 0], dtype)
            else:
                assert float((got - v[far, 0]).abs().max()) > 0.1
            want = attention_reference(q.float().cpu(), [(k, v)], [0], [n - 1], nh, nkv, window, scale)
            close(out.view(1, nh, d), want, dtype)


def test_attention_refuses_sizes_it_cannot_take():
    q = torch.zeros(1, 6 * 16, device=DEV)
    pool = torch.zeros(16, 4, 16, device=DEV)
    table = torch.zeros(1, 1, dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="do not divide"):
        ops().paged_attention_generic(q, pool, pool, q.clone(), table, z, z, 6, 4, 16, 16, None, 1.0)
    with pytest.raises(ValueError, match="beyond 512"):
        ops().paged_attention_generic(q, pool, pool, q.clone(), table, z, z, 1, 1, 1024, 16, None, 1.0)


def test_argmax_ties_and_sampling_against_the_plain_rule():
    import plain_qwen2 as plain
    o = ops()
    V = 3001
    logits = rnd(6, V, seed=14, scale=2.0)
    logits[0, 17] = logits[0, 2900] = 50.0          # ties keep the lower id
    logits[1] = 0.0                                  # all equal: id 0
    logits[2, 3000] = 60.0                           # the last id
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    o.sample(logits, None, None, None, out)
    got = out.tolist()
    assert got[:3] == [17, 0, 3000]
    assert got == [plain.greedy_token(row) for row in logits.cpu()]

    rows = []
    for i, (temp, top_p) in enumerate([(0.8, 1.0), (0.8, 0.9), (1.5, 0.5), (0.3, 0.95), (1.0, 0.0),
                                       (0.0, 0.5), (2.0, 0.999)]):
        for u in (0.0, 0.013, 0.37, 0.5, 0.77, 0.999999):
            rows.append((i % 6, temp, top_p, u))
    batch = torch.stack([logits[r] for r, _, _, _ in rows])
    temps = torch.tensor([t for _, t, _, _ in rows], device=DEV)
    tops = torch.tensor([p for _, _, p, _ in rows], device=DEV)
    us = torch.tensor([u for _, _, _, u in rows], device=DEV)
    out = torch.empty(len(rows), dtype=torch.int32, device=DEV)
    o.sample(batch, temps, tops, us, out)
    for (r, temp, top_p, u), token in zip(rows, out.tolist()):
        row = logits[r].cpu()
        if temp == 0.0:
            assert token == plain.greedy_token(row)
            continue
        kept, mass = plain.sample_intervals(row, temp, top_p)
        assert token in kept, (temp, top_p, u, token)
        # the drawn id's interval in the walking order holds u * kept weight (float32 sums
        # differ in order, so allow the width of a few roundings of the total)
        at = kept.index(token)
        total = sum(mass)
        before = sum(mass[:at])
        slack = 1e-5 * total
        assert before - slack <= u * total < before + mass[at] + slack, (temp, top_p, u, token)
    # top_p 0 keeps only the best id whatever the draw
    assert all(t == plain.greedy_token(logits[r].cpu()) for (r, temp, p, u), t in zip(rows, out.tolist())
               if p == 0.0 and temp > 0)


def test_sampling_follows_the_distribution():
    o = ops()
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 3.0]], device=DEV).repeat(4000, 1).contiguous()
    temps = torch.full((4000,), 0.7, device=DEV)
    tops = torch.ones(4000, device=DEV)
    us = torch.rand(4000, generator=torch.Generator().manual_seed(3)).to(DEV)
    out = torch.empty(4000, dtype=torch.int32, device=DEV)
    o.sample(logits, temps, tops, us, out)
    freq = torch.bincount(out.long().cpu(), minlength=5).float() / 4000
    want = torch.softmax(logits[0].cpu() / 0.7, 0)
    assert float((freq - want).abs().max()) < 0.03


def test_advance_decode():
    o = ops()
    page = 4
    ids = torch.tensor([5, 6, 0, 0], dtype=torch.int32, device=DEV)
    drawn = torch.tensor([9, 8, 7, 7], dtype=torch.int32, device=DEV)
    pos = torch.tensor([2, 7, 0, 0], dtype=torch.int32, device=DEV)
    kv = torch.tensor([3, 8, 0, 0], dtype=torch.int32, device=DEV)
    row_req = torch.tensor([0, 1, -1, -1], dtype=torch.int32, device=DEV)
    slots = torch.tensor([4 * 3 + 2, 4 * 1 + 3, -1, -1], dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, -1, -1], [5, 1, 6], [-1, -1, -1], [-1, -1, -1]], dtype=torch.int32, device=DEV)
    history = torch.zeros(3 * 4, dtype=torch.int32, device=DEV)
    counter = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.advance_decode(ids, drawn, pos, kv, row_req, [slots], [table], page, history, counter)
    assert ids.tolist() == [9, 8, 0, 0] and pos.tolist() == [3, 8, 0, 0] and kv.tolist() == [4, 9, 0, 0]
    assert slots.tolist() == [4 * 3 + 3, 4 * 6 + 0, -1, -1]
    assert int(counter) == 1 and history.tolist()[:4] == [9, 8, 0, 0]
    o.advance_decode(ids, drawn, pos, kv, row_req, [slots], [table], page, history, counter)
    assert slots.tolist()[0] == -1 and history.tolist()[4:6] == [9, 8] and int(counter) == 2


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 32, 24), (14, 2, 64, 16, None),
    (6, 3, 112, 4, 7), (8, 1, 256, 16, None), (7, 1, 64, 16, 100), (12, 2, 128, 64, None),
    (16, 1, 32, 16, None), (24, 2, 64, 16, None), (9, 1, 80, 16, None)])
def test_decode_attention_splits_and_merges(nh, nkv, d, page, window):
    """The split-key kernel: one row per request at the request's last position
    (one split, several splits, pieces longer than a tile), idle rows skipped."""
    dtype = torch.bfloat16
    lengths = [1, 2, 63, 64, 65, 130, 700, 2500]
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=21)
    row_req = list(range(len(lengths))) + [-1, 3]
    pos = [n - 1 for n in lengths] + [0, 40]
    q = rnd(len(pos), nh, d, seed=22, dtype=dtype)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(d)
    for _ in range(2):          # twice: the merge counters must be left ready
        ops().decode_attention(
            q.view(len(pos), nh * d), k_pool, v_pool, out.view(len(pos), nh * d), tables,
            torch.tensor(row_req, dtype=torch.int32, device=DEV),
            torch.tensor(pos, dtype=torch.int32, device=DEV), nh, nkv, d, page, window, scale)
        live = [i for i, r in enumerate(row_req) if r >= 0]
        want = attention_reference(q.float().cpu()[live], dense, [row_req[i] for i in live],
                                   [pos[i] for i in live], nh, nkv, window, scale)
        assert torch.isfinite(out.float()).all()
        close_tensor_core_attention(out[live], want)
        assert bool((out[len(lengths)] == 9.0).all())     # the idle row is not written
        out.fill_(9.0)


@pytest.mark.parametrize("nh,nkv,d", [(14, 2, 64), (28, 4, 128)])
def test_decode_attention_with_64_rows_of_8192_keys(nh, nkv, d):
    """The benchmark's widest decoding shape: 64 rows whose block tables hold 512 pages, most of
    them near 8,192 keys and a few short ones between (the length of a row's pieces doubles
    with its keys; pieces beyond a cluster's eight meet through scratch)."""
    dtype, page = torch.bfloat16, 16
    lengths = [8192 - 61 * i for i in range(56)] + [1, 17, 255, 256, 257, 1000, 3000, 5000]
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=31)
    assert tables.shape[1] > 512
    pos = [n - 1 for n in lengths]
    q = rnd(64, nh, d, seed=32, dtype=dtype)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(d)
    for _ in range(2):
        ops().decode_attention(
            q.view(64, nh * d), k_pool, v_pool, out.view(64, nh * d), tables,
            torch.arange(64, dtype=torch.int32, device=DEV),
            torch.tensor(pos, dtype=torch.int32, device=DEV), nh, nkv, d, page, None, scale)
        want = attention_reference(q.float().cpu(), dense, list(range(64)), pos, nh, nkv, None, scale)
        assert torch.isfinite(out.float()).all()
        close_tensor_core_attention(out, want)
        out.fill_(9.0)


def test_decode_attention_serves_only_the_rows_it_is_given():
    """With a list of rows (the single-token rows of a step that also brings portions), the
    kernel serves those rows and leaves every other row of the output alone."""
    nh, nkv, d, page, dtype = 12, 2, 128, 16, torch.bfloat16
    lengths = [700, 33, 1300, 5]
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=25)
    # ten batch rows: rows 2, 7, 8 and 4 are the last positions of the four requests
    row_req = [-1, -1, 0, -1, 3, -1, -1, 1, 2, -1]
    pos = [0, 0, 699, 0, 4, 0, 0, 32, 1299, 0]
    rows = torch.tensor([8, 2, -1, 7, 4, -1, -1, -1], dtype=torch.int32, device=DEV)
    q = rnd(10, nh, d, seed=26, dtype=dtype)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(d)
    for _ in range(2):
        ops().decode_attention(q.view(10, nh * d), k_pool, v_pool, out.view(10, nh * d), tables,
                               torch.tensor(row_req, dtype=torch.int32, device=DEV),
                               torch.tensor(pos, dtype=torch.int32, device=DEV), nh, nkv, d, page, None, scale,
                               rows=rows)
        live = [2, 4, 7, 8]
        want = attention_reference(q.float().cpu()[live], dense, [row_req[i] for i in live],
                                   [pos[i] for i in live], nh, nkv, None, scale)
        close_tensor_core_attention(out[live], want)
        idle = [i for i in range(10) if i not in live]
        assert bool((out[idle] == 9.0).all())
        out.fill_(9.0)


def test_decode_attention_far_key_across_splits():
    nh, nkv, d, page, n = 7, 1, 64, 16, 1500
    dtype = torch.bfloat16
    k_pool, v_pool, tables, dense = paged_setup([n], nh, nkv, d, page, dtype, seed=23)
    q = rnd(1, nh, d, seed=24, dtype=dtype)
    scale = 1.0 / math.sqrt(d)
    for far in (0, 63, 64, 640, 1499 - 200, 1499 - 201, 1499):
        k, v = dense[0][0].clone(), dense[0][1]
        k[far, 0] = (q[0, 3].float().cpu() * 30.0).to(dtype).float()
        k_pool2 = k_pool.clone()
        k_pool2[int(tables[0, far // page]) * page + far % page, 0] = k[far, 0].to(dtype).to(DEV)
        for window in (None, 200):
            out = torch.empty(1, nh * d, dtype=dtype, device=DEV)
            ops().decode_attention(q.view(1, nh * d), k_pool2, v_pool, out, tables,
                                   torch.zeros(1, dtype=torch.int32, device=DEV),
                                   torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                   nh, nkv, d, page, window, scale)
            want = attention_reference(q.float().cpu(), [(k, v)], [0], [n - 1], nh, nkv, window, scale)
            close_tensor_core_attention(out.view(1, nh, d), want)
            if window is None or far + window >= n - 1:
                close_tensor_core_attention(out.view(nh, d)[3], v[far, 0])


def test_decode_attention_refuses_groups_it_cannot_hold():
    assert not ops().decode_attention_supported(34, 2, 64)     # 17 heads to a group
    assert not ops().decode_attention_supported(4, 2, 24)
    assert ops().decode_attention_supported(14, 2, 64)


@pytest.mark.parametrize("M,N,K", [(1, 16, 32), (3, 130, 72), (8, 1152, 896), (8, 896, 4864), (5, 301, 96),
                                   (16, 64, 64), (17, 200, 176), (33, 1000, 256), (64, 896, 896),
                                   (8, 20000, 96), (2, 896, 1000),
                                   # 9 to 16 rows: the form held to 80 registers (small weights) and the other
                                   (12, 1152, 896), (12, 20000, 96), (16, 4000, 3584),
                                   # large weights
                                   (5, 3584, 18944), (13, 9001, 1032), (1, 152064, 1536)])
def test_linear_small_m(M, N, K):
    """The streaming product for few rows against float64, bfloat16 and float32
    results, with a bias, and cut along k into partial sums."""
    o = ops()
    x = rnd(M, K, seed=31, dtype=torch.bfloat16)
    w = rnd(N, K, seed=32, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=33)
    want = x.double().cpu() @ w.double().cpu().t()
    out32 = torch.empty(M, N, device=DEV)
    o.linear_small_m(x, w, None, out32)
    tol = 2e-5 * float(want.abs().max()) + 1e-6 * K
    assert float((out32.double().cpu() - want).abs().max()) <= tol
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    o.linear_small_m(x, w, bias, out16)
    close(out16, (want + bias.double().cpu()).float(), torch.bfloat16)
    for splits in (2, 5):
        parts = torch.full((splits, M, N), 7.0, device=DEV)
        o.linear_small_m(x, w, None, parts, k_splits=splits)
        assert float((parts.sum(0).double().cpu() - want).abs().max()) <= tol
    again = torch.empty(M, N, device=DEV)
    o.linear_small_m(x, w, None, again)
    assert torch.equal(again, out32)            # fixed order of sums: reproducible
    with pytest.raises(ValueError):
        o.linear_small_m(rnd(65, K, dtype=torch.bfloat16), w, None, torch.empty(65, N, device=DEV))


@pytest.mark.parametrize("M,N,K,splits", [(1, 4000, 3584, (1, 2)), (8, 3584, 18944, (3, 4)), (13, 9001, 1032, (1,)),
                                          (16, 20011, 1536, (1, 2)), (5, 50, 512, (1,)), (9, 3584, 3584, (3, 5)),
                                          (17, 896, 4864, (3, 5)), (32, 1536, 8960, (6,)), (29, 1000, 1032, (1,))])
def test_linear_ring(M, N, K, splits):
    """The product of few rows for large weights (one block a multiprocessor, the weights through
    rings in shared memory) against float64: k cut in pieces, a k that ends inside a step of 64,
    row counts that end inside a tile, fewer tiles than blocks, twice for the same bits."""
    o = ops()
    x = rnd(M, K, seed=131, dtype=torch.bfloat16)
    w = rnd(N, K, seed=132, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=133)
    want = x.double().cpu() @ w.double().cpu().t()
    tol = 2e-5 * float(want.abs().max()) + 1e-6 * K
    for s in splits:
        assert o.linear_ring_supported(M, N, K, s), (M, N, K, s)
        if s == 1:
            out32 = torch.full((M, N), 7.0, device=DEV)
            o.linear_ring(x, w, None, out32)
            assert float((out32.double().cpu() - want).abs().max()) <= tol
            again = torch.full((M, N), 3.0, device=DEV)
            o.linear_ring(x, w, None, again)
            assert torch.equal(again, out32)
            out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            o.linear_ring(x, w, bias, out16)
            close(out16, (want + bias.double().cpu()).float(), torch.bfloat16)
        else:
            parts = torch.full((s, M, N), 7.0, device=DEV)
            o.linear_ring(x, w, None, parts, k_splits=s)
            assert float((parts.sum(0).double().cpu() - want).abs().max()) <= tol, s
    assert not o.linear_ring_supported(33, N, K) and not o.linear_ring_supported(M, N, 100)
    assert not o.linear_ring_supported(M, N, K, 64)


@pytest.mark.parametrize("M,inner,K", [(1, 8960, 1536), (8, 18944, 3584), (14, 5120, 1032), (16, 256, 512),
                                       (17, 4864, 896), (32, 8960, 1536), (25, 640, 520)])
def test_linear_ring_gated(M, inner, K):
    o = ops()
    x = rnd(M, K, seed=141, dtype=torch.bfloat16)
    gate = rnd(inner, K, seed=142, dtype=torch.bfloat16, scale=0.1)
    up = rnd(inner, K, seed=143, dtype=torch.bfloat16, scale=0.1)
    w = o.interleave_gate_up(gate, up)
    assert o.linear_ring_supported(M, 2 * inner, K, 1, True)
    out = torch.full((M, inner), 7.0, dtype=torch.bfloat16, device=DEV)
    o.linear_ring_gated(x, w, out)
    torch.cuda.synchronize()
    g = x.double().cpu() @ gate.double().cpu().t()
    u = x.double().cpu() @ up.double().cpu().t()
    close(out, (g * torch.sigmoid(g) * u).float(), torch.bfloat16)


def test_norm_adds_partial_sums():
    x = rnd(5, 200, seed=41)
    parts = rnd(3, 5, 200, seed=42)
    gain = 1 + rnd(200, seed=43, scale=0.1)
    want_x = x + parts.sum(0)
    out = torch.empty(5, 200, device=DEV)
    x1 = x.clone()
    ops().rms_norm(x1, gain, 1e-6, out, delta=parts)
    assert torch.allclose(x1, want_x, atol=1e-6)
    want = want_x / torch.sqrt((want_x * want_x).mean(-1, keepdim=True) + 1e-6) * gain
    assert torch.allclose(out, want, atol=2e-5)
    x2 = x.clone()
    ops().residual_add(x2, parts)
    assert torch.allclose(x2, want_x, atol=1e-6)


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 32, 24), (14, 2, 64, 16, None),
    (6, 3, 112, 4, 7), (4, 1, 128, 16, None), (2, 2, 64, 16, 100)])
def test_prefill_attention_tiles(nh, nkv, d, page, window):
    """The tensor-core kernel for portions of prompts: portions that start at 0 and
    in the middle of a page, of 1, 2, 63, 64, 65 and 200 rows, beside single rows."""
    dtype = torch.bfloat16
    lengths = [1, 2, 70, 64, 129, 333, 520]
    starts = [0, 0, 7, 0, 64, 133, 519]          # the portion is start .. length - 1
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=51)
    row_req, pos, tiles = [], [], []
    for r, (n, s0) in enumerate(zip(lengths, starts)):
        first = len(pos)
        for p in range(s0, n):
            row_req.append(r)
            pos.append(p)
        for off in range(0, n - s0, 64):
            tiles.append([first + off, min(64, n - s0 - off)])
    q = rnd(len(pos), nh, d, seed=52, dtype=dtype)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(d)
    tiles_t = torch.tensor(tiles + [[0, 0]], dtype=torch.int32, device=DEV)
    ops().prefill_attention(
        q.view(len(pos), nh * d), k_pool, v_pool, out.view(len(pos), nh * d), tables,
        torch.tensor(row_req, dtype=torch.int32, device=DEV),
        torch.tensor(pos, dtype=torch.int32, device=DEV), tiles_t, len(tiles), nh, nkv, d, page,
        window, scale)
    want = attention_reference(q.float().cpu(), dense, row_req, pos, nh, nkv, window, scale)
    assert torch.isfinite(out.float()).all()
    got = out.float().cpu()
    # probabilities are rounded to bfloat16 before they meet the values (2^-9 relative
    # per term), on top of the output's own rounding
    err = (got - want).abs()
    bound = 6e-3 + 2 ** -7 * want.abs()
    bad = (err > bound).nonzero()
    assert bad.numel() == 0, (
        f"first wrong row {int(bad[0][0])} (request {row_req[int(bad[0][0])]}, "
        f"position {pos[int(bad[0][0])]}): {float(err.max())}")


def test_prefill_attention_far_key_and_window_edge():
    nh, nkv, d, page, n = 2, 1, 64, 16, 400
    dtype = torch.bfloat16
    k_pool, v_pool, tables, dense = paged_setup([n], nh, nkv, d, page, dtype, seed=53)
    rows = 70                                   # positions 330 .. 399 in one portion
    q = rnd(rows, nh, d, seed=54, dtype=dtype)
    scale = 1.0 / math.sqrt(d)
    tiles = torch.tensor([[0, 64], [64, 6]], dtype=torch.int32, device=DEV)
    pos = list(range(n - rows, n))
    for far in (0, 63, 64, 200, 399 - 30, 399 - 31, 335):
        k, v = dense[0][0].clone(), dense[0][1]
        k[far, 0] = (q[rows - 1, 0].float().cpu() * 40.0).to(dtype).float()   # for the last row, head 0
        k_pool2 = k_pool.clone()
        k_pool2[int(tables[0, far // page]) * page + far % page, 0] = k[far, 0].to(dtype).to(DEV)
        for window in (None, 30):
            out = torch.empty(rows, nh * d, dtype=dtype, device=DEV)
            ops().prefill_attention(q.view(rows, nh * d), k_pool2, v_pool, out, tables,
                                    torch.zeros(rows, dtype=torch.int32, device=DEV),
                                    torch.tensor(pos, dtype=torch.int32, device=DEV), tiles, 2,
                                    nh, nkv, d, page, window, scale)
            got = out.view(rows, nh, d)[rows - 1, 0].float().cpu()
            if window is None or far + window >= n - 1:
                assert float((got - v[far, 0]).abs().max()) < 0.03
            else:
                assert float((got - v[far, 0]).abs().max()) > 0.1


@pytest.mark.parametrize("M,N,K,block_n", [
    (128, 128, 64, 128), (130, 70, 72, 64), (65, 300, 96, 128), (257, 1000, 200, 0),
    (512, 1152, 896, 128), (300, 2304, 896, 256), (1024, 896, 4864, 0), (200, 301, 1000, 0)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(M, N, K, block_n, out_dtype):
    """The tcgen05/TMEM/TMA product against float64: tiles cut by M, N and K (TMA
    fills what lies outside with zeros), with and without a bias."""
    o = ops()
    a = rnd(M, K, seed=61, dtype=torch.bfloat16)
    w = rnd(N, K, seed=62, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=63)
    want = a.double().cpu() @ w.double().cpu().t()
    for b in (None, bias):
        out = torch.full((M, N), 7.0, dtype=out_dtype, device=DEV)
        o.gemm_tcgen05(a, w, b, out, block_n)
        torch.cuda.synchronize()
        o.gemm_tcgen05_check()
        ref = (want + (b.double().cpu() if b is not None else 0)).float()
        if out_dtype == torch.float32:
            assert float((out.cpu() - ref).abs().max()) <= 2e-5 * float(ref.abs().max()) + 1e-6 * K
        else:
            close(out, ref, torch.bfloat16)
    with pytest.raises(ValueError):
        o.gemm_tcgen05(rnd(M, 12, dtype=torch.bfloat16), rnd(N, 12, dtype=torch.bfloat16), None,
                       torch.empty(M, N, dtype=out_dtype, device=DEV))


@pytest.mark.parametrize("M,inner,K", [(1, 128, 64), (8, 256, 96), (5, 4864, 896), (33, 384, 200),
                                       (64, 128, 72), (65, 128, 64), (300, 640, 896), (2048, 1280, 128),
                                       (17, 4864, 896), (47, 640, 200), (64, 8960, 1536), (8, 8960, 1536), (14, 5120, 1032)])
def test_gated_linear(M, inner, K):
    """Gate and up products with silu(gate) * up folded into the epilogue, for few
    rows (streaming kernel) and many (tcgen05), from the interleaved weight."""
    o = ops()
    x = rnd(M, K, seed=71, dtype=torch.bfloat16)
    gate = rnd(inner, K, seed=72, dtype=torch.bfloat16, scale=0.2)
    up = rnd(inner, K, seed=73, dtype=torch.bfloat16, scale=0.2)
    w = o.interleave_gate_up(gate, up)
    assert w.shape == (2 * inner, K)
    assert torch.equal(w[:128], gate[:128]) and torch.equal(w[128:256], up[:128])
    out = torch.full((M, inner), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gated_linear(x, w, out)
    torch.cuda.synchronize()
    if M > 64:
        o.gemm_tcgen05_check()
    g = x.double().cpu() @ gate.double().cpu().t()
    u = x.double().cpu() @ up.double().cpu().t()
    want = (g * torch.sigmoid(g) * u).float()
    if 16 < M <= 64:
        # this range runs the plain product and then the activation: gate and up are
        # rounded to bfloat16 on the way (three roundings of 2^-9 instead of one)
        got = out.float().cpu()
        assert torch.allclose(got, want, atol=4e-3, rtol=2 ** -6), float((got - want).abs().max())
    else:
        close(out, want, torch.bfloat16)
    with pytest.raises(ValueError):
        o.gated_linear(x, w[:-8], torch.empty(M, inner - 4, dtype=torch.bfloat16, device=DEV))


def activation_reference(name, g):
    if name == "silu":
        return g * torch.sigmoid(g)
    if name == "relu":
        return torch.clamp(g, min=0.0)
    return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))


@pytest.mark.parametrize("activation", ["gelu_pytorch_tanh", "relu"])
def test_the_activation_is_a_parameter_of_every_gated_kernel(activation):
    """Another activation than the served model's through every kernel that applies one: the
    separate gate kernel (both precisions), the gated product of few rows, of a few dozen
    (plain product, then the gate kernel for the interleaved layout), of hundreds (tcgen05
    epilogue, lone CTAs and pairs), and the fused feed-forward of a decoding step."""
    o = ops()
    inner, K = 384, 200
    gate = rnd(inner, K, seed=72, dtype=torch.bfloat16, scale=0.2)
    up = rnd(inner, K, seed=73, dtype=torch.bfloat16, scale=0.2)
    w = o.interleave_gate_up(gate, up)
    for M in (5, 40, 130, 300):
        x = rnd(M, K, seed=70 + M, dtype=torch.bfloat16)
        out = torch.full((M, inner), 7.0, dtype=torch.bfloat16, device=DEV)
        o.gated_linear(x, w, out, activation)
        torch.cuda.synchronize()
        g = x.double().cpu() @ gate.double().cpu().t()
        u = x.double().cpu() @ up.double().cpu().t()
        want = (activation_reference(activation, g) * u).float()
        got = out.float().cpu()
        assert torch.allclose(got, want, atol=4e-3, rtol=2 ** -6), (M, float((got - want).abs().max()))
    o.gemm_tcgen05_check()
    for dtype in (torch.float32, torch.bfloat16):
        gu = rnd(7, 2 * 100, seed=5, dtype=dtype)
        out = torch.empty(7, 100, dtype=dtype, device=DEV)
        o.silu_gate(gu, out, activation)
        g, u = gu.double().cpu()[:, :100], gu.double().cpu()[:, 100:]
        close(out, (activation_reference(activation, g) * u).float(), dtype)
    with pytest.raises(ValueError, match="activations"):
        o.silu_gate(gu, out, "swish-ish")
    # the fused feed-forward
    M, hidden, inner = 6, 160, 384
    splits = o.ffn_small_m_splits(M, hidden, inner)
    x = rnd(M, hidden, seed=81)
    gain = 1.0 + rnd(hidden, seed=83, scale=0.1)
    gate = rnd(inner, hidden, seed=84, dtype=torch.bfloat16, scale=0.06)
    up = rnd(inner, hidden, seed=85, dtype=torch.bfloat16, scale=0.06)
    down = rnd(hidden, inner, seed=86, dtype=torch.bfloat16, scale=0.04)
    xs = x.double().cpu()
    h = (xs / torch.sqrt((xs * xs).mean(-1, keepdim=True) + 1e-5) * gain.double().cpu()).float().to(torch.bfloat16).double()
    g, u = h @ gate.double().cpu().t(), h @ up.double().cpu().t()
    act = (activation_reference(activation, g) * u).float().to(torch.bfloat16).double()
    want = (act @ down.double().cpu().t()).float()
    x_out = torch.empty_like(x)
    out = torch.zeros((splits, M, hidden), dtype=torch.float32, device=DEV)
    o.ffn_small_m(x, x_out, None, gain, 1e-5, o.interleave_gate_up(gate, up), down, out, activation)
    torch.cuda.synchronize()
    o.ffn_small_m_check()
    got = out.sum(0).cpu()
    assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max()) + 1e-5


@pytest.mark.parametrize("M,nh,nkv,d,K", [(1, 4, 2, 16, 64), (8, 14, 2, 64, 896), (5, 3, 1, 32, 96),
                                           (16, 5, 5, 48, 80), (3, 2, 1, 128, 200), (32, 14, 2, 64, 896),
                                           (23, 3, 3, 16, 72)])
def test_qkv_projection_with_rope_and_cache_write_folded_in(M, nh, nkv, d, K):
    """The decoding step's q/k/v kernel against the unfused pieces' arithmetic:
    product + bias in float64, rotation by the float32 tables, rows scattered to
    their cache slots; one row writes no cache."""
    o = ops()
    heads = nh + 2 * nkv
    x = rnd(M, K, seed=81, dtype=torch.bfloat16)
    w = rnd(heads * d, K, seed=82, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(heads * d, seed=83, scale=0.3)
    inv_freq = torch.tensor([1.0 / 1e4 ** (i / d) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 900)
    pos = torch.tensor([(37 * i + 5) % 900 for i in range(M)], dtype=torch.int32, device=DEV)
    slot = torch.tensor([2 * i + 1 for i in range(M)], dtype=torch.int32, device=DEV)
    if M > 1:
        slot[M - 1] = -1
    k_pool = torch.full((2 * M + 2, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((2 * M + 2, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(M, nh * d, dtype=torch.bfloat16, device=DEV)
    o.qkv_rope_small_m(x, w, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d)
    full = (x.double().cpu() @ w.double().cpu().t() + bias.double().cpu()).float().view(M, heads, d)
    c, s = cos[pos.long()].cpu()[:, None, :], sin[pos.long()].cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :d // 2], v[..., d // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    close(q_out.view(M, nh, d), rotate(full[:, :nh]), torch.bfloat16)
    k_want, v_want = rotate(full[:, nh:nh + nkv]), full[:, nh + nkv:]
    for m in range(M):
        if int(slot[m]) < 0:
            continue
        close(k_pool[int(slot[m])], k_want[m], torch.bfloat16)
        close(v_pool[int(slot[m])], v_want[m], torch.bfloat16)
    untouched = [i for i in range(2 * M + 2) if i not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all()) and bool((v_pool[untouched] == 7.0).all())


@pytest.mark.parametrize("hidden", [64, 896, 1000, 8192])
def test_rms_norm_many_rows_vector_path(hidden):
    rows = 100
    x = rnd(rows, hidden, seed=91, scale=2.0)
    delta = rnd(rows, hidden, seed=92, dtype=torch.bfloat16)
    gain = 1 + rnd(hidden, seed=93, scale=0.1)
    want_x = x + delta.float()
    want = want_x / torch.sqrt((want_x * want_x).mean(-1, keepdim=True) + 1e-6) * gain
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
    x1 = x.clone()
    ops().rms_norm(x1, gain, 1e-6, out, delta=delta)
    assert torch.allclose(x1, want_x, atol=1e-6)
    close(out, want, torch.bfloat16)
    out2 = torch.empty_like(out)
    ops().rms_norm(x1, gain, 1e-6, out2)
    close(out2, want, torch.bfloat16)


@pytest.mark.parametrize("rows", [100, 17])
@pytest.mark.parametrize("hidden,S", [(64, 1), (896, 2), (896, 5), (1000, 4), (8192, 3), (132, 2)])
def test_rms_norm_many_rows_of_partial_sums(hidden, S, rows):
    """Many rows whose pending residual is float32 partial sums [S, rows, hidden]: the planes are
    added in index order (the sum below adds them the same way), the stream is updated, the
    output is bfloat16.  132 is no multiple of 8: the general kernel."""
    x = rnd(rows, hidden, seed=94, scale=2.0)
    delta = rnd(S, rows, hidden, seed=95, scale=0.7)
    gain = 1 + rnd(hidden, seed=96, scale=0.1)
    want_x = x.clone()
    for s in range(S):
        want_x = want_x + delta[s]
    want = want_x / torch.sqrt((want_x * want_x).mean(-1, keepdim=True) + 1e-6) * gain
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
    x1 = x.clone()
    ops().rms_norm(x1, gain, 1e-6, out, delta=delta)
    assert torch.equal(x1, want_x)
    close(out, want, torch.bfloat16)


@pytest.mark.parametrize("nh,nkv,d", [(14, 2, 64), (5, 5, 48), (3, 1, 128), (4, 2, 16)])
def test_rope_store_many_rows_vector_path(nh, nkv, d):
    o = ops()
    T = 130
    inv_freq = torch.tensor([1.0 / 1e6 ** (i / d) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 3000)
    qkv = rnd(T, (nh + 2 * nkv) * d, seed=94, dtype=torch.bfloat16)
    bias = rnd((nh + 2 * nkv) * d, seed=95, scale=0.3)
    pos = torch.arange(1500, 1500 + T, dtype=torch.int32, device=DEV)
    slot = torch.randperm(T + 10, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32).to(DEV)
    slot[7] = -1
    k_pool = torch.full((T + 10, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((T + 10, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=DEV)
    o.rope_store(qkv, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, d)
    full = (qkv.float() + bias).view(T, nh + 2 * nkv, d).cpu()
    c, s = cos[pos.long()].cpu()[:, None, :], sin[pos.long()].cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :d // 2], v[..., d // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    close(q_out.view(T, nh, d), rotate(full[:, :nh]), torch.bfloat16)
    k_want, v_want = rotate(full[:, nh:nh + nkv]), full[:, nh + nkv:]
    live = [t for t in range(T) if int(slot[t]) >= 0]
    close(k_pool[slot[live].long()], k_want[live], torch.bfloat16)
    close(v_pool[slot[live].long()], v_want[live], torch.bfloat16)
    untouched = [i for i in range(T + 10) if i not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all())


@pytest.mark.parametrize("nh,nkv,d,page,window", [
    (4, 2, 64, 16, None), (14, 2, 64, 16, None), (3, 1, 64, 8, 100), (4, 1, 128, 16, None),
    (6, 3, 128, 32, 40), (2, 2, 64, 64, None)])
def test_attention_tcgen05_tiles(nh, nkv, d, page, window):
    """The tcgen05 kernel for portions of prompts: portions that start at 0 and in the
    middle of a page, of 1 to 400 rows (tiles of up to 128), beside single rows."""
    dtype = torch.bfloat16
    lengths = [1, 2, 70, 128, 129, 333, 520, 900]
    starts = [0, 0, 7, 0, 64, 133, 519, 500]
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=101)
    row_req, pos, tiles = [], [], []
    for r, (n, s0) in enumerate(zip(lengths, starts)):
        first = len(pos)
        for p in range(s0, n):
            row_req.append(r)
            pos.append(p)
        for off in range(0, n - s0, 128):
            tiles.append([first + off, min(128, n - s0 - off)])
    q = rnd(len(pos), nh, d, seed=102, dtype=dtype)
    out = torch.full_like(q, 9.0)
    scale = 1.0 / math.sqrt(d)
    ops().attention_tcgen05(
        q.view(len(pos), nh * d), k_pool, v_pool, out.view(len(pos), nh * d), tables,
        torch.tensor(row_req, dtype=torch.int32, device=DEV),
        torch.tensor(pos, dtype=torch.int32, device=DEV),
        torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles), nh, nkv, d, page, window, scale)
    torch.cuda.synchronize()
    ops().attention_tcgen05_check(d)
    want = attention_reference(q.float().cpu(), dense, row_req, pos, nh, nkv, window, scale)
    assert torch.isfinite(out.float()).all()
    close_tensor_core_attention(out, want)


def test_attention_tcgen05_far_key_and_window_edge():
    nh, nkv, d, page, n = 2, 1, 64, 16, 700
    dtype = torch.bfloat16
    k_pool, v_pool, tables, dense = paged_setup([n], nh, nkv, d, page, dtype, seed=103)
    rows = 150
    q = rnd(rows, nh, d, seed=104, dtype=dtype)
    scale = 1.0 / math.sqrt(d)
    tiles = torch.tensor([[0, 128], [128, 22]], dtype=torch.int32, device=DEV)
    pos = list(range(n - rows, n))
    for far in (0, 127, 128, 300, 699 - 30, 699 - 31, 640):
        k, v = dense[0][0].clone(), dense[0][1]
        k[far, 0] = (q[rows - 1, 0].float().cpu() * 40.0).to(dtype).float()
        k_pool2 = k_pool.clone()
        k_pool2[int(tables[0, far // page]) * page + far % page, 0] = k[far, 0].to(dtype).to(DEV)
        for window in (None, 30):
            out = torch.empty(rows, nh * d, dtype=dtype, device=DEV)
            ops().attention_tcgen05(q.view(rows, nh * d), k_pool2, v_pool, out, tables,
                                    torch.zeros(rows, dtype=torch.int32, device=DEV),
                                    torch.tensor(pos, dtype=torch.int32, device=DEV), tiles, 2,
                                    nh, nkv, d, page, window, scale)
            got = out.view(rows, nh, d)[rows - 1, 0].float().cpu()
            if window is None or far + window >= n - 1:
                assert float((got - v[far, 0]).abs().max()) < 0.03
            else:
                assert float((got - v[far, 0]).abs().max()) > 0.1
    ops().attention_tcgen05_check(d)


@pytest.mark.parametrize("M,hidden,inner,delta_kind", [
    (1, 64, 128, "none"), (3, 96, 256, "partials"), (8, 896, 4864, "partials"), (8, 896, 4864, "bf16"),
    (13, 160, 384, "partials"), (16, 896, 4864, "f32"), (5, 1536, 1280, "partials")])
def test_ffn_small_m(M, hidden, inner, delta_kind):
    """The whole feed-forward of few rows in one kernel (residual add, norm, gate/up with
    the activation, the barrier over all blocks, down as partial sums), twice in a row so
    that the barrier's counters are seen to come back to zero."""
    o = ops()
    splits = o.ffn_small_m_splits(M, hidden, inner)
    assert splits > 0
    x = rnd(M, hidden, seed=81)
    if delta_kind == "none":
        delta = None
    elif delta_kind == "partials":
        delta = rnd(3, M, hidden, seed=82, scale=0.3)
    elif delta_kind == "f32":
        delta = rnd(M, hidden, seed=82, scale=0.5)
    else:
        delta = rnd(M, hidden, seed=82, scale=0.5, dtype=torch.bfloat16)
    gain = 1.0 + rnd(hidden, seed=83, scale=0.1)
    gate = rnd(inner, hidden, seed=84, dtype=torch.bfloat16, scale=0.06)
    up = rnd(inner, hidden, seed=85, dtype=torch.bfloat16, scale=0.06)
    down = rnd(hidden, inner, seed=86, dtype=torch.bfloat16, scale=0.04)
    w_gu = o.interleave_gate_up(gate, up)
    eps = 1e-5
    # the reference, rounding where the kernel rounds: h and the activation to bfloat16
    xs = x.double().cpu()
    if delta is not None:
        xs = xs + (delta.double().cpu().sum(0) if delta.dim() == 3 else delta.double().cpu())
    h = xs / torch.sqrt((xs * xs).mean(-1, keepdim=True) + eps) * gain.double().cpu()
    h = h.float().to(torch.bfloat16).double()
    g = h @ gate.double().cpu().t()
    u = h @ up.double().cpu().t()
    act = (g * torch.sigmoid(g) * u).float().to(torch.bfloat16).double()
    want = (act @ down.double().cpu().t()).float()
    for _ in range(2):
        x_out = torch.full_like(x, 3.0)
        out = torch.full((splits, M, hidden), 5.0, dtype=torch.float32, device=DEV)
        o.ffn_small_m(x, x_out, delta, gain, eps, w_gu, down, out)
        torch.cuda.synchronize()
        o.ffn_small_m_check()
        assert torch.allclose(x_out.cpu(), xs.float(), atol=1e-5, rtol=1e-6)
        got = out.sum(0).cpu()
        # h and the activation may round the other way on a tie's edge: 2^-8 of their size
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 2e-3 * scale + 1e-5, float((got - want).abs().max())
    assert o.ffn_small_m_splits(17, hidden, inner) == 0 and o.ffn_small_m_splits(4, 100, 128) == 0


@pytest.mark.parametrize("M,N,K,S", [(64, 896, 4864, 19), (33, 100, 264, 2), (200, 256, 1024, 4),
                                     (17, 1152, 896, 7), (128, 132, 640, 5)])
def test_gemm_tcgen05_partials(M, N, K, S):
    """The tcgen05 product cut along k into S pieces (units of work = tile x piece, so that
    a narrow matrix still fills the device): the pieces add up to the product, rows past M
    of a tile stay out of the next piece's plane, and a piece count that would leave a
    piece empty is refused."""
    o = ops()
    a = rnd(M, K, seed=91, dtype=torch.bfloat16)
    w = rnd(N, K, seed=92, dtype=torch.bfloat16, scale=0.1)
    out = torch.full((S, M, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_tcgen05_partials(a, w, out)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()
    want = (a.double().cpu() @ w.double().cpu().t()).float()
    got = out.sum(0).cpu()
    assert torch.allclose(got, want, atol=2e-4 * float(want.abs().max()), rtol=1e-5), float((got - want).abs().max())
    # the pieces are different sums, none of them the fill value
    assert not bool((out == 9.0).any())
    with pytest.raises(ValueError):
        o.gemm_tcgen05_partials(a, w, torch.empty(K, M, N, dtype=torch.float32, device=DEV))


@pytest.mark.parametrize("M,N,K,S", [(2048, 896, 4864, 2), (300, 520, 200, 1), (100, 264, 1032, 3),
                                     (1100, 136, 640, 4), (513, 4, 128, 2)])
def test_gemm_tcgen05_pair_partials(M, N, K, S):
    """Two CTAs on a tile of 256 rows (each loads half of the weight tile, one thread issues the
    products for both): partial sums over S pieces of k, written in two passes of 128 columns.
    Row counts that leave the second CTA of the last pair with some or no rows; widths that end
    inside a tile and inside a pass."""
    o = ops()
    a = rnd(M, K, seed=93, dtype=torch.bfloat16)
    w = rnd(N, K, seed=94, dtype=torch.bfloat16, scale=0.1)
    out = torch.full((S, M, N), 9.0, dtype=torch.float32, device=DEV)
    o.gemm_tcgen05_pair(a, w, None, out, o.PAIR_PARTIALS)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()
    want = (a.double().cpu() @ w.double().cpu().t()).float()
    got = out.sum(0).cpu()
    assert torch.allclose(got, want, atol=2e-4 * float(want.abs().max()), rtol=1e-5), float((got - want).abs().max())
    assert not bool((out == 9.0).any())
    with pytest.raises(ValueError):
        o.gemm_tcgen05_pair(a, w, None, torch.empty(K, M, N, dtype=torch.float32, device=DEV), o.PAIR_PARTIALS)


@pytest.mark.parametrize("M,N,K", [(2048, 1152, 896), (257, 520, 72), (90, 256, 264), (640, 1032, 512)])
@pytest.mark.parametrize("narrow", [False, True])
def test_gemm_tcgen05_pair_plain(M, N, K, narrow):
    """The pair form with bfloat16 output and bias, on 256- and on 128-column tiles; the output
    past M and N stays untouched."""
    o = ops()
    a = rnd(M, K, seed=95, dtype=torch.bfloat16)
    w = rnd(N, K, seed=96, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=97)
    room = torch.full((M + 3, N), 5.0, dtype=torch.bfloat16, device=DEV)
    out = room[:M]
    o.gemm_tcgen05_pair(a, w, bias, out, o.PAIR_PLAIN_128 if narrow else o.PAIR_PLAIN)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()
    want = (a.double().cpu() @ w.double().cpu().t() + bias.double().cpu()).float()
    got = out.float().cpu()
    assert float((got - want).abs().max()) <= 2 ** -8 * float(want.abs().max()) + 1e-3
    assert bool((room[M:] == 5.0).all())


@pytest.mark.parametrize("M,inner,K", [(2048, 4864, 896), (256, 128, 64), (300, 384, 200), (1000, 1280, 512)])
def test_gemm_tcgen05_pair_gated(M, inner, K):
    """silu(gate) * up in the epilogue of the pair form, against the lone-CTA kernel's rule:
    the products in 32-bit, one rounding of the result."""
    o = ops()
    x = rnd(M, K, seed=98, dtype=torch.bfloat16)
    gate = rnd(inner, K, seed=99, dtype=torch.bfloat16, scale=0.1)
    up = rnd(inner, K, seed=100, dtype=torch.bfloat16, scale=0.1)
    w = o.interleave_gate_up(gate, up)
    out = torch.full((M, inner), 3.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tcgen05_pair(x, w, None, out, o.PAIR_GATED)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()
    g = x.double().cpu() @ gate.double().cpu().t()
    u = x.double().cpu() @ up.double().cpu().t()
    want = (g / (1 + torch.exp(-g)) * u).float()
    got = out.float().cpu()
    assert float((got - want).abs().max()) <= 2 ** -7 * float(want.abs().max()) + 1e-3, float((got - want).abs().max())


@pytest.mark.parametrize("nh,nkv,d,S,T", [(14, 2, 64, 7, 40), (3, 1, 32, 2, 70), (4, 4, 128, 5, 17)])
def test_rope_store_from_partial_sums(nh, nkv, d, S, T):
    """Bias, rotation and the cache write straight from float32 partial sums [S, T, width]."""
    o = ops()
    width = (nh + 2 * nkv) * d
    inv_freq = torch.tensor([1.0 / 1e4 ** (i / d) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 600)
    parts = rnd(S, T, width, seed=96)
    bias = rnd(width, seed=97, scale=0.3)
    pos = torch.arange(500, 500 + T, dtype=torch.int32, device=DEV)
    slot = torch.randperm(T + 5, generator=torch.Generator().manual_seed(2))[:T].to(torch.int32).to(DEV)
    slot[3] = -1
    k_pool = torch.full((T + 5, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((T + 5, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(T, nh * d, dtype=torch.bfloat16, device=DEV)
    o.rope_store(parts, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, d)
    full = (parts.sum(0) + bias).view(T, nh + 2 * nkv, d).cpu()
    c, s = cos[pos.long()].cpu()[:, None, :], sin[pos.long()].cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :d // 2], v[..., d // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    close(q_out.view(T, nh, d), rotate(full[:, :nh]), torch.bfloat16)
    live = [t for t in range(T) if int(slot[t]) >= 0]
    close(k_pool[slot[live].long()], rotate(full[:, nh:nh + nkv])[live], torch.bfloat16)
    close(v_pool[slot[live].long()], full[:, nh + nkv:][live], torch.bfloat16)
    untouched = [i for i in range(T + 5) if i not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all())
    with pytest.raises(ValueError):
        o.rope_store(parts, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d, d - 2)


@pytest.mark.parametrize("M,N,K,out_dtype,with_bias", [
    (1, 16, 32, torch.float32, False), (8, 151936, 896, torch.float32, False), (5, 3001, 96, torch.bfloat16, True),
    (16, 20000, 1536, torch.float32, True), (13, 777, 2080, torch.bfloat16, False)])
def test_linear_stream(M, N, K, out_dtype, with_bias):
    """The ring-streaming product for few rows and many weight rows: tiles that end inside
    the matrix (N not a multiple of 16), K longer than a stage (2080 > 1024), both output
    types, blocks with no tile at all (16 rows on a whole device)."""
    o = ops()
    assert o.linear_stream_supported(M, N, K)
    x = rnd(M, K, seed=111, dtype=torch.bfloat16)
    w = rnd(N, K, seed=112, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=113) if with_bias else None
    out = torch.full((M, N), 7.0, dtype=out_dtype, device=DEV)
    for _ in range(2):
        o.linear_stream(x, w, bias, out)
    torch.cuda.synchronize()
    o.linear_stream_check()
    want = x.double().cpu() @ w.double().cpu().t()
    if with_bias:
        want = want + bias.double().cpu()
    close(out, want.float(), out_dtype if out_dtype == torch.bfloat16 else torch.float32)
    assert not o.linear_stream_supported(17, N, K) and not o.linear_stream_supported(4, N, 100)


@pytest.mark.parametrize("M,nh,nkv,d,K,delta_kind", [
    (1, 4, 2, 16, 64, "none"), (8, 14, 2, 64, 896, "partials5"), (5, 3, 1, 32, 96, "bf16"),
    (7, 5, 5, 48, 160, "partials5"), (3, 2, 1, 128, 1024, "f32")])
def test_qkv_projection_with_the_norm_in_front_folded_in(M, nh, nkv, d, K, delta_kind):
    """The q/k/v kernel that also adds the pending residual and computes the RMS norm: the
    new residual sum, and the rotated projections of the normed rows (rounded to bfloat16
    where the kernel rounds them) in their cache slots."""
    o = ops()
    heads = nh + 2 * nkv
    x = rnd(M, K, seed=121)
    delta = {"none": None, "partials5": rnd(5, M, K, seed=122, scale=0.3),
             "f32": rnd(M, K, seed=122, scale=0.5),
             "bf16": rnd(M, K, seed=122, scale=0.5, dtype=torch.bfloat16)}[delta_kind]
    gain = 1.0 + rnd(K, seed=123, scale=0.1)
    eps = 1e-5
    w = rnd(heads * d, K, seed=124, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(heads * d, seed=125, scale=0.3)
    inv_freq = torch.tensor([1.0 / 1e4 ** (i / d) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 900)
    pos = torch.tensor([(37 * i + 5) % 900 for i in range(M)], dtype=torch.int32, device=DEV)
    slot = torch.tensor([2 * i + 1 for i in range(M)], dtype=torch.int32, device=DEV)
    if M > 1:
        slot[M - 1] = -1
    k_pool = torch.full((2 * M + 2, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((2 * M + 2, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(M, nh * d, dtype=torch.bfloat16, device=DEV)
    x_out = torch.full_like(x, 3.0)
    o.qkv_norm_rope_small_m(x, x_out, delta, gain, eps, w, bias, pos, slot, cos, sin, q_out, k_pool, v_pool,
                            nh, nkv, d)
    xs = x.double().cpu()
    if delta is not None:
        xs = xs + (delta.double().cpu().sum(0) if delta.dim() == 3 else delta.double().cpu())
    assert torch.allclose(x_out.cpu(), xs.float(), atol=1e-5, rtol=1e-6)
    h = (xs / torch.sqrt((xs * xs).mean(-1, keepdim=True) + eps) * gain.double().cpu()).float().to(torch.bfloat16)
    full = (h.double() @ w.double().cpu().t() + bias.double().cpu()).float().view(M, heads, d)
    c, s = cos[pos.long()].cpu()[:, None, :], sin[pos.long()].cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :d // 2], v[..., d // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    def near(got, want):   # h may round the other way on a tie's edge: 2^-8 of the sum's terms
        got, want = got.float().cpu(), want.float().cpu()
        assert torch.allclose(got, want, atol=3e-3 * float(want.abs().max()) + 1e-3, rtol=2 ** -7), \
            float((got - want).abs().max())

    near(q_out.view(M, nh, d), rotate(full[:, :nh]))
    k_want, v_want = rotate(full[:, nh:nh + nkv]), full[:, nh + nkv:]
    for m in range(M):
        if int(slot[m]) >= 0:
            near(k_pool[int(slot[m])], k_want[m])
            near(v_pool[int(slot[m])], v_want[m])
    untouched = [i for i in range(2 * M + 2) if i not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all()) and bool((v_pool[untouched] == 7.0).all())
    assert not o.qkv_norm_rope_small_m_supported(9, K, d, d) and not o.qkv_norm_rope_small_m_supported(4, 2048, d, d)


@pytest.mark.parametrize("M,nh,nkv,d,K", [(130, 4, 2, 64, 128), (2048, 14, 2, 64, 896), (300, 2, 1, 128, 200),
                                           (129, 6, 4, 64, 72)])
def test_gemm_qkv_rope(M, nh, nkv, d, K):
    """The tcgen05 q/k/v product of many rows with bias, rotation and cache write in its
    epilogue, against the unfused arithmetic; some rows write no cache."""
    o = ops()
    heads = nh + 2 * nkv
    assert o.gemm_qkv_rope_supported(K, nh, nkv, d, d)
    x = rnd(M, K, seed=131, dtype=torch.bfloat16)
    w = rnd(heads * d, K, seed=132, dtype=torch.bfloat16, scale=0.2)
    bias = rnd(heads * d, seed=133, scale=0.3)
    inv_freq = torch.tensor([1.0 / 1e4 ** (i / d) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, 3000)
    pos = torch.tensor([(37 * i + 5) % 3000 for i in range(M)], dtype=torch.int32, device=DEV)
    slot = torch.randperm(M + 9, generator=torch.Generator().manual_seed(3))[:M].to(torch.int32).to(DEV)
    slot[5] = -1
    slot[M - 1] = -1
    k_pool = torch.full((M + 9, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full((M + 9, nkv, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((M, nh * d), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_qkv_rope(x, w, bias, pos, slot, cos, sin, q_out, k_pool, v_pool, nh, nkv, d)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()
    full = (x.double().cpu() @ w.double().cpu().t() + bias.double().cpu()).float().view(M, heads, d)
    c, s = cos[pos.long()].cpu()[:, None, :], sin[pos.long()].cpu()[:, None, :]

    def rotate(v):
        a, b = v[..., :d // 2], v[..., d // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    close(q_out.view(M, nh, d), rotate(full[:, :nh]), torch.bfloat16)
    live = [t for t in range(M) if int(slot[t]) >= 0]
    close(k_pool[slot[live].long()], rotate(full[:, nh:nh + nkv])[live], torch.bfloat16)
    close(v_pool[slot[live].long()], full[:, nh + nkv:][live], torch.bfloat16)
    untouched = [i for i in range(M + 9) if i not in slot.tolist()]
    assert bool((k_pool[untouched] == 7.0).all()) and bool((v_pool[untouched] == 7.0).all())
    assert not o.gemm_qkv_rope_supported(K, 3, 1, 64, 64) and not o.gemm_qkv_rope_supported(K, nh, nkv, 48, 48)


def test_a_wait_that_runs_out_returns_and_is_reported(monkeypatch, tmp_path):
    """The barrier between the two products of the fused feed-forward waits for a count in
    global memory.  Built with short limits and given a count that can never be met, every
    block's wait runs out: the kernel must come back by itself, the host must learn of it
    through the error word (`raise_if_error`, and through the engine: the draw that follows a
    failed step raises), the barrier's counters must be left ready, and the next launch must
    be right.  No copy is in flight when the wait gives up and nothing is read out of bounds:
    the blocks only skip their second product."""
    o = ops()
    monkeypatch.setattr(o, "_FFN_DEFINES", ("FFN_GRID_WAIT_LIMIT=2048u", "FFN_WAIT_LIMIT=2048u"))
    M, hidden, inner = 4, 128, 256
    splits = o.ffn_small_m_splits(M, hidden, inner)
    x = rnd(M, hidden, seed=1)
    gain = 1.0 + rnd(hidden, seed=2, scale=0.1)
    gate = rnd(inner, hidden, seed=3, dtype=torch.bfloat16, scale=0.06)
    up = rnd(inner, hidden, seed=4, dtype=torch.bfloat16, scale=0.06)
    down = rnd(hidden, inner, seed=5, dtype=torch.bfloat16, scale=0.04)
    w_gu = o.interleave_gate_up(gate, up)
    space = o.ScratchSpace()

    def run():
        x_out = torch.empty_like(x)
        out = torch.zeros((splits, M, hidden), dtype=torch.float32, device=DEV)
        with o.scratch_scope(space):
            o.ffn_small_m(x, x_out, None, gain, 1e-6, w_gu, down, out)
        torch.cuda.synchronize()
        return out.sum(0).cpu()

    o.raise_if_error()
    good = run()
    o.raise_if_error()                       # the short limits are long enough for a sound run
    (act, sync), = space.ffn.values()
    sync[0] = -1_000_000                     # the count of arrived blocks can never reach the grid's size
    bad = run()
    assert o.error_code() != 0
    with pytest.raises(o.KernelError, match="ffn_small_m"):
        o.raise_if_error("in the test")
    assert o.error_code() == 0 and sync.tolist() == [0, 0]
    o.ffn_small_m_check()                    # the library's own flag was cleared with the word
    assert not torch.equal(bad, good)        # the failed launch did not produce the result...
    assert torch.equal(run(), good)          # ...and the one after it does
    o.raise_if_error()

    # the same through an engine: the step runs to its end, reading its ids raises
    import tokenizer_b200 as tb
    from tokenizer_b200.engine import StepEntry
    config = tb.Qwen2Config.from_dict(dict(
        architectures=["Qwen2ForCausalLM"], hidden_act="silu", num_hidden_layers=2, hidden_size=128,
        num_attention_heads=2, num_key_value_heads=1, intermediate_size=256, vocab_size=320,
        rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256,
        use_sliding_window=False, sliding_window=64, max_window_layers=2))
    tb.write_random_model(str(tmp_path), config, seed=5)
    engine = tb.engine_for(tb.load_model(str(tmp_path), dtype="bfloat16"), 128, 16, max_requests=2)
    cache = engine.cache.open("x")
    engine.cache.reserve(cache, 3)
    first = engine.step([StepEntry(cache, [5], [0])]).clone()
    assert engine.sample(first, [0.0], [1.0], [0.0])
    (act, sync), = engine.model.scratch.ffn.values()
    sync[0] = -1_000_000
    logits = engine.step([StepEntry(cache, [6], [0])])
    with pytest.raises(o.KernelError, match="ffn_small_m"):
        engine.sample(logits, [0.0], [1.0], [0.0])
    engine.check()                           # reported once; the engine goes on
    after = engine.step([StepEntry(cache, [7], [0])])
    assert engine.sample(after, [0.0], [1.0], [0.0]) and bool(torch.isfinite(after).all())


def layer_reference(x, delta, gain1, eps1, w_qkv, b_qkv, pos, dense, row_req, w_o, gain2, eps2, gate, up, down,
                    nh, nkv, d, window, theta=10000.0):
    """A pre-norm decoder layer for rows of one token each, in float64 with roundings to bfloat16
    where the kernels round (normed rows, q/k/v, attention output, activation).  `dense[r]` holds
    request r's keys and values up to the row's position (the entry AT the position is replaced by
    the new key and value).  Returns x_mid, x_out, the feed-forward's output, new keys, new values."""
    def bf(t):
        return t.float().to(torch.bfloat16).double()
    x1 = x.double() + (delta.double().sum(0) if delta is not None and delta.dim() == 3 else
                       (delta.double() if delta is not None else 0.0))
    h = bf(x1 / torch.sqrt((x1 * x1).mean(-1, keepdim=True) + eps1) * gain1.double())
    qkv = h @ w_qkv.double().t() + (b_qkv.double() if b_qkv is not None else 0.0)
    M = x.shape[0]
    half = d // 2
    inv_freq = torch.tensor([1.0 / (theta ** (i / d)) for i in range(0, d, 2)], dtype=torch.float64).float()
    x2 = torch.zeros_like(x1)
    k_new, v_new, mixed = [], [], torch.zeros(M, nh * d, dtype=torch.float64)
    for m in range(M):
        ang = torch.tensor(float(pos[m]), dtype=torch.float32) * inv_freq
        cos, sin = torch.cos(ang).double(), torch.sin(ang).double()

        def rot(v):
            a, b = v[..., :half], v[..., half:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
        q = bf(rot(qkv[m, :nh * d].view(nh, d)))
        k = bf(rot(qkv[m, nh * d:(nh + nkv) * d].view(nkv, d)))
        v = bf(qkv[m, (nh + nkv) * d:].view(nkv, d))
        k_new.append(k)
        v_new.append(v)
        if row_req[m] < 0:
            continue
        keys, values = dense[row_req[m]][0].double().clone(), dense[row_req[m]][1].double().clone()
        keys[pos[m]], values[pos[m]] = k, v
        lo = 0 if window is None else max(0, pos[m] - window)
        for hh in range(nh):
            gk = hh // (nh // nkv)
            s = (keys[lo:pos[m] + 1, gk] @ q[hh]) / math.sqrt(d)
            mixed[m, hh * d:(hh + 1) * d] = torch.softmax(s, 0) @ values[lo:pos[m] + 1, gk]
    x2 = x1 + bf(mixed) @ w_o.double().t()
    h2 = bf(x2 / torch.sqrt((x2 * x2).mean(-1, keepdim=True) + eps2) * gain2.double())
    g, u = h2 @ gate.double().t(), h2 @ up.double().t()
    act = bf(g * torch.sigmoid(g) * u)
    return x1.float(), x2.float(), (act @ down.double().t()).float(), k_new, v_new


@pytest.mark.parametrize("M,hidden,inner,nh,nkv,d,page,window,lengths", [
    (1, 128, 256, 2, 1, 64, 16, None, [300]),
    (3, 160, 384, 4, 2, 64, 8, None, [1, 77, 600]),
    (8, 896, 4864, 14, 2, 64, 16, None, [527, 3, 64, 65, 1000, 257, 256, 31]),
    (5, 256, 512, 2, 2, 128, 16, 100, [40, 101, 102, 500, 2]),
    (13, 384, 640, 6, 3, 64, 32, None, [5 + 97 * i for i in range(13)]),
    (16, 1536, 1280, 12, 2, 128, 16, None, [9 + 61 * i for i in range(16)]),
    (7, 192, 256, 16, 1, 64, 16, None, [2500, 1, 300, 17, 900, 64, 2049]),
    (24, 896, 4864, 14, 2, 64, 16, None, [3 + 53 * i for i in range(24)]),
    (32, 256, 640, 4, 2, 128, 16, None, [700 - 21 * i for i in range(32)])])
def test_layer_small_m(M, hidden, inner, nh, nkv, d, page, window, lengths):
    """A whole decoder layer of few rows in one kernel (norm, q/k/v with bias and rotation, cache
    write, attention over the paged keys with pieces merged across blocks, output projection,
    second norm, gated feed-forward), twice in a row so that every counter is seen to come back
    to zero, with an idle row in the padded batch."""
    o = ops()
    down_splits, o_splits = o.layer_small_m_splits(M, hidden, inner, nh, nkv, d)
    assert down_splits > 0 and o_splits > 0
    dtype = torch.bfloat16
    k_pool, v_pool, tables, dense = paged_setup(lengths, nh, nkv, d, page, dtype, seed=41)
    row_req = list(range(M))
    pos = [n - 1 for n in lengths]
    if M >= 5:
        row_req[2] = -1                           # an idle row of a padded batch
    slot = [int(tables[r, p // page]) * page + p % page if r >= 0 else -1 for r, p in zip(row_req, pos)]
    x = rnd(M, hidden, seed=42)
    delta = rnd(3, M, hidden, seed=43, scale=0.3)
    gain1, gain2 = 1.0 + rnd(hidden, seed=44, scale=0.1), 1.0 + rnd(hidden, seed=45, scale=0.1)
    w_qkv = rnd((nh + 2 * nkv) * d, hidden, seed=46, dtype=dtype, scale=0.08)
    b_qkv = rnd((nh + 2 * nkv) * d, seed=47, scale=0.2)
    w_o = rnd(hidden, nh * d, seed=48, dtype=dtype, scale=0.05)
    gate = rnd(inner, hidden, seed=49, dtype=dtype, scale=0.06)
    up = rnd(inner, hidden, seed=50, dtype=dtype, scale=0.06)
    down = rnd(hidden, inner, seed=51, dtype=dtype, scale=0.04)
    inv_freq = torch.tensor([1.0 / (10000.0 ** (i / d)) for i in range(0, d, 2)], dtype=torch.float64).float().to(DEV)
    cos, sin = o.rope_table(inv_freq, max(lengths) + 1)
    want_mid, want_out, want_ff, k_new, v_new = layer_reference(
        x.cpu(), delta.cpu(), gain1.cpu(), 1e-5, w_qkv.cpu(), b_qkv.cpu(), pos, dense, row_req, w_o.cpu(),
        gain2.cpu(), 2e-6, gate.cpu(), up.cpu(), down.cpu(), nh, nkv, d, window)
    dev = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    live = [m for m in range(M) if row_req[m] >= 0]
    for _ in range(2):
        x_mid, x_out = torch.full_like(x, 3.0), torch.full_like(x, 4.0)
        out = torch.full((down_splits, M, hidden), 5.0, dtype=torch.float32, device=DEV)
        o.layer_small_m(x, delta, x_mid, x_out, out, gain1, 1e-5, w_qkv, b_qkv, dev(pos), dev(slot), dev(row_req),
                        tables, cos, sin, k_pool, v_pool, True, w_o, gain2, 2e-6, o.interleave_gate_up(gate, up),
                        down, nh, nkv, d, page, window, 1.0 / math.sqrt(d))
        torch.cuda.synchronize()
        o.layer_small_m_check(d)
        o.raise_if_error()
        assert torch.allclose(x_mid.cpu(), want_mid, atol=1e-5, rtol=1e-6)
        for m in live:                             # the new key and value in the row's slot
            close(k_pool[slot[m]], k_new[m].float(), dtype)
            close(v_pool[slot[m]], v_new[m].float(), dtype)
        scale = float((want_out - want_mid).abs().max())
        err = float((x_out.cpu() - want_out)[live].abs().max())
        assert err <= 1.5e-2 * scale + 1e-4, f"attention half off by {err} of {scale}"
        got = out.sum(0).cpu()
        scale = float(want_ff.abs().max())
        err = float((got - want_ff)[live].abs().max())
        assert err <= 2e-2 * scale + 1e-4, f"feed-forward off by {err} of {scale}"
    assert o.layer_small_m_splits(33, hidden, inner, nh, nkv, d) == (0, 0)
    assert o.layer_small_m_splits(4, 100, inner, nh, nkv, d) == (0, 0)
