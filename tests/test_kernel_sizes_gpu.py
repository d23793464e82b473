"""Sizes drawn at random (a fixed seed) through the few-row product, its gated form and the
decode attention, against float64: k that ends inside a step of 64, odd output counts, head
sizes from 16 to 256, groups of 1 to 16 heads, pages of 8 to 48 slots in shuffled tables,
windows, rows of unequal lengths from a few keys to thousands."""
import math
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from tokenizer_b200.kernels import ops as o
    return o


def rnd(*shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def test_few_row_products_at_random_sizes():
    o = ops()
    rng = random.Random(11)
    for case in range(24):
        M = rng.choice([1, 2, 7, 8, 9, 12, 16, 17, 31, 32, 33, 48, 64])
        K = 8 * rng.randint(1, 260)
        N = rng.choice([1, 5, 16, 33, 250, 896, 1000, 3001, 17000])
        x = rnd(M, K, seed=case, dtype=torch.bfloat16)
        w = rnd(N, K, seed=1000 + case, scale=0.1, dtype=torch.bfloat16)
        want = x.double().cpu() @ w.double().cpu().t()
        tol = 2e-5 * float(want.abs().max()) + 1e-6 * K
        out = torch.empty(M, N, device=DEV)
        o.linear_small_m(x, w, None, out)
        assert float((out.double().cpu() - want).abs().max()) <= tol, (M, N, K)
        splits = rng.choice([2, 3, 5])
        if K // splits >= 8:
            parts = torch.full((splits, M, N), 3.0, device=DEV)
            o.linear_small_m(x, w, None, parts, k_splits=splits)
            assert float((parts.sum(0).double().cpu() - want).abs().max()) <= tol, (M, N, K, splits)
        if case % 3 == 0:
            inner = 128 * rng.randint(1, 6)
            gate = rnd(inner, K, seed=2000 + case, scale=0.2, dtype=torch.bfloat16)
            up = rnd(inner, K, seed=3000 + case, scale=0.2, dtype=torch.bfloat16)
            got = torch.empty(M, inner, dtype=torch.bfloat16, device=DEV)
            o.gated_linear(x, o.interleave_gate_up(gate, up), got)
            g = x.double().cpu() @ gate.double().cpu().t()
            u = x.double().cpu() @ up.double().cpu().t()
            want_act = (g * torch.sigmoid(g) * u).float()
            assert torch.allclose(got.float().cpu(), want_act, atol=4e-3 * max(1.0, float(want_act.abs().max())),
                                  rtol=2 ** -6), (M, inner, K)
    torch.cuda.synchronize()
    o.gemm_tcgen05_check()


def test_ring_products_at_random_sizes():
    """The product that streams a large weight through rings in shared memory (up to 32 rows), its
    pieces of k and its gated form, wherever it takes the sizes drawn."""
    o = ops()
    rng = random.Random(13)
    taken = 0
    for case in range(16):
        M = rng.randint(1, 32)
        K = 8 * rng.randint(64, 1200)
        N = rng.choice([16, 50, 896, 1000, 3001, 9000])
        x = rnd(M, K, seed=9000 + case, dtype=torch.bfloat16)
        w = rnd(N, K, seed=9500 + case, scale=0.1, dtype=torch.bfloat16)
        want = x.double().cpu() @ w.double().cpu().t()
        tol = 2e-5 * float(want.abs().max()) + 1e-6 * K
        for splits in (1, 2, 3, 5):
            if not o.linear_ring_supported(M, N, K, splits):
                continue
            taken += 1
            out = torch.full((splits, M, N), 3.0, device=DEV) if splits > 1 else torch.full((M, N), 3.0, device=DEV)
            o.linear_ring(x, w, None, out, splits)
            got = out.sum(0) if splits > 1 else out
            assert float((got.double().cpu() - want).abs().max()) <= tol, (M, N, K, splits)
        inner = 128 * rng.randint(1, 8)
        if o.linear_ring_supported(M, 2 * inner, K, 1, True):
            taken += 1
            gate = rnd(inner, K, seed=9700 + case, scale=0.1, dtype=torch.bfloat16)
            up = rnd(inner, K, seed=9800 + case, scale=0.1, dtype=torch.bfloat16)
            got = torch.empty(M, inner, dtype=torch.bfloat16, device=DEV)
            o.linear_ring_gated(x, o.interleave_gate_up(gate, up), got)
            g = x.double().cpu() @ gate.double().cpu().t()
            u = x.double().cpu() @ up.double().cpu().t()
            want_act = (g * torch.sigmoid(g) * u).float()
            assert torch.allclose(got.float().cpu(), want_act, atol=4e-3 * max(1.0, float(want_act.abs().max())),
                                  rtol=2 ** -6), (M, inner, K)
    assert taken >= 20


def test_decode_attention_at_random_sizes():
    o = ops()
    rng = random.Random(12)
    for case in range(20):
        d = rng.choice([16, 32, 48, 64, 80, 96, 128, 160, 256])     # most of them built ahead; the others compile here
        nkv = rng.choice([1, 2, 3, 4])
        group = rng.choice([1, 2, 4, 6, 7, 8, 12, 16])
        nh = nkv * group
        page = rng.choice([8, 16, 32, 48])
        rows = rng.choice([1, 3, 8, 20, 64])
        longest = rng.choice([5, 40, 300, 1100, 2600, 6000])
        window = rng.choice([None, None, 7, 200, 1500])
        lengths = [rng.randint(max(1, longest // 3), longest) for _ in range(rows)]
        per = (longest + page - 1) // page + 1
        n_pages = rows * per + 3
        order = list(range(n_pages))
        rng.shuffle(order)
        tables = torch.tensor([[order[r * per + i] for i in range(per)] for r in range(rows)],
                              dtype=torch.int32, device=DEV)
        k = rnd(n_pages * page, nkv, d, seed=5000 + case, dtype=torch.bfloat16)
        v = rnd(n_pages * page, nkv, d, seed=6000 + case, dtype=torch.bfloat16)
        q = rnd(rows, nh * d, seed=7000 + case, dtype=torch.bfloat16)
        pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
        row_req = torch.arange(rows, dtype=torch.int32, device=DEV)
        out = torch.zeros_like(q)
        scale = 1 / math.sqrt(d)
        o.decode_attention(q, k, v, out, tables, row_req, pos, nh, nkv, d, page, window, scale)
        torch.cuda.synchronize()
        kc, vc, qc = k.double().cpu(), v.double().cpu(), q.double().cpu().view(rows, nh, d)
        got = out.view(rows, nh, d).double().cpu()
        for r in rng.sample(range(rows), min(rows, 3)):
            n = lengths[r]
            slots = [int(tables[r, i // page]) * page + i % page for i in range(n)]
            lo = 0 if window is None else max(0, n - 1 - window)
            for h in range(nh):
                keys, values = kc[slots[lo:], h // group], vc[slots[lo:], h // group]
                p = torch.softmax((keys @ qc[r, h]) * scale, 0)
                err = float((got[r, h] - p @ values).abs().max())
                assert err < 0.03, (dict(d=d, nkv=nkv, group=group, page=page, rows=rows, longest=longest,
                                         window=window), r, h, err)
