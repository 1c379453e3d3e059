"""InfLLM-v2 block selection and block-sparse attention (MiniCPM4 target, config 5), kernel level,
through the C ABI, against oracle/sparse.py.

Integer stages (max-pool, top-k, bitmask, visited blocks) are compared bit for bit given the same
bf16 scores; floating-point stages against fp32 PyTorch with the tolerance written in the test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import sparse as osparse

pytestmark = pytest.mark.gpu


def C():
    import cpmcu.C as c
    c.load()
    return c


def dev(t):
    return t.to("cuda").contiguous()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def bf16(t):
    return t.to(torch.bfloat16)


def make_case(T, hq, hkv, L, seed, budget=None):
    g = torch.Generator().manual_seed(seed)
    budget = budget or (L + T + 127) // 128 * 128
    kv_dim = hkv * 128
    q_ld = (hq + 2 * hkv) * 128
    q = bf16(torch.randn(T, q_ld, generator=g))
    # keys with some structure so that block scores differ clearly: a slow random walk plus noise
    base = torch.cumsum(torch.randn(budget // 64 + 1, kv_dim, generator=g), dim=0) * 0.5
    k = bf16(base.repeat_interleave(64, dim=0)[:budget] + torch.randn(budget, kv_dim, generator=g))
    v = bf16(torch.randn(budget, kv_dim, generator=g))
    return q, k, v, budget


SELECT_CASES = [
    # T, hq, hkv, L, top, sink, window, lse, budget (None: just above L; the library picks its top-k kernel by budget)
    (12, 8, 2, 1500, 6, 1, 4, True, None),
    (60, 32, 2, 3000, 16, 1, 8, True, None),
    (7, 8, 2, 2048, 8, 2, 2, False, None),
    (16, 4, 1, 1000, 64, 1, 3, True, None),   # fewer candidate blocks than top-k
    (9, 8, 2, 3000, 12, 1, 4, True, 40960),   # up to 1024 blocks: 32 keys per lane
    (9, 8, 2, 3000, 12, 1, 4, True, 69632),   # more than 1024 blocks: block-wide selection
]


@pytest.mark.parametrize("T,hq,hkv,L,top,sink,window,lse,budget", SELECT_CASES)
def test_block_selection_matches_oracle(T, hq, hkv, L, top, sink, window, lse, budget):
    c = C()
    q, k, v, budget = make_case(T, hq, hkv, L, seed=L + T, budget=budget)
    kv_dim = hkv * 128
    score_ld = (budget // 16 + 127) // 128 * 128
    bm_words = ((L + T + 127) // 128 * 128 // 64 + 63) // 64
    c1 = torch.zeros(budget // 16, kv_dim, dtype=torch.bfloat16, device="cuda")
    c2 = torch.zeros(budget // 64, kv_dim, dtype=torch.bfloat16, device="cuda")
    scores = torch.zeros(hkv, T, score_ld, dtype=torch.bfloat16, device="cuda")
    bm = torch.zeros(hkv, T, bm_words, dtype=torch.int64, device="cuda")
    kv_len = dev(torch.tensor([L], dtype=torch.int32))
    qd, kd = dev(q), dev(k)
    c.call("cpmcu_sparse_select", ptr(qd), q.shape[1], T, hq, hkv, ptr(kd), budget, ptr(kv_len), 0, sink, window, top,
           256, int(lse), ptr(c1), ptr(c2), ptr(scores), score_ld, ptr(bm), bm_words)
    # compressed caches: fp32 mean of bf16 rows, stored as bf16 (one rounding; summation order may differ)
    o_c1 = osparse.compress(k.float(), L, 16)
    o_c2 = osparse.compress(k.float(), L, 64)
    n1, n2 = o_c1.shape[0], o_c2.shape[0]
    assert n1 == max((L - 16) // 16, 0)
    assert float((c1[:n1].float().cpu() - o_c1).abs().max()) <= 2 ** -7 * float(o_c1.abs().max())
    if lse:
        assert float((c2[:n2].float().cpu() - o_c2).abs().max()) <= 2 ** -7 * float(o_c2.abs().max())
    # stage-1 scores from the library's own compressed keys: bf16 store (2^-8) + exp of fp32 dots
    o_scores = osparse.stage1_scores(q[:, : hq * 128].float(), c1[:n1].float().cpu(),
                                     (c2[:n2] if lse else c1[:n1]).float().cpu(), hq, hkv, 128)
    got = scores[:, :, : o_scores.shape[2]].float().cpu()
    err = (got - o_scores).abs()
    assert bool((err <= 2e-2 * o_scores.abs() + 1e-6).all()), float(err.max())
    assert float(scores[:, :, o_scores.shape[2]:].float().abs().max()) == 0.0 if score_ld > o_scores.shape[2] else True
    # max-pool + top-k + bitmask from the SAME scores: bit-exact
    pool = osparse.maxpool_blocks(got, T, L, sink, window)
    o_bm = osparse.topk_blockmask(pool, top, (L + T + 127) // 128 * 128)
    np.testing.assert_array_equal(bm.cpu().numpy().view(np.uint64), o_bm)
    # sink blocks are always selected
    assert all(int(o_bm[g, t, 0]) & ((1 << sink) - 1) == (1 << sink) - 1 for g in range(hkv) for t in range(T))


def test_selection_inactive_below_switch():
    c = C()
    T, hq, hkv, L = 5, 8, 2, 700
    q, k, v, budget = make_case(T, hq, hkv, L, seed=3)
    score_ld = (budget // 16 + 127) // 128 * 128
    bm = torch.zeros(hkv, T, 1, dtype=torch.int64, device="cuda")
    kv_len = dev(torch.tensor([L], dtype=torch.int32))
    qd, kd = dev(q), dev(k)
    c.call("cpmcu_sparse_select", ptr(qd), q.shape[1], T, hq, hkv, ptr(kd), budget, ptr(kv_len), 0, 1, 4, 8, 8192, 1,
           None, None, None, score_ld, ptr(bm), 1)
    assert bool((bm == -1).all())   # all ones: every block is visited
    assert not osparse.sparse_active(osparse.SparseConfig(sparse_switch=8192), L)


def reference_attention(q, k, v, hq, hkv, kv_total, tq, tree_mask, mask_k, vis_blocks):
    d = 128
    grp = hq // hkv
    qh = q[:, : hq * d].float().view(tq, hq, d)
    K = k[:kv_total].float().view(kv_total, hkv, d)
    V = v[:kv_total].float().view(kv_total, hkv, d)
    cols = torch.arange(kv_total)
    vis = cols[None, :] < (kv_total - tq + torch.arange(tq)[:, None] + 1)
    if tree_mask is not None:
        mbeg = kv_total - mask_k
        bits = torch.zeros(tq, kv_total, dtype=torch.bool)
        for t in range(tq):
            for cc in range(mask_k):
                bits[t, mbeg + cc] = (int(tree_mask[t]) >> cc) & 1
        vis = vis & ((cols[None, :] < mbeg) | bits)
    out = torch.zeros(tq, hq, d)
    for h in range(hq):
        s = (qh[:, h] @ K[:, h // grp].t()) / math.sqrt(d)
        s = s.masked_fill(~(vis & vis_blocks[h // grp]), float("-inf"))
        out[:, h] = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0) @ V[:, h // grp]
    return out.reshape(tq, hq * d)


ATTN_CASES = [
    # T, hq, hkv, L, window blocks, bit density, splits, tree mask
    (12, 8, 2, 1500, 4, 0.15, 1, False),
    (12, 8, 2, 1500, 4, 0.15, 3, True),
    (60, 32, 2, 3000, 8, 0.10, 4, True),
    (60, 32, 2, 3000, 2, 0.0, 2, True),     # nothing selected: sink-less, window only
    (1, 32, 2, 4100, 3, 0.05, 2, False),
    (40, 4, 1, 900, 1, 0.3, 1, True),       # grp = 4: 32 tokens per tile, two tiles
]


@pytest.mark.parametrize("T,hq,hkv,L,window,density,splits,tree", ATTN_CASES)
def test_block_sparse_attention_matches_fp32(T, hq, hkv, L, window, density, splits, tree):
    c = C()
    q, k, v, budget = make_case(T, hq, hkv, L, seed=7 * L + T)
    kv_total = L + T
    rng = np.random.default_rng(L + T)
    nblk = (kv_total + 63) // 64
    bm_words = (nblk + 63) // 64
    bits = rng.random((hkv, T, bm_words * 64)) < density
    bits[:, :, nblk:] = False
    mask = np.zeros((hkv, T, bm_words), dtype=np.uint64)
    for w in range(bm_words):
        for b in range(64):
            mask[:, :, w] |= bits[:, :, w * 64 + b].astype(np.uint64) << np.uint64(b)
    tree_mask = None
    if tree:
        # node t sees itself and node 0 (a star-shaped tree): bit t and bit 0
        tree_mask = np.array([(1 << t) | 1 for t in range(T)], dtype=np.uint64)
    vis_blocks = osparse.block_visibility(mask, window, T, kv_total)
    ref = reference_attention(q, k, v, hq, hkv, kv_total, T, tree_mask, T, vis_blocks)
    out = torch.full((T, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    qd, kd, vd = dev(q), dev(k), dev(v)
    bm_d = dev(torch.from_numpy(mask.view(np.int64)))
    tm_d = dev(torch.from_numpy(tree_mask.view(np.int64))) if tree else None
    c.call("cpmcu_sparse_attention", ptr(qd), q.shape[1], ptr(kd), ptr(vd), budget, T, hq, hkv, ptr(kv_len), 0, ptr(tm_d), T,
           ptr(bm_d), bm_words, window, splits, ptr(out), hq * 128)
    err = (out.float().cpu() - ref).abs()
    assert torch.isfinite(out.float()).all()
    assert float(err.max()) <= 3e-2, float(err.max())   # bf16 P and bf16 output, |out| <= ~4


def test_all_ones_mask_equals_dense_attention():
    c = C()
    T, hq, hkv, L = 24, 8, 2, 1100
    q, k, v, budget = make_case(T, hq, hkv, L, seed=11)
    kv_total = L + T
    bm_words = ((kv_total + 63) // 64 + 63) // 64
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    qd, kd, vd = dev(q), dev(k), dev(v)
    bm_d = dev(torch.full((hkv, T, bm_words), -1, dtype=torch.int64))
    a = torch.empty((T, hq * 128), dtype=torch.bfloat16, device="cuda")
    b = torch.empty_like(a)
    c.call("cpmcu_sparse_attention", ptr(qd), q.shape[1], ptr(kd), ptr(vd), budget, T, hq, hkv, ptr(kv_len), 0, None, 0,
           ptr(bm_d), bm_words, 1, 2, ptr(a), hq * 128)
    c.call("cpmcu_tree_attention", ptr(qd), q.shape[1], ptr(kd), ptr(vd), budget, T, hq, hkv, ptr(kv_len), 0, None, None,
           0, 0, 2, ptr(b), hq * 128)
    assert torch.equal(a, b)
