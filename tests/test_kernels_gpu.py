"""Kernel-level parity tests, each through the C ABI of libcpmcu_b200.so.

Floating-point kernels are compared with a plain fp32 PyTorch statement of the
same op (tolerance written in each test); integer stages are compared bit for
bit with the numpy oracle in oracle/tree.py.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def C():
    import cpmcu.C as c
    c.load()
    return c


def dev(t):
    return t.to("cuda").contiguous()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


# ------------------------------------------------------------------ linear
LINEAR_CASES = [
    # M, N, K, grid_limit (0 = one CTA per SM)
    (1, 256, 256, 0), (7, 384, 512, 0), (10, 4200, 1024, 0), (16, 1024, 4096, 0), (60, 4608, 4096, 0),
    (64, 512, 16384, 0), (33, 300, 128, 0), (17, 128, 64, 0), (130, 512, 256, 0), (300, 1024, 512, 0),
    (60, 1000, 2048, 3), (60, 1000, 2048, 7), (10, 4096, 4096, 5), (257, 640, 1024, 11), (1, 73448, 512, 0),
    # shapes whose tiles are cut into 2-4 k-pieces summed inside a thread-block cluster (o, down, draft fc; 30 and
    # 64 tokens for the other token tiles; 61 tokens: the last rank's share of the tokens is short)
    (60, 4096, 4096, 0), (60, 4096, 16384, 0), (10, 4096, 8192, 0), (30, 4096, 4096, 0), (64, 4096, 4096, 0),
    (61, 4608, 4096, 0), (3, 4608, 4096, 0),
    # prefill-sized launches (several token tiles): whole tiles in waves over the grid, the last partial wave cut along
    # K; 4100 tokens = two bands of token tiles, the second one tile high
    (700, 1024, 512, 7), (520, 384, 2048, 5), (2048, 4608, 512, 0), (4100, 1280, 256, 0),
]


@pytest.mark.parametrize("M,N,K,grid", LINEAR_CASES)
def test_linear_matches_fp32_matmul(M, N, K, grid):
    c = C()
    g = torch.Generator().manual_seed(M * 1000003 + N * 101 + K)
    x = dev((torch.randn(M, K, generator=g)).to(torch.bfloat16))
    w = dev((torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16))
    b = dev((torch.randn(N, generator=g)).to(torch.bfloat16))
    for bias in (None, b):
        y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        c.call("cpmcu_linear_bf16", ptr(x), ptr(w), ptr(bias), ptr(y), M, N, K, grid)
        ref = x.float() @ w.float().t()
        if bias is not None:
            ref = ref + bias.float()
        err = (y.float() - ref).abs()
        tol = 1e-2 * ref.abs() + 2e-2 * ref.abs().mean()  # bf16 store: 2^-8 relative, plus accumulation order
        assert torch.isfinite(y.float()).all()
        assert bool((err <= tol).all()), f"max err {err.max().item()} at M={M} N={N} K={K}"


W4_CASES = [
    # M, N, K, grid_limit
    (1, 128, 256, 0), (7, 384, 512, 0), (10, 4096, 1024, 0), (16, 1024, 4096, 0), (60, 4608, 4096, 0),
    (64, 512, 16384, 0), (33, 256, 256, 0), (130, 512, 256, 0), (300, 1024, 512, 0),
    (60, 1024, 2048, 3), (60, 1024, 2048, 7), (10, 4096, 4096, 5), (257, 640, 1024, 11),
    (60, 4096, 4096, 0), (60, 4096, 16384, 0), (30, 4608, 4096, 0), (61, 4096, 4096, 0),   # cluster split-K shapes
    (700, 1024, 512, 7), (4100, 1280, 256, 0), (1000, 512, 2048, 9),                       # waves of whole tiles + a cut tail
]


@pytest.mark.parametrize("M,N,K,grid", W4_CASES)
def test_linear_w4a16_matches_dequantised_matmul(M, N, K, grid):
    """4-bit streaming GEMM against x @ dequant(q)^T, weights in the converter's Marlin layout."""
    from oracle import marlin
    c = C()
    rng = np.random.default_rng(M * 7919 + N * 31 + K)
    w_kn = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    q, s = marlin.quantize_sym_int4(w_kn)
    packed, sperm = marlin.marlin_pack(q, s)
    deq = torch.from_numpy(marlin.dequantize(q, s))                       # [K, N] bf16-valued
    g = torch.Generator().manual_seed(M + N + K)
    x = dev(torch.randn(M, K, generator=g).to(torch.bfloat16))
    qw = dev(torch.from_numpy(packed.copy()))
    sc = dev(torch.from_numpy(sperm.copy()).to(torch.bfloat16))
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_linear_w4a16", ptr(x), ptr(qw), ptr(sc), ptr(y), M, N, K, grid)
    ref = x.float() @ dev(deq)
    err = (y.float() - ref).abs()
    tol = 1e-2 * ref.abs() + 2e-2 * ref.abs().mean()   # bf16 store + accumulation order; weights are exact
    assert torch.isfinite(y.float()).all()
    assert bool((err <= tol).all()), f"max err {err.max().item()} at M={M} N={N} K={K}"
    y2 = torch.empty_like(y)
    c.call("cpmcu_linear_w4a16", ptr(x), ptr(qw), ptr(sc), ptr(y2), M, N, K, grid)
    assert torch.equal(y, y2)                          # ticketed split-K sums in a fixed order


@pytest.mark.parametrize("M,inter,K,grid", [(100, 128, 128, 0), (129, 192, 256, 0), (600, 256, 512, 7), (2048, 2304, 512, 0),
                                            (4100, 640, 256, 0), (1, 64, 64, 0), (7, 320, 256, 0), (10, 2048, 512, 0),
                                            (60, 16384, 4096, 0), (33, 11008, 1024, 0), (60, 1024, 2048, 3)])
def test_linear_with_swiglu_epilogue_equals_linear_then_silu_gate(M, inter, K, grid):
    """The fused gate/up projection + activation against the two separate launches, at decode, draft and prefill row
    counts: bit-identical, because the epilogue rounds both projections to bf16 before the product exactly as the
    stored intermediate would be."""
    c = C()
    g = torch.Generator().manual_seed(M * 31 + inter * 7 + K)
    x = dev(torch.randn(M, K, generator=g).to(torch.bfloat16))
    w = dev((torch.randn(2 * inter, K, generator=g) * 0.08).to(torch.bfloat16))
    gu = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device="cuda")
    # one CTA: every tile is accumulated whole, in k order, as the fused launch does (a launch that cuts tiles along K
    # adds its fp32 partial sums in another order, which moves an occasional bf16 rounding of a projection by one step,
    # hence the second comparison below allows a few bf16 steps of the product)
    c.call("cpmcu_linear_bf16", ptr(x), ptr(w), None, ptr(gu), M, 2 * inter, K, 1)
    want = torch.empty(M, inter, dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_silu_gate", ptr(gu), ptr(want), M, inter)
    got = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_linear_swiglu_bf16", ptr(x), ptr(w), ptr(got), M, inter, K, grid)
    assert torch.isfinite(got.float()).all()
    assert float(want.float().abs().max()) > 0.1
    assert torch.equal(got, want)
    # against the launch as the engine would make it without the fusion (tiles possibly cut along K): one bf16 step
    c.call("cpmcu_linear_bf16", ptr(x), ptr(w), None, ptr(gu), M, 2 * inter, K, grid)
    c.call("cpmcu_silu_gate", ptr(gu), ptr(want), M, inter)
    diff = (got.float() - want.float()).abs()
    assert bool((diff <= 2.0 ** -6 * want.float().abs() + 1e-6).all())


def test_linear_is_deterministic():
    c = C()
    g = torch.Generator().manual_seed(5)
    x = dev(torch.randn(60, 4096, generator=g).to(torch.bfloat16))
    w = dev((torch.randn(4096, 4096, generator=g) * 0.02).to(torch.bfloat16))
    outs = []
    for _ in range(3):
        y = torch.empty(60, 4096, dtype=torch.bfloat16, device="cuda")
        c.call("cpmcu_linear_bf16", ptr(x), ptr(w), None, ptr(y), 60, 4096, 4096, 0)
        outs.append(y.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


def test_linear_rejects_bad_k():
    c = C()
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 100, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        c.call("cpmcu_linear_bf16", ptr(x), ptr(w), None, ptr(y), 4, 128, 100, 0)


# ------------------------------------------------------------------ attention
def ref_attention(q, kc, vc, kv_total, tq_valid, hq, hkv, mask, mask_k, window=0):
    tq = q.shape[0]
    d = 128
    grp = hq // hkv
    K = kc[:kv_total].float().view(kv_total, hkv, d)
    V = vc[:kv_total].float().view(kv_total, hkv, d)
    cols = torch.arange(kv_total, device=q.device)
    rows = torch.arange(tq, device=q.device)
    vis = cols[None, :] < (kv_total - tq_valid + rows[:, None] + 1)
    vis = vis & (rows[:, None] < tq_valid)
    if mask is not None and mask_k > 0:
        mbeg = kv_total - mask_k
        bits = torch.zeros(tq, kv_total, dtype=torch.bool, device=q.device)
        for t in range(tq):
            m = int(mask[t])
            for cc in range(mask_k):
                bits[t, mbeg + cc] = bool((m >> cc) & 1)
        vis = vis & ((cols[None, :] < mbeg) | bits)
    if window > 0:  # block-granular bound per 64-row query block, 128-key blocks
        for blk in range(0, tq, 64):
            lo_blk = (kv_total - tq_valid + blk + 127) // 128 - window // 128
            if lo_blk > 0:
                vis[blk:blk + 64] = vis[blk:blk + 64] & (cols[None, :] >= lo_blk * 128)
    out = torch.zeros(tq, hq, d, device=q.device)
    qf = q.float().view(tq, hq, d)
    for h in range(hq):
        s = (qf[:, h] @ K[:, h // grp].t()) / (d ** 0.5)
        s = s.masked_fill(~vis, float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
        out[:, h] = p @ V[:, h // grp]
    return out


def random_tree_masks(T, rng, max_depth=7):
    """Random ancestor-closed tree: node i hangs under an earlier node of depth < max_depth."""
    parent = [0] * T
    masks = [1] * T
    depth = [1] * T
    for i in range(1, T):
        while True:
            p = int(rng.integers(0, i))
            if depth[p] < max_depth:
                break
        parent[i] = p
        depth[i] = depth[p] + 1
        masks[i] = masks[p] | (1 << i)
    return masks, parent


ATTN_CASES = [
    # tq, hq, hkv, prefix L, mode, splits[, window]
    (10, 32, 2, 1500, "tree", 6, 512), (7, 32, 2, 1301, "valid3", 4, 256), (150, 4, 2, 700, "causal", 1, 384),
    (16, 2, 1, 300, "tree", 1), (16, 2, 1, 300, "tree", 3), (60, 32, 2, 1000, "tree", 4), (60, 32, 2, 129, "tree", 9),
    (10, 8, 2, 517, "tree", 5), (200, 4, 2, 0, "causal", 1), (130, 8, 2, 100, "causal", 1),
    (7, 32, 2, 777, "valid3", 6), (1, 32, 2, 400, "causal", 8), (64, 16, 1, 64, "tree", 2),
    # prefill-sized passes (four or more token tiles, one split): two token tiles per CTA; odd tile counts, a window,
    # a long prefix, rows beyond the valid count
    (600, 32, 2, 300, "causal", 1), (500, 4, 2, 1000, "causal", 1, 384), (300, 16, 1, 0, "causal", 1),
    (1000, 8, 2, 1040, "causal", 1), (260, 4, 2, 900, "valid3", 1), (72, 32, 2, 1900, "causal", 1, 256),
]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_tree_attention_matches_fp32(case):
    tq, hq, hkv, L, mode, splits = case[:6]
    window = case[6] if len(case) > 6 else 0
    c = C()
    rng = np.random.default_rng(tq * 7 + hq * 13 + L)
    g = torch.Generator().manual_seed(tq + hq + L)
    budget = 2048
    kvd = hkv * 128
    q_ld = (hq + 2 * hkv) * 128  # q lives inside a fused qkv row, as in the engine
    qkv = dev((torch.randn(tq, q_ld, generator=g)).to(torch.bfloat16))
    kc = dev((torch.randn(budget, kvd, generator=g)).to(torch.bfloat16))
    vc = dev((torch.randn(budget, kvd, generator=g)).to(torch.bfloat16))
    n_valid = None
    tq_valid = tq
    mask_t, mask_k, masks = None, 0, None
    if mode == "tree":
        kv_total = L + tq
        masks, _ = random_tree_masks(tq, rng)
        mask_t = dev(torch.tensor(np.array(masks, dtype=np.uint64).view(np.int64)))
        mask_k = tq
    elif mode == "causal":
        kv_total = L + tq
    else:  # only the first 3 rows are real, the device says so
        tq_valid = 3
        kv_total = L
        n_valid = dev(torch.tensor([tq_valid], dtype=torch.int32))
    kv_len = dev(torch.tensor([kv_total - 5], dtype=torch.int32))  # exercise the host-side addend
    out = torch.full((tq, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_tree_attention", ptr(qkv), q_ld, ptr(kc), ptr(vc), budget, tq, hq, hkv, ptr(kv_len), 5,
           ptr(n_valid), ptr(mask_t), mask_k, window, splits, ptr(out), hq * 128)
    q = qkv.view(tq, q_ld)[:, : hq * 128].contiguous().view(tq, hq, 128)
    ref = ref_attention(q, kc, vc, kv_total, tq_valid, hq, hkv, masks, mask_k, window)
    got = out.float().view(tq, hq, 128)
    assert torch.isfinite(got).all()
    err = (got[:tq_valid] - ref[:tq_valid]).abs().max().item()
    # P is rounded to bf16 before the PV product and the output is stored in bf16
    assert err < 3e-2, f"max abs err {err}"
    if tq_valid < tq:
        assert float(got[tq_valid:].abs().max()) == 0.0


# ------------------------------------------------------------------ small ops
def test_rms_norm_and_residual_add_bit_exact():
    c = C()
    g = torch.Generator().manual_seed(1)
    rows, dim, eps = 37, 4096, 1e-5
    x = dev(torch.randn(rows, dim, generator=g).to(torch.bfloat16))
    delta = dev(torch.randn(rows, dim, generator=g).to(torch.bfloat16))
    w = dev((1 + 0.1 * torch.randn(dim, generator=g)).to(torch.bfloat16))
    y = torch.empty_like(x)
    x1 = x.clone()
    c.call("cpmcu_rms_norm", ptr(x1), None, 1.0, ptr(w), ptr(y), rows, dim, eps)
    xf = x.float()
    ref = (torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * xf * w.float())
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    # with residual add: x is updated in place with bf16 rounding
    x2 = x.clone()
    c.call("cpmcu_rms_norm", ptr(x2), ptr(delta), 0.5, ptr(w), ptr(y), rows, dim, eps)
    d2 = (delta.float() * 0.5).to(torch.bfloat16)
    xs = (x.float() + d2.float()).to(torch.bfloat16)
    assert torch.equal(x2, xs)
    xf = xs.float()
    ref = (torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * xf * w.float())
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_rope_append_and_silu_and_argmax():
    c = C()
    g = torch.Generator().manual_seed(2)
    rows, hq, hkv, d = 9, 4, 2, 128
    ld = (hq + 2 * hkv) * d
    qkv = dev(torch.randn(rows, ld, generator=g).to(torch.bfloat16))
    orig = qkv.clone()
    inv_freq = dev(1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    pos = dev(torch.tensor([5, 6, 7, 7, 8, 100, 4000, 3, 0], dtype=torch.int32))
    kc = torch.zeros(64, hkv * d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros(64, hkv * d, dtype=torch.bfloat16, device="cuda")
    kv_len = dev(torch.tensor([20], dtype=torch.int32))
    c.call("cpmcu_rope_append", ptr(qkv), rows, hq, hkv, ptr(inv_freq), ptr(pos), ptr(kc), ptr(vc), ptr(kv_len), -3)

    def rope(x, nh):
        x = x.float().view(rows, nh, d)
        f = pos.float()[:, None] * inv_freq[None, :]
        cs, sn = torch.cos(f)[:, None, :], torch.sin(f)[:, None, :]
        a, b = x[..., :64], x[..., 64:]
        return torch.cat([a * cs - b * sn, a * sn + b * cs], -1).reshape(rows, nh * d)

    q_ref = rope(orig[:, : hq * d], hq)
    k_ref = rope(orig[:, hq * d:(hq + hkv) * d], hkv)
    assert (qkv[:, : hq * d].float() - q_ref).abs().max().item() < 4e-2
    assert (kc[17:17 + rows].float() - k_ref).abs().max().item() < 4e-2
    assert torch.equal(vc[17:17 + rows], orig[:, (hq + hkv) * d:])
    assert float(kc[:17].abs().max()) == 0.0 and float(kc[17 + rows:].abs().max()) == 0.0

    inter = 704
    gu = dev(torch.randn(rows, 2 * inter, generator=g).to(torch.bfloat16))
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_silu_gate", ptr(gu), ptr(out), rows, inter)
    gg, uu = gu[:, :inter].float(), gu[:, inter:].float()
    ref = gg * torch.sigmoid(gg) * uu
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-3

    vocab = 73448
    lg = dev(torch.randn(5, vocab, generator=g).to(torch.bfloat16))
    lg[2, 100] = 50.0
    lg[2, 70000] = 50.0  # tie: lowest index wins
    am = torch.empty(5, dtype=torch.int32, device="cuda")
    c.call("cpmcu_argmax", ptr(lg), 5, vocab, ptr(am))
    vals = lg.float()
    mx = vals.max(dim=1).values
    first = [(vals[r] == mx[r]).nonzero()[0].item() for r in range(5)]
    assert am.tolist() == first


# ------------------------------------------------------------------ draft tree (integer stage)
def run_gpu_tree(c, logits, k, num_iter, T, L, remap=None):
    V = logits.shape[1]
    tt = k + k * k * (num_iter - 1)
    ids = torch.zeros(T, dtype=torch.int32, device="cuda")
    pos = torch.zeros(T, dtype=torch.int32, device="cuda")
    mask = torch.zeros(T, dtype=torch.int64, device="cuda")
    par = torch.zeros(T, dtype=torch.int32, device="cuda")
    tv = torch.zeros(tt, dtype=torch.bfloat16, device="cuda")
    tp = torch.zeros(tt, dtype=torch.int32, device="cuda")
    tpar = torch.zeros(max(k * (num_iter - 1), 1), dtype=torch.int32, device="cuda")
    cl = dev(torch.tensor([L], dtype=torch.int32))
    rm = dev(torch.as_tensor(remap, dtype=torch.int32)) if remap is not None else None
    c.call("cpmcu_draft_tree_from_logits", ptr(logits), V, k, num_iter, T, ptr(rm), ptr(cl), ptr(ids), ptr(pos),
           ptr(mask), ptr(par), ptr(tv), ptr(tp), ptr(tpar))
    return (ids.cpu().numpy(), pos.cpu().numpy(), mask.cpu().numpy().view(np.uint64), par.cpu().numpy(),
            tv.float().cpu().numpy(), tp.cpu().numpy(), tpar.cpu().numpy())


@pytest.mark.parametrize("V,k,num_iter,T,coarse", [(4096, 4, 4, 16, False), (73448, 10, 6, 60, False),
                                                   (32768, 10, 6, 60, True), (5000, 8, 3, 64, True),
                                                   (4096, 1, 5, 5, False), (9000, 10, 6, 12, False)])
def test_draft_tree_bit_exact_given_logits(V, k, num_iter, T, coarse):
    from oracle import tree as otree
    c = C()
    g = torch.Generator().manual_seed(V + k)
    rows = 1 + (num_iter - 1) * k
    logits = torch.randn(rows, V, generator=g) * 3.0
    if coarse:  # many exact ties: values on a coarse grid
        logits = torch.round(logits * 2) / 2
    logits = logits.to(torch.bfloat16)
    remap = None
    if V == 32768:
        remap = np.random.default_rng(3).permutation(73448)[:V].astype(np.int32)
    L = 1234
    ids, pos, mask, par, tv, tp, tpar = run_gpu_tree(c, dev(logits), k, num_iter, T, L, remap)

    lf = logits.float().numpy()
    tree = otree.DraftTree(k, num_iter, T, remap)
    tree.level0(otree.log_softmax_bf16(lf[0]))
    for d in range(1, num_iter):
        blk = lf[1 + (d - 1) * k: 1 + d * k]
        tree.level(d, np.stack([otree.log_softmax_bf16(r) for r in blk]))
    o_ids, o_pos, o_mask, o_par, _ = tree.finalize(L, 0)
    tt = tree.total_tried
    same_history = np.array_equal(tv, tree.tried_val[:tt]) and np.array_equal(tp, tree.tried_pos[:tt])
    if not same_history:
        # the only tolerated difference: a log-probability one bf16 step away because the
        # fp32 sum of exponentials was accumulated in another order
        diff = np.abs(tv - tree.tried_val[:tt])
        assert diff.max() <= 0.0626 * 2 and (diff > 0).sum() <= 4, "history differs beyond a rounding flip"
        # integer stage must then still be exact given the history the GPU produced
        tree.tried_val[:tt], tree.tried_pos[:tt] = tv, tp
        tree.tried_parent[: len(tpar)] = tpar
        o_ids, o_pos, o_mask, o_par, _ = tree.finalize(L, 0)
    else:
        if num_iter > 1:
            assert np.array_equal(tpar[: k * (num_iter - 1)], tree.tried_parent[: k * (num_iter - 1)])
    assert np.array_equal(ids[1:], o_ids[1:])
    assert np.array_equal(pos, o_pos)
    assert np.array_equal(mask, o_mask)
    assert np.array_equal(par[1:], o_par[1:])
    # structural invariants of a draft tree
    for i in range(1, T):
        assert par[i] < i and (int(mask[i]) >> i) & 1 and bin(int(mask[i])).count("1") == pos[i] - L + 1


# ------------------------------------------------------------------ verify + compaction (integer stage)
@pytest.mark.parametrize("T,seed", [(16, 0), (60, 1), (60, 2), (64, 3), (2, 4), (60, 5)])
def test_verify_and_compact_bit_exact(T, seed):
    from oracle import tree as otree
    c = C()
    rng = np.random.default_rng(seed)
    L = 50 + seed
    masks, parent = random_tree_masks(T, rng)
    depth = [bin(m).count("1") for m in masks]
    pos = np.array([L + dd - 1 for dd in depth], dtype=np.int32)
    ids = rng.integers(0, 1000, T).astype(np.int32)
    gt = rng.integers(0, 1000, T).astype(np.int32)
    # make a few nodes correct so that paths of several lengths occur
    for i in range(1, T):
        if rng.random() < 0.6:
            ids[i] = gt[parent[i]]
    num_caches, kv_dim, rows = 6, 256, L + T + 8
    caches = [torch.randn(rows, kv_dim, generator=torch.Generator().manual_seed(seed * 10 + j)).to(torch.bfloat16)
              for j in range(num_caches)]
    d_caches = [dev(x) for x in caches]
    ptrs = dev(torch.tensor([x.data_ptr() for x in d_caches], dtype=torch.int64))
    d_ids = dev(torch.tensor(ids))
    result = torch.zeros(18, dtype=torch.int32, device="cuda")
    mask_t = dev(torch.tensor(np.array(masks, dtype=np.uint64).view(np.int64)))
    par_t = dev(torch.tensor(np.array(parent, dtype=np.int32)))
    gt_t, pos_t, len_t = dev(torch.tensor(gt)), dev(torch.tensor(pos)), dev(torch.tensor([L], dtype=torch.int32))
    c.call("cpmcu_verify_and_compact", T, ptr(d_ids), ptr(gt_t), ptr(pos_t), ptr(len_t), ptr(mask_t), ptr(par_t),
           ptr(ptrs), num_caches, kv_dim, 16, ptr(result))
    n, best, path = otree.verify(ids, gt, pos, L, masks, parent)
    res = result.cpu().numpy()
    assert res[0] == n and res[1] == best
    assert list(res[2:2 + n]) == path
    assert d_ids[:n].cpu().tolist() == otree.emitted_tokens(gt, path)
    for j in range(num_caches):
        ref = otree.compact_rows(caches[j].clone().view(torch.int16).numpy(), L, path)
        assert np.array_equal(d_caches[j].cpu().view(torch.int16).numpy(), ref)


@pytest.mark.parametrize("T,seed,scale,prev_rows", [(16, 0, 1.0, 5), (60, 1, 1.0, 7), (60, 2, 12.0, 7), (64, 3, 1.0, 16), (60, 5, 0.5, 3)])
def test_accept_fixup_gathers_hidden_states_embeddings_and_positions(T, seed, scale, prev_rows):
    """The whole one-launch tail of a step (reference MiniCPM4EagleImpl::verify, src/model/minicpm4/
    minicpm4_eagle.cuh:398-418): acceptance, K/V compaction, and for the next draft pass the gather of the target's
    final-norm rows along the accepted path (remap_hidden, src/model/eagle.cuh:108-115), the embeddings of the emitted
    tokens (scaled by scale_emb) and their positions; all bit for bit, capped at the drafter's row budget."""
    from oracle import tree as otree
    c = C()
    rng = np.random.default_rng(100 + seed)
    L, H, V = 70 + seed, 512, 1000
    masks, parent = random_tree_masks(T, rng)
    depth = [bin(m).count("1") for m in masks]
    pos = np.array([L + dd - 1 for dd in depth], dtype=np.int32)
    ids = rng.integers(0, V, T).astype(np.int32)
    gt = rng.integers(0, V, T).astype(np.int32)
    for i in range(1, T):
        if rng.random() < 0.7:
            ids[i] = gt[parent[i]]
    num_caches, kv_dim, rows = 4, 256, L + T + 8
    g = torch.Generator().manual_seed(seed)
    caches = [torch.randn(rows, kv_dim, generator=g).to(torch.bfloat16) for _ in range(num_caches)]
    d_caches = [dev(x) for x in caches]
    ptrs = dev(torch.tensor([x.data_ptr() for x in d_caches], dtype=torch.int64))
    norm_out = dev(torch.randn(64, H, generator=g).to(torch.bfloat16))
    embed = dev(torch.randn(V, H, generator=g).to(torch.bfloat16))
    prev_hidden = torch.full((16, H), 7.0, dtype=torch.bfloat16, device="cuda")
    prev_embed = torch.full((16, H), 7.0, dtype=torch.bfloat16, device="cuda")
    eagle_pos = torch.full((16,), -1, dtype=torch.int32, device="cuda")
    d_ids = dev(torch.tensor(ids))
    result = torch.zeros(18, dtype=torch.int32, device="cuda")
    mask_t = dev(torch.tensor(np.array(masks, dtype=np.uint64).view(np.int64)))
    par_t = dev(torch.tensor(np.array(parent, dtype=np.int32)))
    gt_t, pos_t, len_t = dev(torch.tensor(gt)), dev(torch.tensor(pos)), dev(torch.tensor([L], dtype=torch.int32))
    c.call("cpmcu_accept_fixup", T, ptr(d_ids), ptr(gt_t), ptr(pos_t), ptr(len_t), ptr(mask_t), ptr(par_t), ptr(ptrs),
           num_caches, kv_dim, rows, prev_rows, H, ptr(norm_out), ptr(prev_hidden), ptr(embed), scale, ptr(prev_embed),
           ptr(eagle_pos), ptr(result))
    n, best, path = otree.verify(ids, gt, pos, L, masks, parent)
    tokens = otree.emitted_tokens(gt, path)
    res = result.cpu().numpy()
    assert res[0] == n and res[1] == best and list(res[2:2 + n]) == path
    assert d_ids[:n].cpu().tolist() == tokens
    m = min(n, prev_rows)                      # the drafter keeps at most its row budget
    assert torch.equal(prev_hidden[:m], norm_out[torch.tensor(path[:m], device="cuda")])
    want_emb = embed[torch.tensor(tokens[:m], device="cuda")]
    if scale != 1.0:
        want_emb = (want_emb.float() * scale).to(torch.bfloat16)
    assert torch.equal(prev_embed[:m], want_emb)
    assert eagle_pos[:prev_rows].cpu().tolist() == [L + i for i in range(prev_rows)]
    assert float(prev_hidden[m:].float().min()) == 7.0 and float(prev_embed[m:].float().min()) == 7.0   # untouched
    for j in range(num_caches):
        ref = otree.compact_rows(caches[j].clone().view(torch.int16).numpy(), L, path[:m])
        assert np.array_equal(d_caches[j].cpu().view(torch.int16).numpy(), ref)


def test_accept_fixup_refuses_to_compact_past_the_cache():
    """cache_rows guards the compaction: rows at or beyond it are not touched and the call reports the overflow."""
    c = C()
    T, L = 4, 10
    caches = [torch.zeros(12, 256, dtype=torch.bfloat16, device="cuda")]
    ptrs = dev(torch.tensor([caches[0].data_ptr()], dtype=torch.int64))
    ids = dev(torch.tensor([5, 6, 7, 8], dtype=torch.int32))
    gt = dev(torch.tensor([6, 7, 8, 9], dtype=torch.int32))          # the chain 0-1-2-3 is accepted: n = 4
    pos = dev(torch.tensor([10, 11, 12, 13], dtype=torch.int32))
    mask = dev(torch.tensor([1, 3, 7, 15], dtype=torch.int64))
    par = dev(torch.tensor([0, 0, 1, 2], dtype=torch.int32))
    result = torch.zeros(18, dtype=torch.int32, device="cuda")
    len_t = dev(torch.tensor([L], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="kernel error flags 8"):
        c.call("cpmcu_accept_fixup", T, ptr(ids), ptr(gt), ptr(pos), ptr(len_t), ptr(mask), ptr(par), ptr(ptrs), 1, 256, 12,
               7, 0, None, None, None, 1.0, None, None, ptr(result))
    assert float(caches[0].float().abs().max()) == 0.0
