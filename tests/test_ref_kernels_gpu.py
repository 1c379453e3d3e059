"""The library against the reference project's OWN kernels, through the C ABI.

Two forms: (1) against tests/golden/ref_kernels_golden.json, vectors those kernels produced on a B200
(always runs); (2) live, against oracle/_ref/libcpmcu_ref_kernels.so and libcpmcu_ref_marlin.so on the
same device buffers (skipped when the prebuilt libraries are not in the tree).  Integer stages are
bit-exact; float stages carry their tolerance in the test."""
import ctypes
import importlib.util
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
_spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(HERE, "golden", "make_ref_golden.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)
with open(os.path.join(HERE, "golden", "ref_kernels_golden.json")) as f:
    GOLD = json.load(f)

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcpmcu_ref_kernels.so")
REF_MARLIN = os.path.join(ROOT, "oracle", "_ref", "libcpmcu_ref_marlin.so")


def C():
    import cpmcu.C as c
    c.load()
    return c


_ref = {}


def ref_lib(path=REF_LIB):
    if not os.path.exists(path):
        pytest.skip("prebuilt reference kernels not in the tree (oracle/build_ref.py builds them from a reference checkout)")
    if path not in _ref:
        _ref[path] = ctypes.CDLL(path)
    return _ref[path]


def dev(t):
    return t.to("cuda").contiguous()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def from_bits(b):
    return torch.tensor(b, dtype=torch.int16).view(torch.bfloat16).float()


def lib_tree(c, logits, k, num_iter, T, L, remap):
    V = logits.shape[1]
    tt = k + k * k * (num_iter - 1)
    ids = torch.zeros(64, dtype=torch.int32, device="cuda")
    pos = torch.zeros(64, dtype=torch.int32, device="cuda")
    mask = torch.zeros(64, dtype=torch.int64, device="cuda")
    par = torch.zeros(64, dtype=torch.int32, device="cuda")
    tv = torch.zeros(tt + 64, dtype=torch.bfloat16, device="cuda")
    tp = torch.zeros(tt + 64, dtype=torch.int32, device="cuda")
    tpar = torch.zeros(k * num_iter + 64, dtype=torch.int32, device="cuda")
    cl = dev(torch.tensor([L], dtype=torch.int32))
    return (ids, pos, mask, par, tv, tp, tpar, cl, V, tt)


def check_tree_against(c_case, got, k, num_iter, T, L, remap):
    """got/want: dicts of numpy arrays.  The log-probabilities may differ by a rounding flip (the fp32 sum of
    exponentials is accumulated in another order, and the reference is built with fast-math); when the
    candidate history is identical everything after it must be identical too, otherwise the integer stage
    is re-derived from the library's own history by the (reference-pinned) oracle."""
    from oracle import tree as otree
    want = c_case
    same = np.array_equal(got["tv"], want["tv"]) and np.array_equal(got["tp"], want["tp"])
    if same:
        assert np.array_equal(got["tpar"], want["tpar"])
        for key in ("ids", "pos", "mask", "par"):
            assert np.array_equal(got[key], want[key]), key
        return True
    diff = np.abs(got["tv"] - want["tv"])
    assert diff.max() <= 0.0626 * 2 and (diff > 0).sum() <= 4, "history differs beyond a rounding flip"
    tree = otree.DraftTree(k, num_iter, T, remap)
    tt = tree.total_tried
    tree.tried_val[:tt], tree.tried_pos[:tt] = got["tv"], got["tp"]
    tree.tried_parent[: len(got["tpar"])] = got["tpar"]
    o_ids, o_pos, o_mask, o_par, _ = tree.finalize(L, 0)
    assert np.array_equal(got["ids"], o_ids[1:]) and np.array_equal(got["pos"], o_pos)
    assert np.array_equal(got["mask"], o_mask) and np.array_equal(got["par"], o_par[1:])
    return False


def run_tree(fn, logits, k, num_iter, T, L, remap_np):
    bufs = lib_tree(None, logits, k, num_iter, T, L, remap_np)
    ids, pos, mask, par, tv, tp, tpar, cl, V, tt = bufs
    rm = dev(torch.from_numpy(remap_np)) if remap_np is not None else None
    fn(ptr(logits), V, k, num_iter, T, ptr(rm), ptr(cl), ptr(ids), ptr(pos), ptr(mask), ptr(par), ptr(tv), ptr(tp),
       ptr(tpar))
    torch.cuda.synchronize()
    return {"ids": ids[1:T].cpu().numpy(), "pos": pos[:T].cpu().numpy(),
            "mask": mask[:T].cpu().numpy().view(np.uint64), "par": par[1:T].cpu().numpy(),
            "tv": tv[:tt].float().cpu().numpy(), "tp": tp[:tt].cpu().numpy(),
            "tpar": tpar[: k * (num_iter - 1)].cpu().numpy()}


@pytest.mark.parametrize("case", GOLD["trees"], ids=lambda c: "seed%d" % c["seed"])
def test_draft_tree_equals_reference_golden(case):
    c = C()
    V, k, it, T, L = case["V"], case["k"], case["num_iter"], case["T"], case["cache_length"]
    logits = dev(gen.tree_logits(case["seed"], V, k, it, case["coarse"]))
    remap = gen.fr_remap(case["seed"], V, case["full_vocab"]) if case["full_vocab"] else None
    got = run_tree(lambda *a: c.call("cpmcu_draft_tree_from_logits", *a), logits, k, it, T, L, remap)
    want = {"ids": np.array(case["ids"]), "pos": np.array(case["pos"]),
            "mask": np.array(case["mask"], dtype=np.uint64), "par": np.array(case["parent"]),
            "tv": from_bits(case["tried_val_bits"]).numpy(), "tp": np.array(case["tried_pos"]),
            "tpar": np.array(case["tried_parent"])}
    check_tree_against(want, got, k, it, T, L, remap)


@pytest.mark.parametrize("V,k,it,T,coarse,full", [(73448, 10, 6, 60, False, 0), (32768, 10, 6, 60, True, 73448),
                                                 (4096, 4, 4, 16, True, 0), (9000, 10, 6, 12, False, 0)])
def test_draft_tree_equals_reference_live(V, k, it, T, coarse, full):
    """The headline tree shape (vocabulary 73448 and the 32768-entry FR-Spec subset, 6 levels of 10, 60 nodes)
    on the same device logits through both libraries."""
    c, r = C(), ref_lib()
    L = 4100
    logits = dev(gen.tree_logits(V % 1000 + k, V, k, it, coarse))
    remap = gen.fr_remap(7, V, full) if full else None
    got = run_tree(lambda *a: c.call("cpmcu_draft_tree_from_logits", *a), logits, k, it, T, L, remap)

    def ref_call(*a):
        assert r.refk_draft_tree_from_logits(*a) == 0
    want = run_tree(ref_call, logits, k, it, T, L, remap)
    check_tree_against(want, got, k, it, T, L, remap)


@pytest.mark.parametrize("case", GOLD["verify"], ids=lambda c: "seed%d" % c["seed"])
def test_verify_and_compact_equals_reference_golden(case):
    c = C()
    T, L = case["T"], case["L"]
    ids, gt, pos, masks, parent = gen.verify_inputs(case["seed"], T, L)
    num_caches, dim, rows = 4, 256, L + T + 8
    before = [gen.cache_pattern(j, rows, dim) for j in range(num_caches)]
    caches = [dev(b.view(torch.bfloat16)) for b in before]
    ptrs = dev(torch.tensor([x.data_ptr() for x in caches], dtype=torch.int64))
    pred = dev(torch.tensor(ids, dtype=torch.int32))
    result = torch.zeros(18, dtype=torch.int32, device="cuda")
    mask_t = dev(torch.from_numpy(np.array(masks, dtype=np.uint64).view(np.int64)))
    gt_t, pos_t = dev(torch.tensor(gt, dtype=torch.int32)), dev(torch.tensor(pos, dtype=torch.int32))
    len_t, par_t = dev(torch.tensor([L], dtype=torch.int32)), dev(torch.tensor(parent, dtype=torch.int32))
    c.call("cpmcu_verify_and_compact", T, ptr(pred), ptr(gt_t), ptr(pos_t), ptr(len_t), ptr(mask_t), ptr(par_t),
           ptr(ptrs), num_caches, dim, 16, ptr(result))
    res = result.cpu().tolist()
    n = case["n"]
    assert res[0] == n and res[1] == case["best"] and res[2:2 + n] == case["path"]
    assert pred[:n].cpu().tolist() == case["tokens"]
    for j in range(num_caches):
        want = before[j].clone()
        for i, p in enumerate(case["path"]):
            want[L + i] = before[j][L + p]
        assert torch.equal(caches[j].view(torch.int16).cpu(), want)


@pytest.mark.parametrize("T,hq,hkv,L,top,sink,window,lse", [(12, 8, 2, 4200, 6, 1, 4, True),
                                                           (60, 32, 2, 8000, 16, 1, 8, True),
                                                           (7, 8, 2, 5000, 64, 2, 2, False),
                                                           (5, 8, 2, 33000, 64, 1, 32, True)])
def test_block_selection_equals_reference_live(T, hq, hkv, L, top, sink, window, lse):
    """Compressed keys and the integer part of the selection (max-pool, top-k, bitmask): the reference's
    kernels on the library's own stage-1 scores must give the library's block mask, bit for bit."""
    c, r = C(), ref_lib()
    g = torch.Generator().manual_seed(L + T)
    budget = (L + T + 127) // 128 * 128
    kv_dim, q_ld = hkv * 128, (hq + 2 * hkv) * 128
    q = dev(torch.randn(T, q_ld, generator=g).to(torch.bfloat16))
    base = torch.cumsum(torch.randn(budget // 64 + 1, kv_dim, generator=g), dim=0) * 0.5
    k = dev((base.repeat_interleave(64, dim=0)[:budget] + torch.randn(budget, kv_dim, generator=g)).to(torch.bfloat16))
    score_ld = (budget // 16 + 127) // 128 * 128
    words = (budget // 64 + 63) // 64
    c1 = torch.zeros(budget // 16, kv_dim, dtype=torch.bfloat16, device="cuda")
    c2 = torch.zeros(budget // 64, kv_dim, dtype=torch.bfloat16, device="cuda")
    scores = torch.zeros(hkv, T, score_ld, dtype=torch.bfloat16, device="cuda")
    bm = torch.zeros(hkv, T, words, dtype=torch.int64, device="cuda")
    kv_len = dev(torch.tensor([L], dtype=torch.int32))
    c.call("cpmcu_sparse_select", ptr(q), q_ld, T, hq, hkv, ptr(k), budget, ptr(kv_len), 0, sink, window, top, 256,
           int(lse), ptr(c1), ptr(c2), ptr(scores), score_ld, ptr(bm), words)
    # compressed keys: same fp32 mean, possibly another summation order -> a bf16 rounding flip at most
    n1, n2 = max((L - 16) // 16, 0), max((L - 64) // 64, 0)
    r1 = torch.zeros_like(c1)
    r2 = torch.zeros_like(c2)
    assert r.refk_compress(ptr(k), L, kv_dim, ptr(r1), ptr(r2)) == 0
    for got, want, n in ((c1, r1, n1), (c2, r2, n2 if lse else 0)):
        if n == 0:
            continue
        gf, wf = got[:n].float(), want[:n].float()
        assert float((gf - wf).abs().max()) <= 2 ** -7 * float(wf.abs().max())
        assert float((gf == wf).float().mean()) > 0.98
    out_len = (L + 63) // 64
    pool = torch.zeros(hkv, T, out_len, dtype=torch.bfloat16, device="cuda")
    rbm = torch.zeros(hkv * T, words, dtype=torch.int64, device="cuda")
    assert r.refk_select_from_scores(ptr(scores), hkv, T, T, score_ld, L, sink, window, top, budget, ptr(pool),
                                     ptr(rbm)) == 0
    assert torch.equal(bm.view(hkv * T, words), rbm)


def test_row_kernels_equal_reference_live():
    """rms_norm (+ residual add), rotary embedding, gated SiLU and the embedding gather against the
    reference's kernels.  The reference is built with fast-math, so a result may sit one bf16 step away."""
    c, r = C(), ref_lib()
    g = torch.Generator().manual_seed(5)
    rows, dim, eps = 60, 4096, 1e-5
    x = dev(torch.randn(rows, dim, generator=g).to(torch.bfloat16))
    delta = dev(torch.randn(rows, dim, generator=g).to(torch.bfloat16))
    w = dev((1 + 0.1 * torch.randn(dim, generator=g)).to(torch.bfloat16))

    def close(a, b, frac=0.97):
        af, bf = a.float(), b.float()
        assert float((af - bf).abs().max()) <= 2 ** -7 * float(bf.abs().max()) + 1e-6
        assert float((af == bf).float().mean()) >= frac

    y, ry = torch.empty_like(x), torch.empty_like(x)
    x1 = x.clone()
    c.call("cpmcu_rms_norm", ptr(x1), None, 1.0, ptr(w), ptr(y), rows, dim, eps)
    assert r.refk_rms_norm(ptr(x), ptr(w), ptr(ry), rows, dim, ctypes.c_float(eps)) == 0
    close(y, ry)
    x2, rx2 = x.clone(), x.clone()
    c.call("cpmcu_rms_norm", ptr(x2), ptr(delta), 1.0, ptr(w), ptr(y), rows, dim, eps)
    assert r.refk_add_and_rms_norm(ptr(rx2), ptr(delta), ptr(w), ptr(ry), rows, dim, ctypes.c_float(eps)) == 0
    assert torch.equal(x2, rx2)          # the residual stream itself: one bf16 add, bit-exact
    close(y, ry)

    hq, hkv, d = 32, 2, 128
    ld = (hq + 2 * hkv) * d
    qkv = dev(torch.randn(rows, ld, generator=g).to(torch.bfloat16))
    inv_freq = dev(1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d)))
    pos = dev((torch.arange(rows, dtype=torch.int32) % 7) + 4090)
    rq = qkv[:, : hq * d].contiguous()
    rk = qkv[:, hq * d:(hq + hkv) * d].contiguous()
    kc = torch.zeros(128, hkv * d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros(128, hkv * d, dtype=torch.bfloat16, device="cuda")
    mine = qkv.clone()
    kv_len = dev(torch.tensor([10], dtype=torch.int32))
    c.call("cpmcu_rope_append", ptr(mine), rows, hq, hkv, ptr(inv_freq), ptr(pos), ptr(kc), ptr(vc), ptr(kv_len), 0)
    assert r.refk_rotary(ptr(rq), ptr(rk), rows, hq, hkv, d, ptr(inv_freq), ptr(pos)) == 0
    # fast-math sin/cos at angles up to ~4100 rad lose a few bits; the library uses the accurate versions
    assert float((mine[:, : hq * d].float() - rq.float()).abs().max()) <= 4e-2
    assert float((kc[10:10 + rows].float() - rk.float()).abs().max()) <= 4e-2
    assert float((mine[:, : hq * d].float() == rq.float()).float().mean()) > 0.7

    inter = 16384
    gu = dev(torch.randn(rows, 2 * inter, generator=g).to(torch.bfloat16))
    out, rout = (torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    c.call("cpmcu_silu_gate", ptr(gu), ptr(out), rows, inter)
    assert r.refk_gated_silu(ptr(gu), ptr(rout), rows, inter) == 0
    close(out, rout, frac=0.95)


@pytest.mark.parametrize("M,N,K", [(60, 4608, 4096), (10, 4096, 4096), (7, 1024, 16384), (60, 73448, 4096)])
def test_linear_equals_reference_cublas_live(M, N, K):
    """The library's GEMM against the reference's own call (linear<T>: cublasGemmEx, fp32 accumulate)."""
    c, r = C(), ref_lib()
    g = torch.Generator().manual_seed(M + N)
    x = dev(torch.randn(M, K, generator=g).to(torch.bfloat16))
    w = dev((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16))
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ry = torch.empty_like(y)
    c.call("cpmcu_linear_bf16", ptr(x), ptr(w), None, ptr(y), M, N, K, 0)
    assert r.refk_linear(ptr(x), ptr(w), ptr(ry), M, N, K) == 0
    yf, rf = y.float(), ry.float()
    # both accumulate bf16 products in fp32; only the summation order differs: one bf16 step of the result
    assert bool(((yf - rf).abs() <= 2 ** -7 * rf.abs() + 2e-3 * rf.abs().mean()).all())
    assert float((yf == rf).float().mean()) > 0.9


@pytest.mark.parametrize("M,N,K", [(60, 4608, 4096), (10, 4096, 4096), (60, 4096, 16384), (1, 1024, 1024), (33, 512, 256)])
def test_w4a16_equals_reference_marlin_live(M, N, K):
    """The library's W4A16 GEMM against the reference's Marlin kernel on the same converter-format tensors."""
    from oracle import marlin
    c, r = C(), ref_lib(REF_MARLIN)
    rng = np.random.default_rng(M + N + K)
    w_kn = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    q, s = marlin.quantize_sym_int4(w_kn)
    packed, sperm = marlin.marlin_pack(q, s)
    x = dev(torch.randn(M, K, generator=torch.Generator().manual_seed(K)).to(torch.bfloat16))
    qw = dev(torch.from_numpy(packed.copy()))
    sc = dev(torch.from_numpy(sperm.copy()).to(torch.bfloat16))
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ry = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_linear_w4a16", ptr(x), ptr(qw), ptr(sc), ptr(y), M, N, K, 0)
    assert r.refk_marlin_gemm(ptr(x), ptr(qw), ptr(sc), ptr(ry), M, N, K) == 0
    yf, rf = y.float(), ry.float()
    assert torch.isfinite(rf).all()
    # Marlin multiplies (q - 8) by the scale after the MMA's A-side conversion, the library before it
    # (one extra bf16 rounding of the weight on either side): tolerance of the dequantised-matmul test
    assert bool(((yf - rf).abs() <= 1e-2 * rf.abs() + 2e-2 * rf.abs().mean()).all())
    # and the reference kernel itself reads marlin_pack's layout as the oracle says it does
    deq = x.float() @ dev(torch.from_numpy(marlin.dequantize(q, s)))
    assert bool(((rf - deq).abs() <= 1e-2 * deq.abs() + 2e-2 * deq.abs().mean()).all())
