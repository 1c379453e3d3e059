"""The library's attention kernels against the reference project's OWN attention code, live on the same
device buffers: oracle/_ref/libcpmcu_ref_flash.so is the reference's FlashAttention fork (mha_fwd_kvcache,
mha_fwd_stage1, src/flash_attn/flash_api.hpp:204-392) compiled from a reference checkout by
oracle/build_ref.py; the tests skip when the prebuilt library is not in the tree.

Covers the four ways the speculative step calls it: tree-verify (64-bit tree mask over the last T keys), a
draft level with a sliding window (block-granular, flash_blockmask.h:29-45), the unsplit causal prefill call,
and the InfLLM-v2 pair stage-1 scoring + block-sparse attention.  Tolerance for all float outputs: largest
absolute difference <= 2e-2 of the largest reference magnitude (both sides round P and the output to bf16,
and sum in different orders); the fp32 PyTorch statement is printed beside it for scale."""
import ctypes
import os

import numpy as np
import pytest
import torch

from test_kernels_gpu import random_tree_masks, ref_attention

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_FLASH = os.path.join(ROOT, "oracle", "_ref", "libcpmcu_ref_flash.so")
REL_TOL = 2e-2

_lib = {}


def C():
    import cpmcu.C as c
    c.load()
    return c


def ref_flash():
    if not os.path.exists(REF_FLASH):
        pytest.skip("prebuilt reference attention not in the tree (python -m oracle.build_ref --flash builds it)")
    if "l" not in _lib:
        _lib["l"] = ctypes.CDLL(REF_FLASH)
    return _lib["l"]


def dev(t):
    return t.to("cuda").contiguous()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def u64(values):
    return dev(torch.from_numpy(np.array(values, dtype=np.uint64).view(np.int64)))


def make_qkv(tq, hq, hkv, rows, seed, peaked=1.0):
    g = torch.Generator().manual_seed(seed)
    kvd = hkv * 128
    q_ld = (hq + 2 * hkv) * 128                      # q sits inside a fused qkv row, as in the engine
    qkv = dev((torch.randn(tq, q_ld, generator=g) * peaked).to(torch.bfloat16))
    kc = dev(torch.randn(rows, kvd, generator=g).to(torch.bfloat16))
    vc = dev(torch.randn(rows, kvd, generator=g).to(torch.bfloat16))
    return qkv, kc, vc, q_ld


def max_rel(a, b):
    return float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-20)


def draft_tree_masks(c, k=10, num_iter=6, T=60, seed=5):
    """Tree masks of a real draft tree: the library's tree builder on seeded logits (that stage is pinned bit
    for bit against the reference's own tree kernels elsewhere)."""
    V = 4096
    g = torch.Generator().manual_seed(seed)
    logits = dev((torch.randn(1 + (num_iter - 1) * k, V, generator=g) * 3).to(torch.bfloat16))
    tt = k + k * k * (num_iter - 1)
    ids = torch.zeros(64, dtype=torch.int32, device="cuda")
    pos = torch.zeros(64, dtype=torch.int32, device="cuda")
    mask = torch.zeros(64, dtype=torch.int64, device="cuda")
    par = torch.zeros(64, dtype=torch.int32, device="cuda")
    tv = torch.zeros(tt + 64, dtype=torch.bfloat16, device="cuda")
    tp = torch.zeros(tt + 64, dtype=torch.int32, device="cuda")
    tpar = torch.zeros(k * num_iter + 64, dtype=torch.int32, device="cuda")
    cl = dev(torch.tensor([4096], dtype=torch.int32))
    c.call("cpmcu_draft_tree_from_logits", ptr(logits), V, k, num_iter, T, None, ptr(cl), ptr(ids), ptr(pos), ptr(mask),
           ptr(par), ptr(tv), ptr(tp), ptr(tpar))
    words = mask[:T].cpu().numpy().view(np.uint64)
    assert all(int(words[i]) >> i & 1 for i in range(T))
    return [int(w) for w in words]


TREE_CASES = [
    # tq, hq, hkv, prefix L, splits of the library launch, mask kind
    (60, 32, 2, 4096, 9, "draft"),        # the headline verify shape with a real draft tree
    (60, 32, 2, 4096, 9, "random"),
    (60, 32, 2, 4267, 9, "random"),       # prefix not a multiple of the key tile
    (16, 2, 1, 300, 3, "random"),
    (10, 8, 2, 517, 5, "random"),
    (64, 16, 1, 64, 2, "random"),
    (33, 32, 2, 1000, 4, "random"),
    (1, 32, 2, 400, 8, "none"),           # plain one-token decode
]


@pytest.mark.parametrize("tq,hq,hkv,L,splits,kind", TREE_CASES)
def test_tree_verify_attention_matches_reference(tq, hq, hkv, L, splits, kind):
    c, r = C(), ref_flash()
    kv_total = L + tq
    padded = (kv_total + 127) // 128 * 128
    qkv, kc, vc, q_ld = make_qkv(tq, hq, hkv, padded + 128, seed=tq * 31 + L)
    if kind == "draft":
        masks = draft_tree_masks(c, T=tq)
    elif kind == "random":
        masks, _ = random_tree_masks(tq, np.random.default_rng(L + tq))
    else:
        masks = None
    mask_t = u64(masks) if masks is not None else None
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    ours = torch.full((tq, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_tree_attention", ptr(qkv), q_ld, ptr(kc), ptr(vc), padded + 128, tq, hq, hkv, ptr(kv_len), 0, None,
           ptr(mask_t), tq if masks is not None else 0, 0, splits, ptr(ours), hq * 128)
    q = qkv[:, : hq * 128].contiguous()
    theirs = torch.full((tq, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert r.refk_mha_fwd_kvcache(tq, padded, hq, hkv, ptr(q), ptr(kc), ptr(vc), ptr(kv_len), ptr(mask_t),
                                  tq if masks is not None else 0, ptr(theirs), None, 0) == 0
    assert torch.isfinite(theirs.float()).all() and torch.isfinite(ours.float()).all()
    fp32 = ref_attention(q.view(tq, hq, 128), kc, vc, kv_total, tq, hq, hkv, masks, tq if masks is not None else 0)
    e_ours, e_ref = max_rel(ours.view(tq, hq, 128), fp32), max_rel(theirs.view(tq, hq, 128), fp32)
    print("library vs reference %.4f; vs fp32: library %.4f, reference %.4f" % (max_rel(ours, theirs), e_ours, e_ref))
    assert max_rel(ours, theirs) <= REL_TOL
    assert e_ref <= REL_TOL and e_ours <= REL_TOL


WINDOW_CASES = [
    # tq (= k), draft level d (mask over k*d keys), prefix L, window tokens
    (10, 1, 3000, 1024), (10, 3, 3001, 1024), (10, 5, 3063, 1024), (10, 2, 3064, 1024), (10, 4, 3127, 1024),
    (10, 5, 3200, 1024), (10, 1, 900, 1024), (10, 5, 1100, 1024), (7, 0, 2500, 1024), (10, 3, 5000, 512),
]


@pytest.mark.parametrize("tq,level,L,window", WINDOW_CASES)
def test_draft_window_attention_matches_reference(tq, level, L, window):
    """A draft level: k rows, the tree mask covers the k*level draft keys appended so far, the prefix is cut
    by the block-granular sliding window.  level 0 is the catch-up pass (causal, no tree mask)."""
    c, r = C(), ref_flash()
    hq, hkv = 32, 2
    rng = np.random.default_rng(L + level)
    if level > 0:
        mask_k = tq * level
        kv_total = L + mask_k
        # row i continues some chain of earlier levels: random ancestors plus its own key at the current level
        masks = []
        for i in range(tq):
            w = 1 << (tq * (level - 1) + i)
            for lv in range(level - 1):
                w |= 1 << (tq * lv + int(rng.integers(0, tq)))
            masks.append(w)
    else:
        mask_k, kv_total, masks = 0, L + tq, None
    # eagle_padded_length = (L + 255) / 128 * 128 (src/model/minicpm4/minicpm4_eagle.cuh:307)
    padded = (L + 255) // 128 * 128
    qkv, kc, vc, q_ld = make_qkv(tq, hq, hkv, padded + 128, seed=L * 7 + level)
    mask_t = u64(masks) if masks is not None else None
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    ours = torch.full((tq, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_tree_attention", ptr(qkv), q_ld, ptr(kc), ptr(vc), padded + 128, tq, hq, hkv, ptr(kv_len), 0, None,
           ptr(mask_t), mask_k, window, 8, ptr(ours), hq * 128)
    q = qkv[:, : hq * 128].contiguous()
    theirs = torch.full((tq, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert r.refk_mha_fwd_kvcache(tq, padded, hq, hkv, ptr(q), ptr(kc), ptr(vc), ptr(kv_len), ptr(mask_t), mask_k,
                                  ptr(theirs), None, window) == 0
    assert torch.isfinite(theirs.float()).all() and torch.isfinite(ours.float()).all()
    print("library vs reference %.4f" % max_rel(ours, theirs))
    assert max_rel(ours, theirs) <= REL_TOL


PREFILL_CASES = [
    # tokens, hq, hkv, history, window
    (150, 4, 2, 700, 0), (200, 4, 2, 0, 0), (130, 8, 2, 100, 0), (256, 32, 2, 1024, 0), (300, 8, 2, 1500, 1024),
    (128, 8, 2, 2048, 512),
]


@pytest.mark.parametrize("tokens,hq,hkv,history,window", PREFILL_CASES)
def test_prefill_attention_matches_reference(tokens, hq, hkv, history, window):
    """The chunked-prefill call: causal, no tree mask, cache length given on the host, one split."""
    c, r = C(), ref_flash()
    kv_total = history + tokens
    rows = (kv_total + 255) // 128 * 128
    qkv, kc, vc, q_ld = make_qkv(tokens, hq, hkv, rows, seed=tokens + history)
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    ours = torch.full((tokens, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_tree_attention", ptr(qkv), q_ld, ptr(kc), ptr(vc), rows, tokens, hq, hkv, ptr(kv_len), 0, None, None, 0,
           window, 1, ptr(ours), hq * 128)
    q = qkv[:, : hq * 128].contiguous()
    theirs = torch.full((tokens, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert r.refk_mha_fwd_kvcache(tokens, kv_total, hq, hkv, ptr(q), ptr(kc), ptr(vc), None, None, 0, ptr(theirs), None,
                                  window) == 0
    assert torch.isfinite(theirs.float()).all() and torch.isfinite(ours.float()).all()
    print("library vs reference %.4f" % max_rel(ours, theirs))
    assert max_rel(ours, theirs) <= REL_TOL


# ------------------------------------------------------------------ InfLLM-v2: stage-1 scores, block-sparse attention
def structured_keys(budget, kvd, seed):
    g = torch.Generator().manual_seed(seed)
    base = torch.cumsum(torch.randn(budget // 64 + 1, kvd, generator=g), dim=0) * 0.5
    return (base.repeat_interleave(64, dim=0)[:budget] + torch.randn(budget, kvd, generator=g)).to(torch.bfloat16)


def run_stage1(c, r, qkv, q_ld, kc, T, L, lse, hq, hkv, budget):
    """(library scores [hkv, T, n1], reference scores [hkv, T, n1]) on the same compressed keys."""
    kvd = hkv * 128
    score_ld = (budget // 16 + 127) // 128 * 128
    bm_words = (budget // 64 + 63) // 64
    c1 = torch.zeros(budget // 16 + 16, kvd, dtype=torch.bfloat16, device="cuda")
    c2 = torch.zeros(budget // 64 + 16, kvd, dtype=torch.bfloat16, device="cuda")
    scores = torch.zeros(hkv, T, score_ld, dtype=torch.bfloat16, device="cuda")
    bm = torch.zeros(hkv, T, bm_words, dtype=torch.int64, device="cuda")
    kv_len = dev(torch.tensor([L], dtype=torch.int32))
    c.call("cpmcu_sparse_select", ptr(qkv), q_ld, T, hq, hkv, ptr(kc), budget, ptr(kv_len), 0, 1, 32, 64, 256, int(lse),
           ptr(c1), ptr(c2), ptr(scores), score_ld, ptr(bm), bm_words)
    n1, n2 = max((L - 16) // 16, 0), max((L - 64) // 64, 0)
    q = qkv[:, : hq * 128].contiguous()
    q_round = (T * 16 + 127) // 128 * 128 // 16
    k_round = (n1 + 127) // 128 * 128
    theirs = torch.zeros(hkv, q_round, k_round, dtype=torch.bfloat16, device="cuda")
    qr, kr = ctypes.c_int(0), ctypes.c_int(0)
    assert r.refk_mha_fwd_stage1(T, n1, n2 if lse else n1, hq, hkv, ptr(q), ptr(c1), ptr(c2 if lse else c1), ptr(theirs),
                                 ctypes.byref(qr), ctypes.byref(kr)) == 0
    assert (qr.value, kr.value) == (q_round, k_round)
    return scores[:, :, :n1].float(), theirs[:, :T, :n1].float()


def assert_scores_close(a, b, what):
    assert torch.isfinite(b).all()
    err = (a - b).abs()
    print("%s: max abs diff %.3e, max score %.3e" % (what, float(err.max()), float(b.max())))
    # scores are sums of 16 softmax probabilities stored in bf16: one bf16 step each plus the exp/sum order
    assert bool((err <= REL_TOL * b.abs() + 1e-3 * float(b.max())).all()), float(err.max())


STAGE1_CASES = [
    # T, L, apply_compress_lse
    (60, 32768, True), (60, 32768, False), (12, 3000, True), (7, 9001, False), (1, 20000, True),
]


@pytest.mark.parametrize("T,L,lse", STAGE1_CASES)
def test_stage1_scores_match_reference_one_kv_head(T, L, lse):
    """Stage-1 block scores: the library's scoring kernels against mha_fwd_stage1 on the same compressed keys
    (the library's own, whose means are pinned against the reference's pooling kernel elsewhere), with one KV
    head of 16 query heads: the layout in which the reference kernel's query addressing is the plain one."""
    c, r = C(), ref_flash()
    hq, hkv = 16, 1
    budget = (L + T + 127) // 128 * 128
    g = torch.Generator().manual_seed(L + T)
    q_ld = (hq + 2 * hkv) * 128
    qkv = dev(torch.randn(T, q_ld, generator=g).to(torch.bfloat16))
    kc = dev(structured_keys(budget, hkv * 128, L))
    ours, theirs = run_stage1(c, r, qkv, q_ld, kc, T, L, lse, hq, hkv, budget)
    assert_scores_close(ours, theirs, "stage-1 scores (16 q heads, 1 kv head)")


def reference_stage1_view_of_q(qkv, T, hq, hkv):
    """With more than one KV head the reference's stage-1 kernel does not read the 16 query heads of KV head g of
    token t for score row (g, t).  It runs 64-row tiles over a query tensor whose row stride was set for 16-row
    tiles (flash_api.hpp:225-226 `seqlen_q *= 16; num_heads /= 16`, tile strides `q_row_stride * kBlockM,
    q_head_stride * kBlockM` at flash_fwd_kernel.h:1834-1836, kBlockM = 64 at flash_fwd_launch_template.h:204): tile
    (m, g) covers ALL 32 heads of the two tokens 4m + 2g and 4m + 2g + 1, and its four 16-row groups become the
    score rows 4m .. 4m + 3 of KV head g.  Score row (g, t) therefore holds token 4(t/4) + 2g + (t mod 4)/2, query
    heads 16(t mod 2) .. 16(t mod 2) + 15, against the keys of KV head g.  This returns the query tensor for which
    the plain GQA computation gives exactly those rows."""
    assert hq == 32 and hkv == 2 and T % 4 == 0
    q = qkv[:, : hq * 128].view(T, hq, 128)
    out = qkv.clone()
    view = out[:, : hq * 128].view(T, hq, 128)
    for t in range(T):
        for g in range(hkv):
            src_tok = 4 * (t // 4) + 2 * g + (t % 4) // 2
            src_head = 16 * (t % 2)
            view[t, 16 * g:16 * g + 16] = q[src_tok, src_head:src_head + 16]
    return out


@pytest.mark.parametrize("T,L,lse", [(60, 32768, True), (60, 32768, False), (12, 3000, True), (8, 9001, False)])
def test_stage1_scores_match_reference_under_its_query_addressing(T, L, lse):
    """Two KV heads (the 8B shape): the reference's scores equal the library's scores of the re-addressed query
    tensor described in reference_stage1_view_of_q, i.e. the arithmetic agrees and the reference's own row
    addressing is what differs from plain GQA.  The library keeps the plain addressing."""
    c, r = C(), ref_flash()
    hq, hkv = 32, 2
    budget = (L + T + 127) // 128 * 128
    g = torch.Generator().manual_seed(L + T)
    q_ld = (hq + 2 * hkv) * 128
    qkv = dev(torch.randn(T, q_ld, generator=g).to(torch.bfloat16))
    kc = dev(structured_keys(budget, hkv * 128, L))
    plain, theirs = run_stage1(c, r, qkv, q_ld, kc, T, L, lse, hq, hkv, budget)
    viewed, theirs2 = run_stage1(c, r, reference_stage1_view_of_q(qkv, T, hq, hkv), q_ld, kc, T, L, lse, hq, hkv, budget)
    assert_scores_close(viewed, theirs, "stage-1 scores (library on the reference's view of q vs reference)")
    # rows whose source is the plain one agree without any re-addressing: (g=0, t=4m) and (g=1, t=4m+3)
    assert_scores_close(plain[0, 0::4], theirs[0, 0::4], "rows (kv head 0, t = 4m)")
    assert_scores_close(plain[1, 3::4], theirs[1, 3::4], "rows (kv head 1, t = 4m + 3)")


SPARSE_ATTN_CASES = [
    # T, L, window blocks, top-k, tree mask
    (60, 9000, 32, 64, True), (60, 32768, 32, 64, True), (12, 3000, 4, 6, True), (1, 4100, 3, 8, False),
]


@pytest.mark.parametrize("T,L,window,top,tree", SPARSE_ATTN_CASES)
def test_block_sparse_attention_matches_reference(T, L, window, top, tree):
    """The head-group block-sparse call with block masks the library selected (their integer derivation is
    pinned against the reference's pooling / top-k kernels elsewhere), tree mask on the last T keys."""
    c, r = C(), ref_flash()
    hq, hkv = 32, 2
    kvd = hkv * 128
    kv_total = L + T
    padded = (kv_total + 127) // 128 * 128
    budget = padded + 128
    g = torch.Generator().manual_seed(3 * L + T)
    q_ld = (hq + 2 * hkv) * 128
    qkv = dev(torch.randn(T, q_ld, generator=g).to(torch.bfloat16))
    kc = dev(structured_keys(budget, kvd, L + 1))
    vc = dev(torch.randn(budget, kvd, generator=g).to(torch.bfloat16))
    score_ld = (budget // 16 + 127) // 128 * 128
    bm_words = (padded // 64 + 63) // 64            # the reference's words per row for seqlen_k = padded
    bm = torch.zeros(hkv, T, bm_words, dtype=torch.int64, device="cuda")
    kv_len_sel = dev(torch.tensor([L], dtype=torch.int32))
    c.call("cpmcu_sparse_select", ptr(qkv), q_ld, T, hq, hkv, ptr(kc), budget, ptr(kv_len_sel), 0, 1, window, top, 256, 1,
           None, None, None, score_ld, ptr(bm), bm_words)
    assert not bool((bm == -1).all())               # selection is active
    masks = None
    if tree:
        masks, _ = random_tree_masks(T, np.random.default_rng(L))
    mask_t = u64(masks) if masks is not None else None
    kv_len = dev(torch.tensor([kv_total], dtype=torch.int32))
    ours = torch.full((T, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    c.call("cpmcu_sparse_attention", ptr(qkv), q_ld, ptr(kc), ptr(vc), budget, T, hq, hkv, ptr(kv_len), 0, ptr(mask_t),
           T if tree else 0, ptr(bm), bm_words, window, 4, ptr(ours), hq * 128)
    q = qkv[:, : hq * 128].contiguous()
    theirs = torch.full((T, hq * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert r.refk_mha_fwd_kvcache(T, padded, hq, hkv, ptr(q), ptr(kc), ptr(vc), ptr(kv_len), ptr(mask_t),
                                  T if tree else 0, ptr(theirs), ptr(bm), window) == 0
    assert torch.isfinite(theirs.float()).all() and torch.isfinite(ours.float()).all()
    print("library vs reference %.4f" % max_rel(ours, theirs))
    assert max_rel(ours, theirs) <= REL_TOL
