"""CPU tests of the InfLLM-v2 selection oracle (oracle/sparse.py): the integer rules the CUDA kernels are
checked against (lengths of the compressed caches, forced / excluded blocks, tie order, window bound)."""
import numpy as np
import torch

from oracle import sparse as osparse


def test_compressed_lengths_follow_the_reference_formula():
    # MiniCPM4KVCache::compress: len = max((L - stride) / stride, 0)
    assert [osparse.compressed_len(L, 16) for L in (0, 15, 16, 31, 32, 47, 48, 1000)] == [0, 0, 0, 0, 1, 1, 2, 61]
    assert [osparse.compressed_len(L, 64) for L in (0, 64, 127, 128, 8256)] == [0, 0, 0, 1, 128]
    cfg = osparse.SparseConfig(sparse_switch=8192, apply_compress_lse=True)
    assert not osparse.sparse_active(cfg, 8255) and osparse.sparse_active(cfg, 8256)
    cfg = osparse.SparseConfig(sparse_switch=8192, apply_compress_lse=False)
    assert not osparse.sparse_active(cfg, 8207) and osparse.sparse_active(cfg, 8208)


def test_compress_is_a_windowed_mean():
    k = torch.arange(200 * 4, dtype=torch.float32).reshape(200, 4)
    c1 = osparse.compress(k, 200, 16)
    assert c1.shape[0] == 11
    ref = k[32:64].mean(dim=0)
    assert torch.allclose(c1[2], ref.to(torch.bfloat16).float())


def test_maxpool_forces_sink_blocks_and_excludes_the_local_window():
    hkv, T, L = 1, 3, 64 * 10 + 5
    n1 = osparse.compressed_len(L, 16)
    scores = torch.zeros(hkv, T, (n1 + 127) // 128 * 128)
    scores[0, :, :n1] = torch.arange(n1, dtype=torch.float32) / 100.0
    pool = osparse.maxpool_blocks(scores, T, L, init_blocks=2, local_blocks=3)
    assert pool.shape == (1, 3, 11)
    assert torch.isposinf(pool[0, :, :2]).all()
    # q_block = (t + L) // 64 = 10: blocks k > 7 are left to the local window
    assert torch.isneginf(pool[0, :, 8:]).all() and torch.isfinite(pool[0, :, 2:8]).all()
    # block k pools compressed entries 4k - 1 .. 4k + 3
    assert float(pool[0, 0, 5]) == float(scores[0, 0, 19:24].max())


def test_topk_prefers_lower_indices_on_ties_and_counts_bits():
    pool = torch.tensor([[[float("inf"), 0.5, 0.5, 0.5, 0.25, float("-inf")]]])
    m = osparse.topk_blockmask(pool, 3, 6 * 64)
    assert int(m[0, 0, 0]) == 0b000111          # +inf first, then the two lowest-indexed of the tied 0.5s
    m = osparse.topk_blockmask(pool, 64, 6 * 64)
    assert int(m[0, 0, 0]) == 0b111111          # fewer blocks than top-k: all of them


def test_block_visibility_window_bound():
    mask = np.zeros((1, 2, 1), dtype=np.uint64)
    mask[0, 0, 0] = 0b1
    tq, kv_total, window = 2, 64 * 6 + 2, 2
    vis = osparse.block_visibility(mask, window, tq, kv_total)
    # token t: left = ceil((t + kv_total - tq) / 64) - window = 6 - 2 (t = 0) and 7 - 2 (t = 1)
    assert vis[0, 0, :64].all() and not vis[0, 0, 64:256].any() and vis[0, 0, 256:].all()
    assert not vis[0, 1, :320].any() and vis[0, 1, 320:].all()


def test_selection_is_off_before_the_switch():
    cfg = osparse.SparseConfig(sparse_switch=8192)
    q = torch.zeros(1, 2 * 128)
    k = torch.zeros(512, 128)
    assert osparse.select_blocks(cfg, q, k, 300, 2, 1, 128, 301) is None


def test_golden_selection_reproduces():
    """tests/golden/sparse_golden.json (made by tests/golden/make_sparse_golden.py from this oracle)."""
    import importlib.util
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("make_sparse_golden", os.path.join(here, "golden", "make_sparse_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    gold = json.load(open(os.path.join(here, "golden", "sparse_golden.json")))
    for case in gold["selection"]:
        again = mod.selection_case(case["seed"], case["T"], case["hq"], case["hkv"], case["L"], case["top"],
                                   case["sink"], case["window"], case["lse"])
        assert again["mask"] == case["mask"]
        assert abs(again["score_sum"] - case["score_sum"]) <= 1e-6 * abs(case["score_sum"])
        # every row selects min(top, blocks) blocks and the sink blocks among them
        blocks = (case["L"] + 63) // 64
        for head in case["mask"]:
            for row in head:
                assert sum(bin(w).count("1") for w in row) == min(case["top"], blocks)
                assert row[0] & ((1 << case["sink"]) - 1) == (1 << case["sink"]) - 1
