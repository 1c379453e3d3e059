"""Golden vectors from the reference project's OWN device kernels.

oracle/_ref/libcpmcu_ref_kernels.so (built by oracle/build_ref.py from the reference checkout) is run
on a GPU over deterministic inputs; the outputs go to tests/golden/ref_kernels_golden.json.  The CPU
tests pin the oracle against this file and the GPU tests pin the library against it, so both are
checked against the reference itself and not only against each other.

    python tests/golden/make_ref_golden.py [output.json]      # needs a CUDA device and the library

Inputs are regenerated from (seed, shape) by `det_uniform`, a counter-based splitmix64 generator
written out here, so they do not depend on any library's random streams.
"""
import ctypes
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libcpmcu_ref_kernels.so")


# ------------------------------------------------------------------ deterministic inputs
def det_u64(seed, n):
    """splitmix64 of the counters seed * 2^32 + i."""
    with np.errstate(over="ignore"):
        z = (np.uint64(seed) << np.uint64(32)) + np.arange(n, dtype=np.uint64) + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def det_uniform(seed, shape):
    """float64 in [0, 1) with 24 random bits."""
    n = int(np.prod(shape))
    return ((det_u64(seed, n) >> np.uint64(40)).astype(np.float64) / float(1 << 24)).reshape(shape)


def det_ints(seed, n, hi):
    return (det_u64(seed, n) % np.uint64(hi)).astype(np.int64)


def to_bf16(x):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16)


def bits(t):
    """bf16 tensor -> list of its 16-bit patterns (as signed ints)."""
    return t.contiguous().view(torch.int16).cpu().flatten().tolist()


def tree_logits(seed, V, k, num_iter, coarse):
    """[1 + (num_iter-1)*k, V] bf16: a bell-shaped spread of about +-9 so that log-probabilities differ
    widely; `coarse` puts the values on a grid of 0.5 (many exact ties)."""
    rows = 1 + (num_iter - 1) * k
    u = det_uniform(seed, (3, rows, V))
    x = (u[0] + u[1] + u[2] - 1.5) * 6.0
    if coarse:
        x = np.round(x * 2) / 2
    return to_bf16(x)


def fr_remap(seed, V, full_vocab):
    """V distinct full-vocabulary ids, ascending (as a frequency-ranked subset is stored)."""
    order = np.argsort(det_u64(seed, full_vocab), kind="stable")[:V]
    return np.sort(order).astype(np.int32)


def verify_inputs(seed, T, L):
    r = det_u64(seed, 8 * T)
    parent, masks, depth = [0] * T, [1] * T, [1] * T
    for i in range(1, T):
        j = 0
        while True:
            p = int(r[(8 * i + j) % len(r)] % np.uint64(i))
            j += 1
            if depth[p] < 7 or j > 6:
                break
        if depth[p] >= 7:
            p = 0
        parent[i], depth[i], masks[i] = p, depth[p] + 1, masks[p] | (1 << i)
    pos = [L + d - 1 for d in depth]
    ids = det_ints(seed + 1000, T, 50).tolist()
    gt = det_ints(seed + 2000, T, 50).tolist()
    coin = det_uniform(seed + 3000, (T,))
    for i in range(1, T):
        if coin[i] < 0.6:
            ids[i] = gt[parent[i]]
    return ids, gt, pos, masks, parent


def cache_pattern(j, rows, dim):
    """Cache j: every element of row r holds the 16-bit pattern (131 * j + 7 * r + column) mod 30000."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(dim, dtype=np.int64)[None, :]
    return torch.from_numpy(((131 * j + 7 * r + c) % 30000).astype(np.int16))


def select_scores(seed, hkv, T, k_round, n_valid):
    """Stage-1 scores [hkv][T][k_round] bf16: positive, a few hundred distinct values (ties occur), zero
    beyond n_valid as the stage-1 kernel leaves them."""
    u = det_uniform(seed, (hkv, T, k_round))
    x = np.round(u * u * 400) / 1024.0
    x[:, :, n_valid:] = 0.0
    return to_bf16(x)


def compress_keys(seed, L, dim):
    return to_bf16((det_uniform(seed, (L, dim)) - 0.5) * 4.0)


TREE_CASES = [
    # seed, V, k, num_iter, T, coarse, FR-Spec full vocabulary (0 = none)
    (11, 4096, 4, 4, 16, False, 0),
    (12, 8192, 10, 6, 60, False, 0),
    (13, 5000, 8, 3, 64, True, 0),
    (14, 2048, 10, 6, 60, True, 6000),
    (15, 3000, 10, 6, 32, False, 0),
]
VERIFY_CASES = [(21, 16, 40), (22, 60, 77), (23, 64, 300), (24, 2, 5), (25, 60, 1000), (26, 60, 12)]
SELECT_CASES = [
    # seed, hkv, T, cache_len, top, sink, window
    (31, 2, 12, 4200, 6, 1, 4),
    (32, 2, 60, 8000, 16, 1, 8),
    (33, 1, 7, 5000, 64, 2, 2),
    (34, 2, 9, 70000, 12, 1, 4),     # more than 1024 blocks: the multi-block top-k path
    (35, 2, 5, 33000, 64, 1, 32),    # the long-context setting (top 64, window 32 blocks)
]
COMPRESS_CASES = [(41, 300, 256), (42, 1000, 128)]


def dptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "ref_kernels_golden.json")
    lib = ctypes.CDLL(REF_LIB)
    dev = "cuda"
    out = {"trees": [], "verify": [], "select": [], "compress": []}

    for seed, V, k, num_iter, T, coarse, full in TREE_CASES:
        L = 1234
        logits = tree_logits(seed, V, k, num_iter, coarse).to(dev)
        remap = torch.from_numpy(fr_remap(seed, V, full)).to(dev) if full else None
        tt = k + k * k * (num_iter - 1)
        ids = torch.zeros(64, dtype=torch.int32, device=dev)
        pos = torch.zeros(64, dtype=torch.int32, device=dev)
        mask = torch.zeros(64, dtype=torch.int64, device=dev)
        par = torch.zeros(64, dtype=torch.int32, device=dev)
        tv = torch.zeros(tt + 64, dtype=torch.bfloat16, device=dev)
        tp = torch.zeros(tt + 64, dtype=torch.int32, device=dev)
        tpar = torch.zeros(k * num_iter + 64, dtype=torch.int32, device=dev)
        cl = torch.tensor([L], dtype=torch.int32, device=dev)
        rc = lib.refk_draft_tree_from_logits(dptr(logits), V, k, num_iter, T, dptr(remap), dptr(cl), dptr(ids),
                                             dptr(pos), dptr(mask), dptr(par), dptr(tv), dptr(tp), dptr(tpar))
        assert rc == 0, rc
        out["trees"].append({
            "seed": seed, "V": V, "k": k, "num_iter": num_iter, "T": T, "coarse": coarse, "full_vocab": full,
            "cache_length": L, "ids": ids[1:T].cpu().tolist(), "pos": pos[:T].cpu().tolist(),
            "mask": [int(m) for m in mask[:T].cpu().numpy().view(np.uint64)], "parent": par[1:T].cpu().tolist(),
            "tried_val_bits": bits(tv[:tt]), "tried_pos": tp[:tt].cpu().tolist(),
            "tried_parent": tpar[:k * (num_iter - 1)].cpu().tolist()})

    for seed, T, L in VERIFY_CASES:
        ids, gt, pos, masks, parent = verify_inputs(seed, T, L)
        num_caches, dim, rows = 4, 256, L + T + 8
        caches = [cache_pattern(j, rows, dim).to(dev) for j in range(num_caches)]
        before = [c.clone() for c in caches]
        ptrs = torch.tensor([c.data_ptr() for c in caches], dtype=torch.int64, device=dev)
        pred = torch.tensor(ids + [0] * (64 - T), dtype=torch.int32, device=dev)
        gt_t = torch.tensor(gt + [0] * (64 - T), dtype=torch.int32, device=dev)
        pos_t = torch.tensor(pos + [0] * (64 - T), dtype=torch.int32, device=dev)
        mask_t = torch.from_numpy(np.array(masks + [0] * (64 - T), dtype=np.uint64).view(np.int64)).to(dev)
        par_t = torch.tensor(parent + [0] * (64 - T), dtype=torch.int32, device=dev)
        cl = torch.tensor([L], dtype=torch.int32, device=dev)
        result = torch.zeros(2 + 64, dtype=torch.int32, device=dev)
        rc = lib.refk_verify_and_compact(T, dptr(pred), dptr(gt_t), dptr(pos_t), dptr(cl), dptr(mask_t), dptr(par_t),
                                         dptr(ptrs), num_caches, dim, 64, dptr(result))
        assert rc == 0, rc
        res = result.cpu().tolist()
        n = res[0]
        path = res[2:2 + n]
        # rows L .. L+n-1 of every cache must be whole copies of rows L + path[i]; all other rows untouched
        for j in range(num_caches):
            want = before[j].clone()
            for i in range(n):
                want[L + i] = before[j][L + path[i]]
            assert torch.equal(caches[j], want)
        out["verify"].append({"seed": seed, "T": T, "L": L, "n": n, "best": res[1], "path": path,
                              "tokens": pred[:n].cpu().tolist()})

    for seed, hkv, T, cache_len, top, sink, window in SELECT_CASES:
        n1 = max((cache_len - 16) // 16, 0)
        k_round = (n1 + 127) // 128 * 128
        scores = select_scores(seed, hkv, T, k_round, n1).to(dev)
        out_len = (cache_len + 63) // 64
        padded = (cache_len + T + 127) // 128 * 128
        words = ((padded + 63) // 64 + 63) // 64
        pool = torch.zeros(hkv, T, out_len, dtype=torch.bfloat16, device=dev)
        bm = torch.zeros(hkv * T, words, dtype=torch.int64, device=dev)
        rc = lib.refk_select_from_scores(dptr(scores), hkv, T, T, k_round, cache_len, sink, window, top, padded,
                                         dptr(pool), dptr(bm))
        assert rc == 0, rc
        out["select"].append({"seed": seed, "hkv": hkv, "T": T, "cache_len": cache_len, "top": top, "sink": sink,
                              "window": window, "k_round": k_round, "words": words,
                              "pool_bits": bits(pool) if out_len <= 160 else None,
                              "blockmask": [int(m) for m in bm.cpu().numpy().view(np.uint64).flatten()]})

    for seed, L, dim in COMPRESS_CASES:
        keys = compress_keys(seed, L, dim).to(dev)
        n1, n2 = max((L - 16) // 16, 0), max((L - 64) // 64, 0)
        c1 = torch.zeros(n1, dim, dtype=torch.bfloat16, device=dev)
        c2 = torch.zeros(n2, dim, dtype=torch.bfloat16, device=dev)
        rc = lib.refk_compress(dptr(keys), L, dim, dptr(c1), dptr(c2))
        assert rc == 0, rc
        out["compress"].append({"seed": seed, "L": L, "dim": dim, "c1_bits": bits(c1), "c2_bits": bits(c2)})

    with open(out_path, "w") as f:
        json.dump(out, f)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
