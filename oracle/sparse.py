"""InfLLM-v2 block selection of the MiniCPM4 target (config 5): compressed key caches, stage-1
scoring, max-pooling to 64-token blocks, top-k -> bitmask, and the key visibility the block-sparse
attention kernel derives from it (numpy / PyTorch CPU).

TEST INFRASTRUCTURE ONLY (see oracle/tree.py).  PARITY PINNED for `compress`, `maxpool_blocks` and
`topk_blockmask` against the reference's own kernels (bit-exact against their B200 outputs in
tests/golden/ref_kernels_golden.json, see tests/test_ref_golden_cpu.py).  UNPINNED for `stage1_scores`
and `block_visibility`: those restate the reference's attention code, which needs the un-vendored
CUTLASS tree to compile, from the sources cited in each function.
"""
import math

import numpy as np
import torch

from .tree import bf16_round

BLOCK = 64       # tokens per selectable block (maxpooling_func block_size, flash kBlockN of the head-level kernel)
C1_STRIDE = 16   # MiniCPM4KVCache::c1_stride, windows of 32 tokens
C2_STRIDE = 64   # MiniCPM4KVCache::c2_stride, windows of 128 tokens


class SparseConfig:
    """Arguments of init_minicpm4_model (src/entry.cu:138-158)."""

    def __init__(self, sink_window_size=1, block_window_size=32, sparse_topk_k=64, sparse_switch=8192,
                 apply_compress_lse=True):
        self.sink_window_size, self.block_window_size = sink_window_size, block_window_size
        self.sparse_topk_k, self.sparse_switch = sparse_topk_k, sparse_switch
        self.apply_compress_lse = apply_compress_lse


def _rnd(x):
    return torch.from_numpy(bf16_round(x.numpy().astype(np.float32)))


def compressed_len(next_kv_length, stride):
    """MiniCPM4KVCache::compress (src/model/minicpm4/minicpm4_kvcache.cuh:243-254)."""
    return max((next_kv_length - stride) // stride, 0)


def compress(k_cache, next_kv_length, stride):
    """Mean of 2*stride consecutive key rows every `stride` rows, fp32 sum, stored in the model dtype
    (meanpooling_16_kernel / meanpooling_64_kernel, minicpm4_kvcache.cuh:6-62).  k_cache: [rows, dim]."""
    n = compressed_len(next_kv_length, stride)
    out = torch.zeros(n, k_cache.shape[1])
    for i in range(n):
        out[i] = k_cache[i * stride: i * stride + 2 * stride].sum(dim=0) / float(2 * stride)
    return _rnd(out)


def sparse_active(cfg, next_kv_length):
    """minicpm4_attn.cuh:107 / :231."""
    if cfg.apply_compress_lse:
        return compressed_len(next_kv_length, C2_STRIDE) * C2_STRIDE >= cfg.sparse_switch
    return compressed_len(next_kv_length, C1_STRIDE) * C1_STRIDE >= cfg.sparse_switch


def stage1_scores(q, c1, c_lse, hq, hkv, d):
    """mha_fwd_stage1 (flash_api.hpp:204-290; flash_fwd_kernel.h:1770-2265): per query head the row max
    and exp-sum over the `c_lse` keys, then exp(s - max) / sum over the c1 keys, summed over the heads of
    a KV group and stored in the model dtype.  Returns [hkv, T, k_round] with zeros beyond len(c1)
    (k_round = len(c1) rounded up to 128)."""
    T = q.shape[0]
    grp = hq // hkv
    n1 = c1.shape[0]
    k_round = (n1 + 127) // 128 * 128
    scale = 1.0 / math.sqrt(d)
    qh = q.view(T, hq, d)
    k1 = c1.view(n1, hkv, d)
    kl = c_lse.view(c_lse.shape[0], hkv, d)
    out = torch.zeros(hkv, T, k_round)
    for g in range(hkv):
        acc = torch.zeros(T, n1)
        for h in range(g * grp, (g + 1) * grp):
            sl = (qh[:, h, :] @ kl[:, g, :].t()) * scale
            m = sl.max(dim=-1, keepdim=True).values
            den = torch.exp(sl - m).sum(dim=-1, keepdim=True)
            s1 = (qh[:, h, :] @ k1[:, g, :].t()) * scale
            acc += torch.exp(s1 - m) / den
        out[g, :, :n1] = acc
    return _rnd(out)


def maxpool_blocks(scores, T, cache_len, init_blocks, local_blocks, kernel_size=5, stride=4, padding=1):
    """maxpooling_kernel (minicpm4_kvcache.cuh:64-108).  scores: [hkv, T, k_round]; returns
    [hkv, T, ceil(cache_len / 64)] with +inf for the first init_blocks blocks and -inf for blocks
    k > q_block - local_blocks, q_block = (t + cache_len) // 64."""
    hkv, _, k_len = scores.shape
    out_len = (cache_len + BLOCK - 1) // BLOCK
    out = torch.zeros(hkv, T, out_len)
    for t in range(T):
        q_block = (t + cache_len) // BLOCK
        for k in range(out_len):
            if k < init_blocks:
                out[:, t, k] = float("inf")
            elif q_block - local_blocks < k:
                out[:, t, k] = float("-inf")
            else:
                start = max(k * stride - padding, 0)
                end = min(k * stride - padding + kernel_size, k_len)
                out[:, t, k] = scores[:, t, start:end].max(dim=-1).values
    return out


def topk_blockmask(pool, top, k_len):
    """TopK::prefill (src/model/topk.cuh:255-288: value descending, lower index first) followed by
    kernel_topk_to_uint64 (minicpm4_kvcache.cuh:110-141).  pool: [hkv, T, out_len]; returns uint64
    [hkv, T, n_words], n_words = ceil(ceil(k_len / 64) / 64)."""
    hkv, T, out_len = pool.shape
    n_words = ((k_len + BLOCK - 1) // BLOCK + 63) // 64
    mask = np.zeros((hkv, T, n_words), dtype=np.uint64)
    vals = pool.numpy()
    for g in range(hkv):
        for t in range(T):
            order = sorted(range(out_len), key=lambda i: (-vals[g, t, i], i))
            for i in order[:top]:
                mask[g, t, i // 64] |= np.uint64(1) << np.uint64(i % 64)
    return mask


def select_blocks(cfg, q, k_cache, next_kv_length, hq, hkv, d, k_len):
    """Everything between the KV append and the attention call of MiniCPM4Attention::prefill / decode
    (minicpm4_attn.cuh:96-166, :226-290).  Returns the uint64 block mask or None when selection is
    not active (dense attention)."""
    if next_kv_length == 0 or not sparse_active(cfg, next_kv_length):
        return None
    c1 = compress(k_cache, next_kv_length, C1_STRIDE)
    c_lse = compress(k_cache, next_kv_length, C2_STRIDE) if cfg.apply_compress_lse else c1
    T = q.shape[0]
    scores = stage1_scores(q, c1, c_lse, hq, hkv, d)
    pool = maxpool_blocks(scores, T, next_kv_length, cfg.sink_window_size, cfg.block_window_size)
    return topk_blockmask(pool, cfg.sparse_topk_k, k_len)


def block_visibility(mask, block_window, tq, kv_total):
    """Keys the block-sparse kernel visits for (kv head, token): blocks b >= k_window_left or with their
    bit set, k_window_left = ceil((t + kv_total - tq) / 64) - block_window
    (src/flash_attn/src/flash_blockmask.h:9-34, :37-96).  Returns bool [hkv, tq, kv_total]."""
    hkv = mask.shape[0]
    vis = torch.zeros(hkv, tq, kv_total, dtype=torch.bool)
    nblk = (kv_total + BLOCK - 1) // BLOCK
    for t in range(tq):
        left = (t + kv_total - tq + BLOCK - 1) // BLOCK - block_window
        for b in range(nblk):
            lo, hi = b * BLOCK, min((b + 1) * BLOCK, kv_total)
            if b >= left:
                vis[:, t, lo:hi] = True
            else:
                for g in range(hkv):
                    if (int(mask[g, t, b // 64]) >> (b % 64)) & 1:
                        vis[g, t, lo:hi] = True
    return vis
