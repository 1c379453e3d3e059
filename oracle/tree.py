"""CPU oracle for the integer stages of the speculative step (numpy).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the
cpu_baseline / reference arms of bench.py.  Nothing in the product imports it.

PARITY PINNED against the reference's own device kernels: the reference ships no
golden vectors for this path and has no CPU implementation, but its kernels for
these stages compile from its own files (oracle/ref_kernels.cu, oracle/build_ref.py).
Their outputs on a B200 are committed as tests/golden/ref_kernels_golden.json
(generator: tests/golden/make_ref_golden.py) and tests/test_ref_golden_cpu.py holds
this file to them bit for bit: log-softmax + top-k + frontier bookkeeping + final
selection + tree build (with and without the FR-Spec remap), verify, emitted tokens.

bf16 values are carried as numpy float32 arrays whose values are exactly
representable in bf16; `bf16_round` performs round-to-nearest-even.
"""
import numpy as np


def bf16_round(x):
    """Round float32 values to the nearest bf16 (ties to even); returns float32."""
    a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    u = a.view(np.uint32).astype(np.uint64)
    nan = np.isnan(a)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    out[nan] = np.nan
    return out.reshape(np.shape(x))


def topk_desc(vals, k):
    """Top-k by value descending, ties to the lower index.

    Follows the comparator of the reference's bitonic top-k
    (src/model/topk.cuh:17,26,37: `v1 > v2 || (v1 == v2 && pos < pos2)`), and the
    repeated 32-wide passes for k > 32 (topk.cuh:273-286), which together yield a
    stable descending sort truncated to k.
    """
    vals = np.asarray(vals, dtype=np.float32)
    order = np.lexsort((np.arange(vals.size), -vals.astype(np.float64)))
    idx = order[:k].astype(np.int32)
    return vals[idx], idx


def log_softmax_bf16(logits_row):
    """bf16(x - max - log(sum exp(x - max))) over bf16 logits with fp32 math.

    Follows log_softmax_kernel (src/model/eagle.cuh:29-89): max and sum in fp32,
    result stored in the model dtype.  The summation order differs (the reference
    uses a 1024-thread tree under fast-math), so values within one fp32 ulp of a
    bf16 rounding boundary may round differently.
    """
    x = np.asarray(logits_row, dtype=np.float32)
    mx = x.max()
    s = np.exp((x - mx).astype(np.float32)).astype(np.float32).sum(dtype=np.float32)
    return bf16_round(x - mx - np.float32(np.log(s)))


class DraftTree:
    """Frontier expansion and tree construction of one draft() call.

    Restates EagleImpl::draft / MiniCPM4EagleImpl::draft bookkeeping
    (src/model/eagle.cuh:451-495, src/model/minicpm4/minicpm4_eagle.cuh:319-393)
    and build_dynamic_tree_kernel (src/model/eagle.cuh:188-218).
    """

    def __init__(self, k, num_iter, tree_size, token_id_remap=None):
        assert tree_size <= 64
        self.k, self.num_iter, self.tree_size = k, num_iter, tree_size
        self.total_tried = k + k * k * (num_iter - 1)
        self.remap = None if token_id_remap is None else np.asarray(token_id_remap, dtype=np.int32)
        self.tried_val = np.zeros(self.total_tried, dtype=np.float32)
        self.tried_pos = np.zeros(self.total_tried, dtype=np.int32)
        self.tried_parent = np.zeros(max(k * (num_iter - 1), 1), dtype=np.int32)
        self.fr_score = np.zeros(k, dtype=np.float32)
        self.fr_id = np.zeros(k, dtype=np.int32)
        self.fr_mask = np.zeros(k, dtype=np.uint64)
        self.fr_parent_row = np.zeros(k, dtype=np.int32)  # row of the level's hidden states each frontier node copies

    def _remap(self, ids):
        ids = np.asarray(ids, dtype=np.int32)
        return ids if self.remap is None else self.remap[ids]

    def level0(self, logprob_row):
        """d = 0 (eagle.cuh:451-462): seed the frontier from one row's top-k."""
        k = self.k
        v, j = topk_desc(logprob_row, k)
        self.tried_val[:k] = v
        self.tried_pos[:k] = j
        self.fr_id = self._remap(j).astype(np.int32)
        self.fr_score = v.copy()
        self.fr_mask = (np.uint64(1) << np.arange(k, dtype=np.uint64)).astype(np.uint64)
        self.fr_parent_row = np.zeros(k, dtype=np.int32)

    def level(self, d, logprob_rows):
        """d >= 1 (eagle.cuh:463-489): cumulative scores, history, next frontier."""
        k = self.k
        kk = k * k
        vals = np.zeros((k, k), dtype=np.float32)
        pos = np.zeros((k, k), dtype=np.int32)
        for r in range(k):
            v, j = topk_desc(logprob_rows[r], k)
            vals[r] = bf16_round(v + self.fr_score[r])  # cumsum_kernel: bf16 add (eagle.cuh:103-106)
            pos[r] = j
        base = k + (d - 1) * kk
        self.tried_val[base:base + kk] = vals.reshape(-1)
        self.tried_pos[base:base + kk] = pos.reshape(-1)
        sv, si = topk_desc(vals.reshape(-1), k)
        self.tried_parent[(d - 1) * k:(d - 1) * k + k] = si + base          # set_parent_kernel
        old = self.fr_mask.copy()
        self.fr_mask = np.array([old[si[i] // k] | (np.uint64(1) << np.uint64(k * d + i)) for i in range(k)],
                                dtype=np.uint64)                              # update_tree_kernel
        self.fr_parent_row = (si // k).astype(np.int32)                       # remap_hidden_kernel
        self.fr_id = self._remap(pos.reshape(-1)[si]).astype(np.int32)       # remap_id_kernel
        self.fr_score = sv.copy()

    def finalize(self, cache_length, root_id=0):
        """Final top-(tree_size-1) and build_dynamic_tree_kernel (eagle.cuh:188-218)."""
        k, T = self.k, self.tree_size
        kk = k * k
        _, sel = topk_desc(self.tried_val[:self.total_tried], T - 1)
        rank = {int(p): i + 1 for i, p in enumerate(sel)}
        ids = np.zeros(T, dtype=np.int32)
        pos = np.zeros(T, dtype=np.int32)
        mask = np.zeros(T, dtype=np.uint64)
        parent = np.zeros(T, dtype=np.int32)
        ids[0] = root_id
        pos[0] = cache_length
        mask[0] = 1
        for i in range(1, T):
            p = int(sel[i - 1])
            depth = 1 if p < k else (p - k) // kk + 2
            pos[i] = cache_length + depth
            if p < k:
                q = -1
            elif p - k < kk:
                q = (p - k) // k
            else:
                q = int(self.tried_parent[(p - k - kk) // k])
            par = 0 if q == -1 else rank[q]
            parent[i] = par
            mask[i] = (np.uint64(1) << np.uint64(i)) | mask[par]
            ids[i] = self._remap(self.tried_pos[p])
        return ids, pos, mask, parent, sel.astype(np.int32)


def verify(tree_ids, gt, position_ids, cache_length, attn_mask, tree_parent):
    """Greedy acceptance: restates verify_kernel (src/model/tree_drafter.cuh:5-46).

    Returns (accept_len, best_node, path) with path[d] = node at depth d on the
    accepted root path.
    """
    T = len(tree_ids)
    correct = 1
    for i in range(1, T):
        if int(tree_ids[i]) == int(gt[int(tree_parent[i])]):
            correct |= 1 << i
    best_len, best = 1, 0
    for i in range(T):
        m = int(attn_mask[i])
        if (correct & m) == m:
            depth = int(position_ids[i]) - int(cache_length) + 1
            if depth > best_len:
                best_len, best = depth, i
    path = [0] * best_len
    m = int(attn_mask[best])
    for i in range(T):
        if (m >> i) & 1:
            path[int(position_ids[i]) - int(cache_length)] = i
    return best_len, best, path


def compact_rows(cache, cache_length, path):
    """KV fix-up: row L+i <- row L+path[i] (fix_kvcache_kernel_1/2, tree_drafter.cuh:48-77)."""
    L = int(cache_length)
    tmp = [cache[L + p].copy() for p in path]
    for i, row in enumerate(tmp):
        cache[L + i] = row
    return cache


def emitted_tokens(gt, path):
    """pred[i] = gt[path[i]] (fix_kvcache_kernel_2, tree_drafter.cuh:73-75)."""
    return [int(gt[p]) for p in path]
