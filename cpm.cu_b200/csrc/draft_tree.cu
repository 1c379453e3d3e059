// EAGLE draft-tree kernels: log-softmax + per-row top-k over the draft
// vocabulary, frontier expansion with cumulative log-probabilities, final
// selection of the tree nodes and construction of positions / parents / packed
// ancestor masks.
//
// Replaces, with identical integer results given identical bf16 inputs:
//   log_softmax_kernel                      src/model/eagle.cuh:29-89
//   bitonic top-k (value desc, index asc)   src/model/topk.cuh:7-42,159-213,273-286
//   add/repeat/init_tree/set_parent/update_tree/cumsum/remap_* kernels
//                                           src/model/eagle.cuh:11-127
//   build_dynamic_tree_kernel               src/model/eagle.cuh:188-218
// The reference runs ~12 tiny launches and three device copies per level plus a
// host round trip for the tree; here a level is one launch and the tree one.
#include <algorithm>

#include "common.cuh"
#include "draft_tree.cuh"

namespace {

constexpr int SEG = 2048;          // vocabulary entries per CTA in the scan kernels
constexpr int SCAN_THREADS = 512;  // 4 entries per thread; 16 warps, so the last CTA takes up to 16 rows in one pass

// Order-preserving key: larger key == earlier in (value desc, index asc) order.
__device__ __forceinline__ uint32_t bf16_orderable(bf16 v) {
    const uint16_t b = __bfloat16_as_ushort(v);
    if ((b & 0x7F80) == 0x7F80 && (b & 0x007F) != 0) return 0;  // NaN sorts last
    return (b & 0x8000) ? static_cast<uint16_t>(~b) : static_cast<uint16_t>(b | 0x8000);
}
__device__ __forceinline__ unsigned long long make_key(bf16 v, int idx) {
    return (static_cast<unsigned long long>(bf16_orderable(v)) << 32) |
           static_cast<unsigned long long>(0xFFFFFFFFu - static_cast<uint32_t>(idx));
}
__device__ __forceinline__ int key_index(unsigned long long k) {
    return static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(k & 0xFFFFFFFFull));
}

// Warp-wide maximum of 64-bit keys as two 32-bit hardware reductions (value half, then the index half
// among the lanes that hold the winning value).
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
    const uint32_t hi = static_cast<uint32_t>(v >> 32), lo = static_cast<uint32_t>(v);
    const uint32_t H = __reduce_max_sync(0xffffffffu, hi);
    const uint32_t L = __reduce_max_sync(0xffffffffu, hi == H ? lo : 0u);
    return (static_cast<unsigned long long>(H) << 32) | L;
}

__device__ __forceinline__ bf16 bf16_from_orderable(uint32_t o) {
    const uint16_t b = (o & 0x8000u) ? static_cast<uint16_t>(o & 0x7FFFu) : static_cast<uint16_t>(~o);
    return __ushort_as_bfloat16(b);
}

// Select the `k` largest of `n` unique 32-bit keys held in shared memory by one warp (the keys are consumed);
// result r (0 = largest) is returned to lane r.  Callers pack (orderable 16-bit value << 16) | (0xFFFF - position)
// with positions that rise with the candidate index among equal values.
__device__ uint32_t warp_select(uint32_t* keys, int n, int k, int lane) {
    uint32_t mine = 0u;
    for (int round = 0; round < k; ++round) {
        uint32_t best = 0u;
        for (int i = lane; i < n; i += 32) best = max(best, keys[i]);
        best = __reduce_max_sync(0xffffffffu, best);
        if (lane == round) mine = best;
        for (int i = lane; i < n; i += 32) {
            if (keys[i] == best) keys[i] = 0u;
        }
        __syncwarp();
    }
    return mine;
}

// One launch per draft level: log-softmax statistics, top-k and frontier expansion.
//
// Every CTA owns one (row, 2048-entry vocabulary segment): it reduces the segment's (max, sum of exp) and extracts
// the segment's k largest LOGITS (written in index order, with the k-th largest value beside the statistics).  The
// CTA that is counted last on the ticket, i.e. after every segment of every row is in global memory, turns the
// candidates into log-probabilities lp = bf16(x - max - log(sum)) (the reference's in-place log_softmax stores the
// model dtype), picks each row's k best by (lp descending, index ascending) and runs the level's bookkeeping.  No
// grid-wide wait: only the last CTA reads what the others wrote.
//
// Exactness of picking by logit first: lp is a non-decreasing function of the logit, but bf16 rounding maps many
// logits to one lp, and among equal lp the reference prefers the LOWER index, which a segment's logit order does not
// know.  An element outside a segment's k best logits can only belong to the row's answer if that segment's own k-th
// candidate still reaches the answer's threshold lp (all k of its candidates compete in the top bucket); the last
// CTA detects that and re-selects such a row exactly from the full logit row.  With 36 segments and k = 10 this needs
// ten of a row's best entries inside one segment; the small vocabularies of the tests take the path routinely.
__global__ void draft_level_kernel(DraftTreeState st, const bf16* __restrict__ logits, int ld, int vocab, int nseg,
                                   float4* __restrict__ stats, unsigned long long* __restrict__ cand,
                                   unsigned* __restrict__ ticket, int level, const int32_t* __restrict__ last_row_ptr,
                                   int group_rows) {
    grid_dependency_sync();
    // last CTA: candidate lists of `group_rows` rows (64-bit (logit, ~index) entries, then 32-bit selection keys)
    extern __shared__ unsigned long long sh_keys[];
    __shared__ float sh_m[SCAN_THREADS / 32];
    __shared__ float sh_s[SCAN_THREADS / 32];
    __shared__ uint32_t wtop[SCAN_THREADS / 32][32];
    __shared__ int s_last;
    const int k = st.k;
    const int rows = (level == 0) ? 1 : k;
    const int row = blockIdx.y, seg = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (level == 0 && last_row_ptr) ? *last_row_ptr : 0;
    {
        const bf16* x = logits + static_cast<size_t>(row + row0) * ld;
        const int begin = seg * SEG;
        const int end = min(begin + SEG, vocab);
        // Inside a segment a 32-bit key orders the logits: (orderable 16-bit value << 16) | (0xFFFF - local index),
        // larger = earlier in (value desc, index asc) order, 0 = no entry.  One compare, one hardware reduction.
        static_assert(SEG <= 65536, "local index must fit 16 bits");
        float v[SEG / SCAN_THREADS];
        uint32_t keys[SEG / SCAN_THREADS];
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < SEG / SCAN_THREADS; ++j) {
            const int local = j * SCAN_THREADS + threadIdx.x;
            const int i = begin + local;
            if (i < end) {
                const bf16 xv = x[i];
                v[j] = __bfloat162float(xv);
                keys[j] = (bf16_orderable(xv) << 16) | static_cast<uint32_t>(0xFFFF - local);
            } else {
                v[j] = -INFINITY;
                keys[j] = 0u;
            }
            m = fmaxf(m, v[j]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) sh_m[warp] = m;
        __syncthreads();
        m = sh_m[0];
#pragma unroll
        for (int w = 1; w < SCAN_THREADS / 32; ++w) m = fmaxf(m, sh_m[w]);
        float sum = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int j = 0; j < SEG / SCAN_THREADS; ++j) sum += expf(v[j] - m);  // exp(-inf) = 0 for padding
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) sh_s[warp] = sum;
        // each warp extracts the k best of its 256 keys (no block-wide barrier per round), then warp 0 merges
        // the 8 x k survivors; k <= 32
        for (int round = 0; round < k; ++round) {
            uint32_t best = 0u;
#pragma unroll
            for (int j = 0; j < SEG / SCAN_THREADS; ++j) best = max(best, keys[j]);
            best = __reduce_max_sync(0xffffffffu, best);
            if (lane == 0) wtop[warp][round] = best;
#pragma unroll
            for (int j = 0; j < SEG / SCAN_THREADS; ++j) {
                if (keys[j] == best) keys[j] = 0u;  // keys are unique (the index is part of the key)
            }
        }
        __syncthreads();
        if (warp == 0) {
            uint32_t mine[SCAN_THREADS / 32];
#pragma unroll
            for (int w = 0; w < SCAN_THREADS / 32; ++w) mine[w] = (lane < k) ? wtop[w][lane] : 0u;
            uint32_t picked = 0u;  // lane r: the segment's r-th largest logit
            for (int round = 0; round < k; ++round) {
                uint32_t best = 0u;
#pragma unroll
                for (int w = 0; w < SCAN_THREADS / 32; ++w) best = max(best, mine[w]);
                best = __reduce_max_sync(0xffffffffu, best);
                if (lane == round) picked = best;
#pragma unroll
                for (int w = 0; w < SCAN_THREADS / 32; ++w) {
                    if (mine[w] == best) mine[w] = 0u;
                }
            }
            // write the k candidates in index order (empty entries last): among equal lp the position in the row's
            // list, segment after segment, then rises with the vocabulary index
            const uint32_t lidx = (lane < k && picked) ? (0xFFFFu - (picked & 0xFFFFu)) : 0x10000u + lane;
            int rank = 0;
            for (int o = 0; o < k; ++o) rank += (__shfl_sync(0xffffffffu, lidx, o) < lidx) ? 1 : 0;
            if (lane < k) {
                const uint32_t idx = static_cast<uint32_t>(begin) + (lidx & 0xFFFFu);
                // (orderable logit << 32) | ~index, the row-wide form of make_key(); 0 = no entry
                cand[(static_cast<size_t>(row) * nseg + seg) * k + rank] =
                    picked ? ((static_cast<unsigned long long>(picked >> 16) << 32) | (0xFFFFFFFFu - idx)) : 0ull;
            }
            const uint32_t kth = __shfl_sync(0xffffffffu, picked, k - 1);  // 0 when the segment has fewer than k entries
            if (lane == 0) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < SCAN_THREADS / 32; ++w) t += sh_s[w];
                stats[static_cast<size_t>(row) * nseg + seg] = make_float4(m, t, __uint_as_float(kth >> 16), 0.f);
            }
        }
    }
    // ---- ticket: the last CTA to get here sees every CTA's statistics and candidates
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = (atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1) ? 1 : 0;
        __threadfence();
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *ticket = 0u;  // ready for the next launch

    __shared__ bf16 s_val[32 * 32];
    __shared__ int s_pos[32 * 32];
    __shared__ uint32_t s_ckey[32 * 32];
    __shared__ int s_sel[32];
    __shared__ uint64_t s_oldmask[32];
    const int per_row = nseg * k;
    constexpr int NW = SCAN_THREADS / 32;
    for (int g0 = 0; g0 < rows; g0 += group_rows) {
        const int gn = min(group_rows, rows - g0);
        uint32_t* sel_keys = reinterpret_cast<uint32_t*>(sh_keys + static_cast<size_t>(group_rows) * per_row);
        // one coalesced pass brings the group's candidate lists on chip
        for (int i = threadIdx.x; i < gn * per_row; i += SCAN_THREADS) sh_keys[i] = cand[static_cast<size_t>(g0) * per_row + i];
        __syncthreads();
        for (int rr = warp; rr < gn; rr += NW) {
            const int r = g0 + rr;
            unsigned long long* mycand = sh_keys + static_cast<size_t>(rr) * per_row;
            uint32_t* mysel = sel_keys + static_cast<size_t>(rr) * per_row;
            // row-wide log-sum-exp offset from the segment partials, fixed reduction order within the warp
            const float4* rst = stats + static_cast<size_t>(r) * nseg;
            float mx = -INFINITY;
            for (int sg = lane; sg < nseg; sg += 32) mx = fmaxf(mx, rst[sg].x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float sum = 0.f;
            for (int sg = lane; sg < nseg; sg += 32) {
                const float4 q = rst[sg];
                sum += q.y * expf(q.x - mx);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float ls = logf(sum);
            // selection keys: (orderable lp << 16) | (0xFFFF - position in the list)
            for (int i = lane; i < per_row; i += 32) {
                const unsigned long long c = mycand[i];
                uint32_t key = 0u;
                if (c) {
                    const bf16 lp = __float2bfloat16(__bfloat162float(bf16_from_orderable(static_cast<uint32_t>(c >> 32))) - mx - ls);
                    key = (bf16_orderable(lp) << 16) | static_cast<uint32_t>(0xFFFF - i);
                }
                mysel[i] = key;
            }
            __syncwarp();
            uint32_t got = warp_select(mysel, per_row, k, lane);
            // threshold = the row's k-th best lp.  A segment whose own k-th candidate still reaches it may hide further
            // entries of the threshold bucket (with lower indices): re-select such a row exactly.
            const uint32_t kth = __shfl_sync(0xffffffffu, got, k - 1);
            const uint32_t tau = kth >> 16;
            bool saturated = false;
            for (int sg = lane; sg < nseg; sg += 32) {
                const uint32_t xk = __float_as_uint(rst[sg].z);
                if (kth != 0u && xk != 0u) {
                    const bf16 lp = __float2bfloat16(__bfloat162float(bf16_from_orderable(xk)) - mx - ls);
                    if (bf16_orderable(lp) >= tau) saturated = true;
                }
            }
            bf16 my_lp = __float2bfloat16(0.f);
            int my_idx = 0;
            if (__any_sync(0xffffffffu, saturated)) {
                // k rounds of "largest key below the previous pick" over the whole logit row
                const bf16* x = logits + static_cast<size_t>(r + row0) * ld;
                unsigned long long prev = ~0ull, mine64 = 0ull;
                for (int round = 0; round < k; ++round) {
                    unsigned long long best = 0ull;
                    for (int i = lane; i < vocab; i += 32) {
                        const bf16 lp = __float2bfloat16(__bfloat162float(x[i]) - mx - ls);
                        const unsigned long long key = make_key(lp, i);
                        if (key < prev && key > best) best = key;
                    }
                    best = warp_max_u64(best);
                    if (lane == round) mine64 = best;
                    prev = best;
                }
                if (mine64) {
                    my_idx = key_index(mine64);
                    my_lp = __float2bfloat16(__bfloat162float(x[my_idx]) - mx - ls);
                }
            } else if (got) {
                const unsigned long long c = mycand[0xFFFF - (got & 0xFFFFu)];
                my_idx = key_index(c);
                my_lp = __float2bfloat16(__bfloat162float(bf16_from_orderable(static_cast<uint32_t>(c >> 32))) - mx - ls);
            }
            if (lane < k) {
                s_val[r * k + lane] = my_lp;
                s_pos[r * k + lane] = my_idx;
            }
        }
        __syncthreads();
    }

    if (level == 0) {
        if (threadIdx.x < k) {
            const int i = threadIdx.x;
            st.tried_val[i] = s_val[i];
            st.tried_pos[i] = s_pos[i];
            st.fr_score[i] = s_val[i];
            st.fr_id[i] = st.token_id_remap ? st.token_id_remap[s_pos[i]] : s_pos[i];
            st.fr_mask[i] = 1ull << i;
            // frontier hidden state: the last valid row of the catch-up pass, for every node
            st.fr_src[i] = last_row_ptr ? *last_row_ptr : 0;
        }
        return;
    }

    // cumulative log-prob in bf16 (reference cumsum_kernel: value += frontier score, rounded to bf16)
    const int kk = k * k;
    const int base = k + (level - 1) * kk;
    for (int i = threadIdx.x; i < kk; i += blockDim.x) {
        const int r = i / k;
        const bf16 v = __float2bfloat16(__bfloat162float(s_val[i]) + __bfloat162float(st.fr_score[r]));
        s_val[i] = v;
        st.tried_val[base + i] = v;
        st.tried_pos[base + i] = s_pos[i];
        s_ckey[i] = (bf16_orderable(v) << 16) | static_cast<uint32_t>(0xFFFF - i);
    }
    if (threadIdx.x < k) s_oldmask[threadIdx.x] = st.fr_mask[threadIdx.x];
    __syncthreads();
    if (warp == 0) {
        const uint32_t got = warp_select(s_ckey, kk, k, lane);
        if (lane < k) s_sel[lane] = 0xFFFF - static_cast<int>(got & 0xFFFFu);
    }
    __syncthreads();
    if (threadIdx.x < k) {
        const int i = threadIdx.x;
        const int sel = s_sel[i];
        st.tried_parent[(level - 1) * k + i] = sel + base;
        st.fr_mask[i] = s_oldmask[sel / k] | (1ull << (k * level + i));
        st.fr_score[i] = s_val[sel];
        st.fr_id[i] = st.token_id_remap ? st.token_id_remap[s_pos[sel]] : s_pos[sel];
        st.fr_src[i] = sel / k;
    }
}

// hid_out[r] = h_rows[src[r]]: one CTA per row.
__global__ void gather_rows_kernel(const bf16* __restrict__ h_rows, int h_ld, const int32_t* __restrict__ src,
                                   bf16* __restrict__ hid_out, int hid_ld, int hidden) {
    grid_dependency_sync();
    const int r = blockIdx.x;
    const uint4* s4 = reinterpret_cast<const uint4*>(h_rows + static_cast<size_t>(src[r]) * h_ld);
    uint4* d4 = reinterpret_cast<uint4*>(hid_out + static_cast<size_t>(r) * hid_ld);
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) d4[c] = s4[c];
}

// ---- final selection of tree_size-1 candidates + tree arrays.  One CTA.
__global__ void tree_finalize_kernel(DraftTreeState st, const int32_t* __restrict__ cache_length,
                                     int32_t* __restrict__ tree_draft_ids, int32_t* __restrict__ tree_pos,
                                     uint64_t* __restrict__ tree_mask, int32_t* __restrict__ tree_parent,
                                     int* __restrict__ error) {
    grid_dependency_sync();
    __shared__ unsigned long long s_key[2048];
    __shared__ int s_sel[64];       // node i (1-based) <-> tried index s_sel[i-1]
    __shared__ int s_rank[2048];    // tried index -> node id (0 if not selected)
    __shared__ int s_par[64];
    const int k = st.k, T = st.tree_size, TT = st.total_tried;
    const int L = cache_length[0];
    for (int i = threadIdx.x; i < TT; i += blockDim.x) {
        s_key[i] = make_key(st.tried_val[i], i);
        s_rank[i] = 0;
    }
    __syncthreads();
    // rank by counting: position in (value desc, index asc) order
    for (int i = threadIdx.x; i < TT; i += blockDim.x) {
        const unsigned long long mine = s_key[i];
        int r = 0;
        for (int j = 0; j < TT; ++j) r += (s_key[j] > mine) ? 1 : 0;
        if (r < T - 1) {
            s_sel[r] = i;
            s_rank[i] = r + 1;
        }
    }
    __syncthreads();
    const int kk = k * k;
    if (threadIdx.x < T) {
        const int i = threadIdx.x;
        if (i == 0) {
            tree_pos[0] = L;
            s_par[0] = 0;
        } else {
            int p = s_sel[i - 1];
            st.sel_pos[i - 1] = p;
            const int depth = (p < k) ? 1 : (p - k) / kk + 2;
            tree_pos[i] = L + depth;
            int q;
            if (p < k) {
                q = -1;
            } else if (p - k < kk) {
                q = (p - k) / k;
            } else {
                q = st.tried_parent[(p - k - kk) / k];
            }
            int par = (q < 0) ? 0 : s_rank[q];
            if (q >= 0 && par == 0) {  // parent not selected: scores were not monotone (NaN/Inf input)
                atomicOr(error, ERR_BAD_TREE);
            }
            if (par >= i) {
                atomicOr(error, ERR_BAD_TREE);
                par = 0;
            }
            s_par[i] = par;
            tree_parent[i] = par;
            const int tok = st.tried_pos[p];
            tree_draft_ids[i] = st.token_id_remap ? st.token_id_remap[tok] : tok;
        }
    }
    __syncthreads();
    if (threadIdx.x < T) {
        const int i = threadIdx.x;
        uint64_t m = (1ull << i) | 1ull;
        int q = s_par[i];
        int guard = 0;
        while (q > 0 && guard++ < 64) {
            m |= 1ull << q;
            q = s_par[q];
        }
        tree_mask[i] = m;
    }
}

}  // namespace

int draft_num_segments(int vocab) { return ceil_div(vocab, SEG); }

size_t draft_scan_workspace_bytes(int rows, int vocab, int k) {
    const int nseg = draft_num_segments(vocab);
    (void)rows;
    return static_cast<size_t>(32) * nseg * (sizeof(float4) + static_cast<size_t>(k) * sizeof(unsigned long long)) + 1024;
}  // the first word is the level kernel's ticket and must be zero before the first launch

void launch_draft_topk_expand(const DraftTreeState& st, const bf16* logits, int ld, int vocab, int level,
                              void* scan_ws, const bf16* h_rows, int h_ld, const int32_t* last_row_ptr, bf16* hid_out,
                              int hid_ld, int hidden, cudaStream_t s) {
    const int k = st.k;
    const int rows = (level == 0) ? 1 : k;
    const int nseg = draft_num_segments(vocab);
    CPM_REQUIRE(k >= 1 && k <= 32, "draft: topk_per_iter must be in [1,32]");
    CPM_REQUIRE(hidden % 8 == 0, "draft: hidden size must be a multiple of 8");
    CPM_REQUIRE(nseg <= 128, "draft: vocabulary larger than 262144 entries");
    // workspace: [ticket | statistics 32 x nseg | candidates 32 x nseg x k]; the ticket is zero between launches
    unsigned* ticket = reinterpret_cast<unsigned*>(scan_ws);
    float4* stats = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(scan_ws) + 256);
    unsigned long long* cand = reinterpret_cast<unsigned long long*>(
        reinterpret_cast<uint8_t*>(stats) + align_up(static_cast<int64_t>(32) * nseg * sizeof(float4), 256));
    // the last CTA takes the rows in groups whose candidate lists (8 + 4 bytes per entry) fit its shared memory
    const size_t per_row_bytes = static_cast<size_t>(nseg) * k * (sizeof(unsigned long long) + sizeof(uint32_t));
    CPM_REQUIRE(nseg * k <= 65535, "draft: candidate list too long for 16-bit positions");
    CPM_REQUIRE(per_row_bytes <= 160 * 1024, "draft: a row's candidate list is too large for one CTA");
    const int group_rows = static_cast<int>(std::max<size_t>(1, std::min<size_t>(rows, (160 * 1024) / per_row_bytes)));
    const size_t shmem = group_rows * per_row_bytes;
    static size_t configured = 0;
    if (shmem > 24 * 1024 && shmem > configured) {   // the kernel also has about 12 KB of static shared memory
        CUDA_CHECK(cudaFuncSetAttribute(draft_level_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(160 * 1024)));
        configured = 160 * 1024;
    }
    launch_kernel(draft_level_kernel, dim3(nseg, rows), dim3(SCAN_THREADS), shmem, s, st, logits, ld, vocab, nseg, stats, cand,
                  ticket, level, last_row_ptr, group_rows);
    if (hid_out != nullptr) {
        launch_kernel(gather_rows_kernel, dim3(k), dim3(128), 0, s, h_rows, h_ld, static_cast<const int32_t*>(st.fr_src),
                      hid_out, hid_ld, hidden);
    }
}

void launch_tree_finalize(const DraftTreeState& st, const int32_t* cache_length, int32_t* tree_draft_ids,
                          int32_t* tree_pos, uint64_t* tree_mask, int32_t* tree_parent, cudaStream_t s) {
    CPM_REQUIRE(st.total_tried <= 2048, "draft: total tried candidates exceed 2048");
    CPM_REQUIRE(st.tree_size >= 2 && st.tree_size <= 64, "draft: tree_size must be in [2,64]");
    CPM_REQUIRE(st.tree_size - 1 <= st.total_tried, "draft: tree larger than the candidate set");
    launch_kernel(tree_finalize_kernel, dim3(1), dim3(512), 0, s, st, cache_length, tree_draft_ids, tree_pos, tree_mask,
                  tree_parent, runtime().d_error);
}
