// InfLLM-v2 block selection for the MiniCPM4 target (sm_100a): compressed key caches, stage-1
// scoring, max-pooling to 64-token blocks and top-k -> per-(kv head, token) block bitmask.
//
// Replaces, for the sparse target layers of the reference,
//   MiniCPM4KVCache::compress + meanpooling_{16,64}_kernel   src/model/minicpm4/minicpm4_kvcache.cuh:6-62, :243-254
//   mha_fwd_stage1 (flash stage-1 kernel + hdim16_reduce)      src/flash_attn/flash_api.hpp:204-290,
//                                                              src/flash_attn/src/flash_fwd_kernel.h:51-110, :1770-2265
//   maxpooling_func / TopK::prefill / topk_to_uint64_func      minicpm4_kvcache.cuh:64-201, src/model/topk.cuh:255-288
// as called from MiniCPM4Attention::prefill / decode (minicpm4_attn.cuh:96-166, :226-290).
//
// All lengths are derived on the device from the number of accepted KV rows L = *kv_len + kv_add
// (the reference keeps next_kv_length, c1_len, c2_len on the host), so the kernels can sit inside a
// captured step.  When selection is not active (compressed length below sparse_switch) the mask
// kernel writes all-ones masks and the attention kernel visits every block.
#include <mma.h>

#include "common.cuh"
#include "sparse_select.cuh"

namespace {

constexpr int C1_STRIDE = 16, C2_STRIDE = 64, BLOCK = 64;

__device__ __forceinline__ int compressed_len(int L, int stride) {
    const int n = (L - stride) / stride;
    return n > 0 ? n : 0;
}

__device__ __forceinline__ bool selection_active(int L, int sparse_switch, int compress_lse) {
    if (L <= 0) return false;
    return compress_lse ? compressed_len(L, C2_STRIDE) * C2_STRIDE >= sparse_switch
                        : compressed_len(L, C1_STRIDE) * C1_STRIDE >= sparse_switch;
}

// ---- compressed key caches: entry i = mean of rows [i * stride, i * stride + 2 * stride) of the layer's K cache.
// grid (max_new, layers, 2): blockIdx.z = 0 -> c1 (stride 16), 1 -> c2 (stride 64); entries [done, len(L)).
__global__ void sparse_compress_kernel(bf16* const* __restrict__ caches, int kv_dim, bf16* __restrict__ c1,
                                       size_t c1_layer_stride, bf16* __restrict__ c2, size_t c2_layer_stride,
                                       const int32_t* __restrict__ kv_len, int kv_add, const int32_t* __restrict__ done) {
    grid_dependency_sync();
    const int which = blockIdx.z, layer = blockIdx.y;
    if (which == 1 && c2 == nullptr) return;
    const int stride = which ? C2_STRIDE : C1_STRIDE;
    const int L = *kv_len + kv_add;
    const int idx = done[which] + blockIdx.x;
    if (idx >= compressed_len(L, stride)) return;
    const bf16* k = caches[2 * layer] + static_cast<size_t>(idx) * stride * kv_dim;
    bf16* out = (which ? c2 + layer * c2_layer_stride : c1 + layer * c1_layer_stride) + static_cast<size_t>(idx) * kv_dim;
    const int rows = 2 * stride;
    for (int c = threadIdx.x * 2; c < kv_dim; c += blockDim.x * 2) {
        float s0 = 0.f, s1 = 0.f;
        for (int r = 0; r < rows; ++r) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(k + static_cast<size_t>(r) * kv_dim + c);
            s0 += __low2float(v);
            s1 += __high2float(v);
        }
        *reinterpret_cast<__nv_bfloat162*>(out + c) = __floats2bfloat162_rn(s0 / rows, s1 / rows);
    }
}

__global__ void sparse_commit_kernel(const int32_t* __restrict__ kv_len, int kv_add, int32_t* __restrict__ done) {
    grid_dependency_sync();
    const int L = *kv_len + kv_add;
    done[0] = compressed_len(L, C1_STRIDE);
    done[1] = compressed_len(L, C2_STRIDE);
}

// ---- stage 1.  Scores are a small GEMM (tokens x heads against a few thousand compressed keys, 0.6 GFLOP
// per layer at 32k context) that is latency- and L2-bound, not tensor-bound: warp-level mma (wmma, 16 x 16 x 16
// bf16) with the 16 heads of a KV group as the M = 16 fragment is enough and keeps the kernel short.
//   lse kernel    grid (ceil(T / 8), hkv, key chunks of 128): per (token, head, chunk) the max and exp-sum of
//                 q.k over the LSE keys; the score kernel merges the chunks
//   score kernel  grid (ceil(T / 8), hkv, key chunks of 128): exp(q.k1 - max) / sum, summed over the group's
//                 heads, one 16-key fragment per warp
constexpr int S1_THREADS = 256, S1_MAXGRP = 16, S1_QLD = 128 + 8;

struct Stage1Args {
    const bf16* q;       // token t, head h at q + t * q_ld + h * 128
    int q_ld, grp, hkv, kv_dim;
    const bf16* c1;      // this layer's [n1][kv_dim]
    const bf16* c_lse;   // this layer's c2 (or c1)
    int lse_stride;      // C2_STRIDE or C1_STRIDE
    const int32_t* kv_len;
    int kv_add;
    const int32_t* n_valid;
    int sparse_switch, compress_lse;
    float scale_log2;
    float2* lse;         // [hkv][T][16][lse_chunks]: (max, exp-sum) of q.k per token, head and 128-key chunk of the LSE keys
    int lse_chunks;
    bf16* scores;        // [hkv][T][score_ld]
    int score_ld, T;
};

// Q rows of up to S1_TOK tokens x 16 heads of KV group g as bf16 [S1_TOK][16][S1_QLD] (zero rows beyond grp / T).
// S1_TOK = tokens per CTA: 8 for prefill chunks (key fragments reused eight times), 2 for decode-sized launches,
// where the per-warp token loop is the critical path and a four times larger grid shortens it.
template <int S1_TOK>
__device__ __forceinline__ void s1_load_q(const Stage1Args& a, int t0, int g, int t_end, bf16* q_s) {
    for (int i = threadIdx.x; i < S1_TOK * S1_MAXGRP * 16; i += S1_THREADS) {
        const int c = (i & 15) * 8, h = (i >> 4) & 15, tt = i >> 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (h < a.grp && t0 + tt < t_end) {
            v = *reinterpret_cast<const uint4*>(a.q + static_cast<size_t>(t0 + tt) * a.q_ld + (g * a.grp + h) * 128 + c);
        }
        *reinterpret_cast<uint4*>(q_s + (tt * S1_MAXGRP + h) * S1_QLD + c) = v;
    }
}

using KeyFrag = nvcuda::wmma::fragment<nvcuda::wmma::matrix_b, 16, 16, 16, __nv_bfloat16, nvcuda::wmma::col_major>;

// The 16 keys starting at `keys` (row stride kv_dim) as eight B fragments: loaded once per key fragment,
// all eight loads in flight together, and reused for every token.
__device__ __forceinline__ void s1_load_keys(const bf16* keys, int kv_dim, KeyFrag fb[8]) {
#pragma unroll
    for (int k = 0; k < 8; ++k) nvcuda::wmma::load_matrix_sync(fb[k], keys + k * 16, kv_dim);
}

// out[16 heads][16 keys] = Q(tt) K(frag)^T.
__device__ __forceinline__ void s1_frag_scores(const bf16* q_tok, const KeyFrag fb[8], float* out /*[16][16]*/) {
    using namespace nvcuda;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
    wmma::fill_fragment(acc, 0.f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
        wmma::load_matrix_sync(fa, q_tok + k * 16, S1_QLD);
        wmma::mma_sync(acc, fa, fb[k], acc);
    }
    wmma::store_matrix_sync(out, acc, 16, wmma::mem_row_major);
    __syncwarp();
}

template <int S1_TOK>
__global__ void __launch_bounds__(S1_THREADS) sparse_stage1_lse_kernel(const Stage1Args a) {
    grid_dependency_sync();
    __shared__ __align__(32) bf16 q_s[S1_TOK * S1_MAXGRP * S1_QLD];
    __shared__ __align__(32) float frag[S1_THREADS / 32][256];
    // after the key loop the fragment buffers hold the per-warp (max, sum) of every (token, head)
    float (*red_m)[S1_TOK * S1_MAXGRP] = reinterpret_cast<float (*)[S1_TOK * S1_MAXGRP]>(&frag[0][0]);
    float (*red_s)[S1_TOK * S1_MAXGRP] = reinterpret_cast<float (*)[S1_TOK * S1_MAXGRP]>(&frag[S1_THREADS / 64][0]);
    const int t0 = blockIdx.x * S1_TOK, g = blockIdx.y;
    const int L = *a.kv_len + a.kv_add;
    if (!selection_active(L, a.sparse_switch, a.compress_lse)) return;
    const int t_end = (a.n_valid != nullptr) ? min(*a.n_valid, a.T) : a.T;
    if (t0 >= t_end) return;
    const int nl = compressed_len(L, a.lse_stride);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (blockIdx.z * 128 >= nl) return;
    const int f = blockIdx.z * (S1_THREADS / 32) + warp;  // one 16-key fragment per warp
    // the key fragment is requested before the query rows: both global round trips overlap
    KeyFrag fb[8];
    if (f * 16 < nl) s1_load_keys(a.c_lse + static_cast<size_t>(f) * 16 * a.kv_dim + g * 128, a.kv_dim, fb);
    s1_load_q<S1_TOK>(a, t0, g, t_end, q_s);
    __syncthreads();
    // lane: head h = lane & 15, keys (lane >> 4) * 8 .. + 7 of the fragment
    const int h = lane & 15, kh = lane >> 4;
    float m[S1_TOK], s[S1_TOK];
#pragma unroll
    for (int tt = 0; tt < S1_TOK; ++tt) { m[tt] = -INFINITY; s[tt] = 0.f; }
    if (f * 16 < nl) {
#pragma unroll
        for (int tt = 0; tt < S1_TOK; ++tt) {
            s1_frag_scores(q_s + tt * S1_MAXGRP * S1_QLD, fb, frag[warp]);
            float mx = m[tt];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (f * 16 + kh * 8 + j < nl) mx = fmaxf(mx, frag[warp][h * 16 + kh * 8 + j]);
            }
            float sum = (mx == -INFINITY) ? 0.f : s[tt] * exp2f((m[tt] - mx) * a.scale_log2);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (f * 16 + kh * 8 + j < nl) sum += exp2f((frag[warp][h * 16 + kh * 8 + j] - mx) * a.scale_log2);
            }
            m[tt] = mx;
            s[tt] = sum;
            __syncwarp();  // frag[warp] is overwritten by the next token
        }
    }
    __syncthreads();  // every warp is done with its fragment buffer
    // merge the two key halves of a head (lanes h and h + 16), then the eight warps
#pragma unroll
    for (int tt = 0; tt < S1_TOK; ++tt) {
        const float om = __shfl_xor_sync(0xffffffffu, m[tt], 16), os = __shfl_xor_sync(0xffffffffu, s[tt], 16);
        const float mx = fmaxf(m[tt], om);
        const float sum = (mx == -INFINITY) ? 0.f
                                            : (m[tt] == -INFINITY ? 0.f : s[tt] * exp2f((m[tt] - mx) * a.scale_log2)) +
                                                  (om == -INFINITY ? 0.f : os * exp2f((om - mx) * a.scale_log2));
        if (kh == 0) { red_m[warp][tt * S1_MAXGRP + h] = mx; red_s[warp][tt * S1_MAXGRP + h] = sum; }
    }
    __syncthreads();
    if (threadIdx.x < S1_TOK * S1_MAXGRP) {
        const int tt = threadIdx.x >> 4, hh = threadIdx.x & 15;
        float mx = -INFINITY;
        const int e = tt * S1_MAXGRP + hh;
        for (int w = 0; w < S1_THREADS / 32; ++w) mx = fmaxf(mx, red_m[w][e]);
        float sum = 0.f;
        for (int w = 0; w < S1_THREADS / 32; ++w) {
            if (red_m[w][e] != -INFINITY) sum += red_s[w][e] * exp2f((red_m[w][e] - mx) * a.scale_log2);
        }
        if (t0 + tt < t_end) {
            a.lse[((static_cast<size_t>(g) * a.T + t0 + tt) * S1_MAXGRP + hh) * a.lse_chunks + blockIdx.z] = make_float2(mx, sum);
        }
    }
}

template <int S1_TOK>
__global__ void __launch_bounds__(S1_THREADS) sparse_stage1_score_kernel(const Stage1Args a) {
    grid_dependency_sync();
    __shared__ __align__(32) bf16 q_s[S1_TOK * S1_MAXGRP * S1_QLD];
    __shared__ __align__(32) float frag[S1_THREADS / 32][256];
    __shared__ float2 lse_s[S1_TOK][S1_MAXGRP];
    const int t0 = blockIdx.x * S1_TOK, g = blockIdx.y;
    const int L = *a.kv_len + a.kv_add;
    if (!selection_active(L, a.sparse_switch, a.compress_lse)) return;
    const int t_end = (a.n_valid != nullptr) ? min(*a.n_valid, a.T) : a.T;
    if (t0 >= t_end) return;
    const int n1 = compressed_len(L, C1_STRIDE);
    const int k_round = (n1 + 127) / 128 * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int key0 = (blockIdx.z * (S1_THREADS / 32) + warp) * 16;  // this warp's 16 keys
    if (blockIdx.z * 128 >= k_round) return;
    KeyFrag fb[8];   // requested before the query rows and the LSE partials: the global round trips overlap
    if (key0 < n1) s1_load_keys(a.c1 + static_cast<size_t>(key0) * a.kv_dim + g * 128, a.kv_dim, fb);
    s1_load_q<S1_TOK>(a, t0, g, t_end, q_s);
    if (threadIdx.x < S1_TOK * S1_MAXGRP) {
        // merge the chunk partials of this (token, head): (max, 1 / exp-sum) over all LSE keys
        const int tt = threadIdx.x >> 4, hh = threadIdx.x & 15;
        float2 r = make_float2(0.f, 0.f);
        if (t0 + tt < t_end) {
            const int nchunk = (compressed_len(L, a.lse_stride) + 127) / 128;
            const float2* part = a.lse + ((static_cast<size_t>(g) * a.T + t0 + tt) * S1_MAXGRP + hh) * a.lse_chunks;
            float mx = -INFINITY;
            for (int c = 0; c < nchunk; ++c) mx = fmaxf(mx, part[c].x);
            float sum = 0.f;
            for (int c = 0; c < nchunk; ++c) {
                if (part[c].x != -INFINITY) sum += part[c].y * exp2f((part[c].x - mx) * a.scale_log2);
            }
            r = make_float2(mx == -INFINITY ? 0.f : mx, sum > 0.f ? 1.f / sum : 0.f);
        }
        lse_s[tt][hh] = r;
    }
    __syncthreads();
    const int key = lane & 15, hh0 = (lane >> 4) * 8;  // lane: one key, eight of the sixteen heads
#pragma unroll 1
    for (int tt = 0; tt < S1_TOK; ++tt) {
        if (t0 + tt >= t_end) break;
        float mine = 0.f;
        if (key0 < n1) {
            s1_frag_scores(q_s + tt * S1_MAXGRP * S1_QLD, fb, frag[warp]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int hh = hh0 + j;
                if (hh < a.grp) mine += exp2f((frag[warp][hh * 16 + key] - lse_s[tt][hh].x) * a.scale_log2) * lse_s[tt][hh].y;
            }
            __syncwarp();
        }
        mine += __shfl_xor_sync(0xffffffffu, mine, 16);
        if (lane < 16) {
            a.scores[(static_cast<size_t>(g) * a.T + t0 + tt) * a.score_ld + key0 + key] =
                __float2bfloat16(key0 + key < n1 ? mine : 0.f);
        }
    }
}

// ---- max-pool to 64-token blocks, top-k, bitmask.  grid (T, hkv), 256 threads, up to 4096 blocks.
constexpr int PT_THREADS = 256, PT_PER = 16;

__device__ __forceinline__ unsigned long long score_key(bf16 v, int idx) {
    // order: value descending, lower index first  (0 is below every key)
    unsigned short b = __bfloat16_as_ushort(v);
    b = (b & 0x8000u) ? static_cast<unsigned short>(~b) : static_cast<unsigned short>(b | 0x8000u);
    return (static_cast<unsigned long long>(b) << 32) | static_cast<unsigned int>(0x7fffffff - idx);
}

struct PoolArgs {
    const bf16* scores;  // [hkv][T][score_ld]
    int score_ld, T;
    const int32_t* kv_len;
    int kv_add;
    const int32_t* n_valid;
    int sparse_switch, compress_lse;
    int init_blocks, local_blocks, topk;
    uint64_t* blockmask;  // [hkv][T][bm_words]
    int bm_words;
};

// Pooled score of block k for query token t (maxpooling_kernel of the reference) as a selection key.
__device__ __forceinline__ unsigned long long pooled_key(const PoolArgs& a, const bf16* in, int k, int k_len, int q_block) {
    bf16 v;
    if (k < a.init_blocks) {
        v = __ushort_as_bfloat16(0x7f80);  // +inf
    } else if (q_block - a.local_blocks < k) {
        v = __ushort_as_bfloat16(0xff80);  // -inf
    } else {
        int start = k * 4 - 1, end = start + 5;
        start = max(start, 0);
        end = min(end, k_len);
        float mx = __bfloat162float(in[start]);
        for (int i = start + 1; i < end; ++i) mx = fmaxf(mx, __bfloat162float(in[i]));
        v = __float2bfloat16(mx);
    }
    return score_key(v, k);
}

// One CTA of 128 threads per (kv head, token) row for up to 128 * PB blocks; thread i owns the PB consecutive
// blocks i * PB ...  The row's scores are staged in shared memory (coalesced).  Instead of extracting one
// maximum per round, the k-th largest 16-bit score is found by a bitwise binary search with block-wide counts
// (16 steps, one barrier each), every block above it is taken, and the remaining picks among the blocks equal
// to it go to the lowest indices (exclusive scan of the per-thread counts in thread = index order): the same
// set as "value descending, lower index first".  grid (T, hkv).
template <int PB>
__global__ void __launch_bounds__(128) sparse_pool_topk_block_kernel(const PoolArgs a) {
    grid_dependency_sync();
    constexpr int CAP = 128 * PB * 4 + 128;   // staged scores: four per block and the pooling halo
    __shared__ __align__(16) bf16 row_s[CAP];
    __shared__ uint32_t s_cnt[2][4];
    __shared__ uint32_t s_tot[2][4];
    __shared__ unsigned long long s_words[PB * 2];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int t = blockIdx.x, g = blockIdx.y;
    uint64_t* out = a.blockmask + (static_cast<size_t>(g) * a.T + t) * a.bm_words;
    const int L = *a.kv_len + a.kv_add;
    if (!selection_active(L, a.sparse_switch, a.compress_lse)) {
        for (int w = tid; w < a.bm_words; w += 128) out[w] = ~0ull;
        return;
    }
    if (a.n_valid != nullptr && t >= *a.n_valid) {
        for (int w = tid; w < a.bm_words; w += 128) out[w] = 0ull;
        return;
    }
    const int n1 = compressed_len(L, C1_STRIDE);
    const int k_len = (n1 + 127) / 128 * 128;
    const int out_len = (L + BLOCK - 1) / BLOCK;
    const int q_block = (t + L) / BLOCK;
    const bf16* in = a.scores + (static_cast<size_t>(g) * a.T + t) * a.score_ld;
    for (int i = tid * 8; i < k_len && i < CAP; i += 1024) {
        *reinterpret_cast<uint4*>(row_s + i) = *reinterpret_cast<const uint4*>(in + i);
    }
    if (tid < PB * 2) s_words[tid] = 0ull;
    __syncthreads();
    uint32_t val[PB];  // orderable 16-bit score of block tid * PB + j, 0 = no such block
    uint32_t valid = 0;
#pragma unroll
    for (int j = 0; j < PB; ++j) {
        const int k = tid * PB + j;
        val[j] = (k < out_len) ? static_cast<uint32_t>(pooled_key(a, row_s, k, k_len, q_block) >> 32) : 0u;
        valid += val[j] != 0u;
    }
    // block-wide sum of a per-thread count; `slot` alternates so that one barrier per call is enough
    auto block_sum = [&](uint32_t v, int slot) {
        v = __reduce_add_sync(0xffffffffu, v);
        if (lane == 0) s_cnt[slot][wid] = v;
        __syncthreads();
        return s_cnt[slot][0] + s_cnt[slot][1] + s_cnt[slot][2] + s_cnt[slot][3];
    };
    const uint32_t total = block_sum(valid, 0);
    uint32_t kth = 1u;                 // everything valid is taken when there are at most topk blocks
    uint32_t need = 0xffffffffu;       // picks left for the blocks equal to kth
    if (total > static_cast<uint32_t>(a.topk)) {   // uniform across the CTA
        kth = 0u;
        for (int bit = 15; bit >= 0; --bit) {
            const uint32_t cand = kth | (1u << bit);
            uint32_t c = 0;
#pragma unroll
            for (int j = 0; j < PB; ++j) c += val[j] >= cand;
            if (block_sum(c, bit & 1) >= static_cast<uint32_t>(a.topk)) kth = cand;   // slots 1, 0, 1, ... after the 0 above
        }
        uint32_t gt = 0;
#pragma unroll
        for (int j = 0; j < PB; ++j) gt += val[j] > kth;
        need = static_cast<uint32_t>(a.topk) - block_sum(gt, 1);
    }
    // blocks equal to kth before this thread's, in index order
    uint32_t eq = 0;
#pragma unroll
    for (int j = 0; j < PB; ++j) eq += (val[j] == kth) && (val[j] != 0u);
    uint32_t incl = eq;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) s_tot[0][wid] = incl;
    __syncthreads();
    uint32_t rank = incl - eq;
    for (int w = 0; w < wid; ++w) rank += s_tot[0][w];
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < PB; ++j) {
        const bool is_eq = (val[j] == kth) && (val[j] != 0u);
        const bool take = (val[j] > kth) || (is_eq && (need == 0xffffffffu || rank < need));
        rank += is_eq;
        bits |= static_cast<uint32_t>(take) << j;
    }
    if (bits) atomicOr(&s_words[(tid * PB) >> 6], static_cast<unsigned long long>(bits) << ((tid * PB) & 63));
    __syncthreads();
    for (int w = tid; w < a.bm_words; w += 128) out[w] = (w < PB * 2) ? s_words[w] : 0ull;
}

__global__ void __launch_bounds__(PT_THREADS) sparse_pool_topk_kernel(const PoolArgs a) {
    grid_dependency_sync();
    __shared__ unsigned long long sh_best[PT_THREADS / 32];
    __shared__ unsigned long long words[64];
    const int t = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;
    uint64_t* out = a.blockmask + (static_cast<size_t>(g) * a.T + t) * a.bm_words;
    const int L = *a.kv_len + a.kv_add;
    if (!selection_active(L, a.sparse_switch, a.compress_lse)) {
        for (int w = tid; w < a.bm_words; w += PT_THREADS) out[w] = ~0ull;
        return;
    }
    if (a.n_valid != nullptr && t >= *a.n_valid) {
        for (int w = tid; w < a.bm_words; w += PT_THREADS) out[w] = 0ull;
        return;
    }
    const int n1 = compressed_len(L, C1_STRIDE);
    const int k_len = (n1 + 127) / 128 * 128;
    const int out_len = (L + BLOCK - 1) / BLOCK;
    const int q_block = (t + L) / BLOCK;
    const bf16* in = a.scores + (static_cast<size_t>(g) * a.T + t) * a.score_ld;
    unsigned long long keys[PT_PER];
#pragma unroll
    for (int j = 0; j < PT_PER; ++j) {
        const int k = j * PT_THREADS + tid;
        keys[j] = 0ull;
        if (k < out_len) {
            bf16 v;
            if (k < a.init_blocks) {
                v = __ushort_as_bfloat16(0x7f80);  // +inf
            } else if (q_block - a.local_blocks < k) {
                v = __ushort_as_bfloat16(0xff80);  // -inf
            } else {
                int start = k * 4 - 1, end = start + 5;
                start = max(start, 0);
                end = min(end, k_len);
                float mx = __bfloat162float(in[start]);
                for (int i = start + 1; i < end; ++i) mx = fmaxf(mx, __bfloat162float(in[i]));
                v = __float2bfloat16(mx);
            }
            keys[j] = score_key(v, k);
        }
    }
    if (tid < 64) words[tid] = 0ull;
    __syncthreads();
    for (int round = 0; round < a.topk; ++round) {
        unsigned long long best = 0ull;
#pragma unroll
        for (int j = 0; j < PT_PER; ++j) best = (keys[j] > best) ? keys[j] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = (other > best) ? other : best;
        }
        if ((tid & 31) == 0) sh_best[tid >> 5] = best;
        __syncthreads();
        best = sh_best[0];
#pragma unroll
        for (int w = 1; w < PT_THREADS / 32; ++w) best = (sh_best[w] > best) ? sh_best[w] : best;
        __syncthreads();
        if (best == 0ull) break;  // fewer blocks than topk: all of them are selected
        const int idx = 0x7fffffff - static_cast<int>(best & 0xffffffffu);
        if (tid == 0) words[idx >> 6] |= 1ull << (idx & 63);
#pragma unroll
        for (int j = 0; j < PT_PER; ++j) {
            if (keys[j] == best) keys[j] = 0ull;
        }
    }
    __syncthreads();
    for (int w = tid; w < a.bm_words; w += PT_THREADS) out[w] = (w < 64) ? words[w] : 0ull;
}

}  // namespace

void launch_sparse_compress(const SparseBuffers& b, bf16* const* caches, int layers, int kv_dim, const int32_t* kv_len,
                            int kv_add, int max_new, cudaStream_t s) {
    ProfileScope prof(KC_OTHER, s);
    if (max_new < 1) max_new = 1;
    launch_kernel(sparse_compress_kernel, dim3(max_new, layers, b.c2 ? 2 : 1), dim3(128), 0, s, caches, kv_dim, b.c1,
                  b.c1_layer_stride, b.c2, b.c2_layer_stride, kv_len, kv_add, static_cast<const int32_t*>(b.done));
    launch_kernel(sparse_commit_kernel, dim3(1), dim3(1), 0, s, kv_len, kv_add, b.done);
}

void launch_sparse_select(const SparseBuffers& b, const SparseConfig& cfg, int layer, const bf16* q, int q_ld, int T,
                          int hq, int hkv, const int32_t* kv_len, int kv_add, const int32_t* n_valid, cudaStream_t s) {
    ProfileScope prof(KC_OTHER, s);
    const int grp = hq / hkv;
    CPM_REQUIRE(grp >= 1 && grp <= S1_MAXGRP, "sparse selection: at most 16 query heads per KV head");
    CPM_REQUIRE(T <= b.max_tokens, "sparse selection: more query tokens than the buffers hold");
    Stage1Args a;
    a.q = q; a.q_ld = q_ld; a.grp = grp; a.hkv = hkv; a.kv_dim = hkv * 128;
    a.c1 = b.c1 + layer * b.c1_layer_stride;
    a.c_lse = cfg.compress_lse ? b.c2 + layer * b.c2_layer_stride : a.c1;
    a.lse_stride = cfg.compress_lse ? C2_STRIDE : C1_STRIDE;
    a.kv_len = kv_len; a.kv_add = kv_add; a.n_valid = n_valid;
    a.sparse_switch = cfg.sparse_switch; a.compress_lse = cfg.compress_lse ? 1 : 0;
    a.scale_log2 = 1.4426950408889634f / sqrtf(128.f);
    a.scores = b.scores; a.score_ld = b.score_ld; a.T = T;
    a.lse = b.lse;
    a.lse_chunks = b.score_ld / 128;
    const int lse_z = cfg.compress_lse ? ceil_div(a.lse_chunks, 4) : a.lse_chunks;
    if (T <= 64) {
        launch_kernel(sparse_stage1_lse_kernel<2>, dim3(ceil_div(T, 2), hkv, lse_z), dim3(S1_THREADS), 0, s, a);
        launch_kernel(sparse_stage1_score_kernel<2>, dim3(ceil_div(T, 2), hkv, b.score_ld / 128), dim3(S1_THREADS), 0, s, a);
    } else {
        launch_kernel(sparse_stage1_lse_kernel<8>, dim3(ceil_div(T, 8), hkv, lse_z), dim3(S1_THREADS), 0, s, a);
        launch_kernel(sparse_stage1_score_kernel<8>, dim3(ceil_div(T, 8), hkv, b.score_ld / 128), dim3(S1_THREADS), 0, s, a);
    }
    PoolArgs p;
    p.scores = b.scores; p.score_ld = b.score_ld; p.T = T;
    p.kv_len = kv_len; p.kv_add = kv_add; p.n_valid = n_valid;
    p.sparse_switch = cfg.sparse_switch; p.compress_lse = a.compress_lse;
    p.init_blocks = cfg.sink_blocks; p.local_blocks = cfg.window_blocks; p.topk = cfg.topk;
    p.blockmask = b.blockmask; p.bm_words = b.bm_words;
    CPM_REQUIRE(b.bm_words <= 64, "sparse selection: at most 4096 blocks (262144 tokens)");
    const int max_blocks = b.score_ld / 4 + 1;  // score_ld >= budget / 16
    if (max_blocks <= 512) {
        launch_kernel(sparse_pool_topk_block_kernel<4>, dim3(T, hkv), dim3(128), 0, s, p);
    } else if (max_blocks <= 1024) {
        launch_kernel(sparse_pool_topk_block_kernel<8>, dim3(T, hkv), dim3(128), 0, s, p);
    } else {
        launch_kernel(sparse_pool_topk_kernel, dim3(T, hkv), dim3(PT_THREADS), 0, s, p);
    }
}
