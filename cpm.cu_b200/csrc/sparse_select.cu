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

// ---- stage 1: for query token t and kv head g (grid (T, hkv), 256 threads): per head the max and
// exp-sum of q.k over the LSE keys, then sum over the group's heads of exp(q.k1 - max) / sum for every
// c1 key.  Thread (key lane kk = tid & 63, head set hs = tid >> 6) handles heads hs, hs + 4, ...
constexpr int S1_THREADS = 256, S1_KEYS = 64, S1_MAXGRP = 16, S1_HPT = S1_MAXGRP / 4;

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
    bf16* scores;        // [hkv][T][score_ld]
    int score_ld, T;
};

__device__ __forceinline__ void s1_dots(const bf16* __restrict__ ktile, const float* __restrict__ q_s, int kk, int hs, int grp,
                                        float acc[S1_HPT]) {
#pragma unroll
    for (int j = 0; j < S1_HPT; ++j) acc[j] = 0.f;
    const bf16* krow = ktile + kk * (128 + 8);
#pragma unroll 4
    for (int d = 0; d < 128; d += 2) {
        const __nv_bfloat162 kv = *reinterpret_cast<const __nv_bfloat162*>(krow + d);
        const float k0 = __low2float(kv), k1 = __high2float(kv);
#pragma unroll
        for (int j = 0; j < S1_HPT; ++j) {
            const int h = hs + 4 * j;
            if (h < grp) acc[j] = fmaf(k1, q_s[h * 128 + d + 1], fmaf(k0, q_s[h * 128 + d], acc[j]));
        }
    }
}

__global__ void __launch_bounds__(S1_THREADS) sparse_stage1_kernel(const Stage1Args a) {
    grid_dependency_sync();
    __shared__ float q_s[S1_MAXGRP * 128];
    __shared__ __align__(16) bf16 ktile[S1_KEYS * (128 + 8)];
    __shared__ float red_m[S1_MAXGRP][S1_KEYS], red_s[S1_MAXGRP][S1_KEYS];
    __shared__ float head_m[S1_MAXGRP], head_inv[S1_MAXGRP];
    __shared__ float part[4][S1_KEYS];
    const int t = blockIdx.x, g = blockIdx.y;
    const int L = *a.kv_len + a.kv_add;
    if (!selection_active(L, a.sparse_switch, a.compress_lse)) return;
    if (a.n_valid != nullptr && t >= *a.n_valid) return;
    const int n1 = compressed_len(L, C1_STRIDE);
    const int nl = compressed_len(L, a.lse_stride);
    const int tid = threadIdx.x, kk = tid & 63, hs = tid >> 6;
    for (int i = tid; i < a.grp * 128; i += S1_THREADS) {
        q_s[i] = __bfloat162float(a.q[static_cast<size_t>(t) * a.q_ld + (g * a.grp + i / 128) * 128 + (i & 127)]);
    }
    auto load_tile = [&](const bf16* base, int k0, int n) {
        __syncthreads();  // previous tile fully consumed
        for (int i = tid; i < S1_KEYS * 16; i += S1_THREADS) {
            const int r = i >> 4, c = (i & 15) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k0 + r < n) v = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(k0 + r) * a.kv_dim + g * 128 + c);
            *reinterpret_cast<uint4*>(ktile + r * (128 + 8) + c) = v;
        }
        __syncthreads();
    };
    // pass 1: running max / exp-sum per head over the LSE keys (each thread: its key lane, its heads)
    float m[S1_HPT], s[S1_HPT];
#pragma unroll
    for (int j = 0; j < S1_HPT; ++j) { m[j] = -INFINITY; s[j] = 0.f; }
    for (int k0 = 0; k0 < nl; k0 += S1_KEYS) {
        load_tile(a.c_lse, k0, nl);
        if (k0 + kk < nl) {
            float acc[S1_HPT];
            s1_dots(ktile, q_s, kk, hs, a.grp, acc);
#pragma unroll
            for (int j = 0; j < S1_HPT; ++j) {
                const float mn = fmaxf(m[j], acc[j]);
                s[j] = s[j] * exp2f((m[j] - mn) * a.scale_log2) + exp2f((acc[j] - mn) * a.scale_log2);
                m[j] = mn;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < S1_HPT; ++j) {
        const int h = hs + 4 * j;
        if (h < a.grp) { red_m[h][kk] = m[j]; red_s[h][kk] = s[j]; }
    }
    __syncthreads();
    if (tid < a.grp) {
        float mx = -INFINITY;
        for (int i = 0; i < S1_KEYS; ++i) mx = fmaxf(mx, red_m[tid][i]);
        float sum = 0.f;
        for (int i = 0; i < S1_KEYS; ++i) {
            if (red_m[tid][i] != -INFINITY) sum += red_s[tid][i] * exp2f((red_m[tid][i] - mx) * a.scale_log2);
        }
        head_m[tid] = (mx == -INFINITY) ? 0.f : mx;
        head_inv[tid] = 1.f / sum;
    }
    __syncthreads();
    // pass 2: normalised probabilities over the c1 keys, summed over the group's heads
    bf16* out = a.scores + (static_cast<size_t>(g) * a.T + t) * a.score_ld;
    const int k_round = (n1 + 127) / 128 * 128;
    for (int k0 = 0; k0 < k_round; k0 += S1_KEYS) {
        float mine = 0.f;
        if (k0 < n1) {
            load_tile(a.c1, k0, n1);
            if (k0 + kk < n1) {
                float acc[S1_HPT];
                s1_dots(ktile, q_s, kk, hs, a.grp, acc);
#pragma unroll
                for (int j = 0; j < S1_HPT; ++j) {
                    const int h = hs + 4 * j;
                    if (h < a.grp) mine += exp2f((acc[j] - head_m[h]) * a.scale_log2) * head_inv[h];
                }
            }
        } else {
            __syncthreads();
        }
        part[hs][kk] = mine;
        __syncthreads();
        if (hs == 0) out[k0 + kk] = __float2bfloat16((part[0][kk] + part[1][kk]) + (part[2][kk] + part[3][kk]));
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
    if (max_new < 1) max_new = 1;
    launch_kernel(sparse_compress_kernel, dim3(max_new, layers, b.c2 ? 2 : 1), dim3(128), 0, s, caches, kv_dim, b.c1,
                  b.c1_layer_stride, b.c2, b.c2_layer_stride, kv_len, kv_add, static_cast<const int32_t*>(b.done));
    launch_kernel(sparse_commit_kernel, dim3(1), dim3(1), 0, s, kv_len, kv_add, b.done);
}

void launch_sparse_select(const SparseBuffers& b, const SparseConfig& cfg, int layer, const bf16* q, int q_ld, int T,
                          int hq, int hkv, const int32_t* kv_len, int kv_add, const int32_t* n_valid, cudaStream_t s) {
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
    launch_kernel(sparse_stage1_kernel, dim3(T, hkv), dim3(S1_THREADS), 0, s, a);
    PoolArgs p;
    p.scores = b.scores; p.score_ld = b.score_ld; p.T = T;
    p.kv_len = kv_len; p.kv_add = kv_add; p.n_valid = n_valid;
    p.sparse_switch = cfg.sparse_switch; p.compress_lse = a.compress_lse;
    p.init_blocks = cfg.sink_blocks; p.local_blocks = cfg.window_blocks; p.topk = cfg.topk;
    p.blockmask = b.blockmask; p.bm_words = b.bm_words;
    CPM_REQUIRE(b.bm_words <= 64, "sparse selection: at most 4096 blocks (262144 tokens)");
    launch_kernel(sparse_pool_topk_kernel, dim3(T, hkv), dim3(PT_THREADS), 0, s, p);
}
