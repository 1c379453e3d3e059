// Row-wise helper kernels of the speculative step: RMSNorm (with the in-place
// residual add the reference fuses into it), embedding gather, NeoX rotary
// embedding fused with the KV-cache append, SwiGLU gating, residual add and the
// target argmax.  Each is bound by a few hundred KB of traffic per launch; they
// exist so that every rounding point matches the reference kernels:
//   src/model/norm.cuh:8-99, embedding.cuh:7-52, rotary.cuh:7-34,
//   attn.cuh:14-40 (copy_to_kvcache / permute), activation.cuh:7-18,
//   elementwise.cuh:8-87.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    const int nw = blockDim.x >> 5;
    float t = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) sh[0] = t;
    }
    __syncthreads();
    t = sh[0];
    __syncthreads();
    return t;
}

// y = x * rsqrt(mean(x^2) + eps) * w, optionally after x += round(delta * scale).
// One CTA per row; every thread owns up to VPT 16-byte vectors of the row, loads them
// all up front and keeps them in registers between the two passes.
template <bool ADD, int VPT>
__global__ void rms_norm_kernel(bf16* __restrict__ x, int ldx, const bf16* __restrict__ delta, float delta_scale,
                                const bf16* __restrict__ w, bf16* __restrict__ y, int ldy, int dim, float eps) {
    grid_dep_trigger();
    __shared__ float sh[32];
    const size_t base = static_cast<size_t>(blockIdx.x) * ldx;
    const size_t dbase = static_cast<size_t>(blockIdx.x) * dim;
    const size_t ybase = static_cast<size_t>(blockIdx.x) * ldy;
    const int nvec = dim >> 3;
    // the norm weights never depend on the previous kernel: fetched before the dependency wait
    uint4 wv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) wv[j] = __ldg(reinterpret_cast<const uint4*>(w + v * 8));
    }
    grid_dep_wait();
    uint4 xv[VPT], dv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            xv[j] = *reinterpret_cast<const uint4*>(x + base + v * 8);
            if (ADD) dv[j] = *reinterpret_cast<const uint4*>(delta + dbase + v * 8);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            bf16* xe = reinterpret_cast<bf16*>(&xv[j]);
            if (ADD) {
                const bf16* de = reinterpret_cast<const bf16*>(&dv[j]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    bf16 dl = de[e];
                    if (delta_scale != 1.0f) dl = __float2bfloat16(__bfloat162float(dl) * delta_scale);
                    xe[e] = __float2bfloat16(__bfloat162float(xe[e]) + __bfloat162float(dl));
                }
                *reinterpret_cast<uint4*>(x + base + v * 8) = xv[j];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float f = __bfloat162float(xe[e]);
                ss += f * f;
            }
        }
    }
    ss = block_sum(ss, sh);
    const float rs = rsqrtf(ss / dim + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = threadIdx.x + j * blockDim.x;
        if (v < nvec) {
            const bf16* xe = reinterpret_cast<const bf16*>(&xv[j]);
            const bf16* we = reinterpret_cast<const bf16*>(&wv[j]);
            uint4 ov;
            bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
            for (int e = 0; e < 8; ++e) oe[e] = __float2bfloat16(rs * __bfloat162float(xe[e]) * __bfloat162float(we[e]));
            *reinterpret_cast<uint4*>(y + ybase + v * 8) = ov;
        }
    }
}

__global__ void embedding_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ table,
                                 bf16* __restrict__ out, int ld_out, int dim, float scale) {
    grid_dependency_sync();
    const int row = blockIdx.x;
    const size_t src = static_cast<size_t>(ids[row]) * dim;
    const size_t dst = static_cast<size_t>(row) * ld_out;
    for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(table + src + i);
        if (scale != 1.0f) {
            bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(__bfloat162float(e[j]) * scale);
        }
        *reinterpret_cast<uint4*>(out + dst + i) = v;
    }
}

// Embedding rows (blockIdx.y == 0) and, in the same launch, gathered hidden rows
// hid_out[r] = h_rows[src[r]] (blockIdx.y == 1): the two halves of the draft layer's input.
__global__ void embedding_gather_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ table,
                                        bf16* __restrict__ out, int ld_out, int dim, float scale,
                                        const bf16* __restrict__ h_rows, int h_ld, const int32_t* __restrict__ src,
                                        bf16* __restrict__ hid_out, int hid_ld) {
    grid_dependency_sync();
    const int row = blockIdx.x;
    if (blockIdx.y == 1) {
        const uint4* s4 = reinterpret_cast<const uint4*>(h_rows + static_cast<size_t>(src[row]) * h_ld);
        uint4* d4 = reinterpret_cast<uint4*>(hid_out + static_cast<size_t>(row) * hid_ld);
        for (int c = threadIdx.x; c < dim / 8; c += blockDim.x) d4[c] = s4[c];
        return;
    }
    const size_t from = static_cast<size_t>(ids[row]) * dim;
    const size_t dst = static_cast<size_t>(row) * ld_out;
    for (int i = threadIdx.x * 8; i < dim; i += blockDim.x * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(table + from + i);
        if (scale != 1.0f) {
            bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16(__bfloat162float(e[j]) * scale);
        }
        *reinterpret_cast<uint4*>(out + dst + i) = v;
    }
}

// One CTA per token row.  q heads rotate in place; k heads rotate into the
// cache; v heads are copied into the cache.  The d/2 sines and cosines of the row's
// position are computed once per CTA; each thread then rotates element pairs
// (c, c+1) and (c + d/2, c + d/2 + 1) with 4-byte accesses.
__global__ void rope_append_kernel(bf16* __restrict__ qkv, int hq, int hkv, int d, const float* __restrict__ inv_freq,
                                   const int32_t* __restrict__ pos, const int32_t* __restrict__ pos_base, int pos_off,
                                   int pos_step, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                   const int32_t* __restrict__ kv_len, int kv_off,
                                   const int32_t* __restrict__ n_valid, int cache_rows, int* __restrict__ error) {
    grid_dependency_sync();
    __shared__ float s_cos[128], s_sin[128];
    const int r = blockIdx.x;
    const int half = d >> 1;
    const int ld = (hq + 2 * hkv) * d;
    bf16* row = qkv + static_cast<size_t>(r) * ld;
    const int p = (pos != nullptr) ? pos[r] : (*pos_base + pos_off + r * pos_step);
    bool store_kv = (n_valid == nullptr) || (r < *n_valid);
    const long long kv_row = static_cast<long long>(*kv_len) + kv_off + r;
    if (store_kv && kv_row >= cache_rows) {  // host-side length checks come first; this only keeps memory intact
        store_kv = false;
        if (threadIdx.x == 0) atomicOr(error, ERR_KV_OVERFLOW);
    }
    const int kv_dim = hkv * d;
    if (threadIdx.x < half) {
        float sn, cs;
        sincosf(p * inv_freq[threadIdx.x], &sn, &cs);
        s_cos[threadIdx.x] = cs;
        s_sin[threadIdx.x] = sn;
    }
    __syncthreads();
    const int pairs = half >> 1;  // bf16x2 pairs per half head
    for (int i = threadIdx.x; i < (hq + hkv) * pairs; i += blockDim.x) {
        const int h = i / pairs, c = (i - h * pairs) * 2;
        bf16* hp = row + h * d;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(hp + c);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(hp + c + half);
        const float a0 = __bfloat162float(lo.x), a1 = __bfloat162float(lo.y);
        const float b0 = __bfloat162float(hi.x), b1 = __bfloat162float(hi.y);
        __nv_bfloat162 o_lo, o_hi;
        o_lo.x = __float2bfloat16(a0 * s_cos[c] - b0 * s_sin[c]);
        o_lo.y = __float2bfloat16(a1 * s_cos[c + 1] - b1 * s_sin[c + 1]);
        o_hi.x = __float2bfloat16(a0 * s_sin[c] + b0 * s_cos[c]);
        o_hi.y = __float2bfloat16(a1 * s_sin[c + 1] + b1 * s_cos[c + 1]);
        if (h < hq) {
            *reinterpret_cast<__nv_bfloat162*>(hp + c) = o_lo;
            *reinterpret_cast<__nv_bfloat162*>(hp + c + half) = o_hi;
        } else if (store_kv && kv_row >= 0) {
            bf16* kd = k_cache + kv_row * kv_dim + (h - hq) * d;
            *reinterpret_cast<__nv_bfloat162*>(kd + c) = o_lo;
            *reinterpret_cast<__nv_bfloat162*>(kd + c + half) = o_hi;
        }
    }
    if (store_kv && kv_row >= 0) {
        const bf16* vsrc = row + (hq + hkv) * d;
        bf16* vdst = v_cache + kv_row * kv_dim;
        for (int i = threadIdx.x * 8; i < kv_dim; i += blockDim.x * 8) {
            *reinterpret_cast<uint4*>(vdst + i) = *reinterpret_cast<const uint4*>(vsrc + i);
        }
    }
}

__global__ void silu_gate_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter, int interleaved) {
    grid_dependency_sync();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= inter) return;
    const bf16* g = gate_up + static_cast<size_t>(r) * 2 * inter;
    // [gate | up] halves, or per 64 features 64 gate columns followed by their 64 up columns
    const int gc = interleaved ? (c / 64) * 128 + (c % 64) : c;
    const int uc = interleaved ? gc + 64 : inter + c;
    const uint4 gv = *reinterpret_cast<const uint4*>(g + gc);
    const uint4 uv = *reinterpret_cast<const uint4*>(g + uc);
    const bf16* ge = reinterpret_cast<const bf16*>(&gv);
    const bf16* ue = reinterpret_cast<const bf16*>(&uv);
    uint4 ov;
    bf16* oe = reinterpret_cast<bf16*>(&ov);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        oe[e] = __float2bfloat16(silu_mul(__bfloat162float(ge[e]), __bfloat162float(ue[e])));
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * inter + c) = ov;
}

__global__ void add_scaled_kernel(bf16* __restrict__ x, const bf16* __restrict__ a, const bf16* __restrict__ b,
                                  float scale_b, size_t n) {
    grid_dependency_sync();
    const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const __nv_bfloat162 av = *reinterpret_cast<const __nv_bfloat162*>(a + i);
    __nv_bfloat162 bv = *reinterpret_cast<const __nv_bfloat162*>(b + i);
    if (scale_b != 1.0f) {
        bv.x = __float2bfloat16(__bfloat162float(bv.x) * scale_b);
        bv.y = __float2bfloat16(__bfloat162float(bv.y) * scale_b);
    }
    __nv_bfloat162 o;
    o.x = __float2bfloat16(__bfloat162float(av.x) + __bfloat162float(bv.x));
    o.y = __float2bfloat16(__bfloat162float(av.y) + __bfloat162float(bv.y));
    *reinterpret_cast<__nv_bfloat162*>(x + i) = o;
}

__global__ void scale_kernel(bf16* __restrict__ out, const bf16* __restrict__ in, float scale, size_t n) {
    grid_dependency_sync();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16(__bfloat162float(in[i]) * scale);
}

// Row argmax over bf16 logits, lowest index wins ties.  Stage 1: each CTA scans one
// 8192-entry chunk of a row with 16-byte loads; stage 2: one warp per row merges.
constexpr int AM_CHUNK = 8192;

__device__ __forceinline__ void am_better(float& best, int& bi, float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}

// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC 2011): a
// counter-based generator, so the noise of element i of row r at draw c is a pure function of (seed, r, c, i)
// and a sampled step is reproducible whatever the launch shape.
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

// Sampling parameters of the row pick: temperature <= 0 means plain argmax.  With a temperature the pick is
// argmax_i(logit_i / temperature + G_i), G_i independent standard Gumbel noise: the Gumbel-max form of drawing
// from softmax(logits / temperature) (what the reference does with torch.multinomial,
// cpmcu/speculative/tree_drafter.py:230-231), which keeps the two-stage argmax structure.
struct PickNoise {
    float inv_temperature;        // 0: no noise
    unsigned long long seed;
    const int32_t* draw;          // device counter of draws so far (may be null), plus
    int draw_add;
};

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
    const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1), 24 bits
    return -logf(-logf(u));
}

template <bool NOISY>
__global__ void argmax_partial_kernel(const bf16* __restrict__ logits, int vocab, int ld, int nchunk,
                                      float* __restrict__ pval, int* __restrict__ pidx, PickNoise noise) {
    grid_dependency_sync();
    __shared__ float sv[32];
    __shared__ int si[32];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const bf16* x = logits + static_cast<size_t>(row) * ld;
    const int begin = chunk * AM_CHUNK, end = min(begin + AM_CHUNK, vocab);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    const uint32_t draw = NOISY ? static_cast<uint32_t>((noise.draw ? *noise.draw : 0) + noise.draw_add) : 0u;
    const uint2 key = make_uint2(static_cast<uint32_t>(noise.seed), static_cast<uint32_t>(noise.seed >> 32));
    // value of element i: the logit, or logit / temperature + Gumbel noise; one Philox block serves 4 elements
    auto value4 = [&](const bf16* e, int i, float* out) {   // i a multiple of 4
        if constexpr (NOISY) {
            const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(i >> 2), static_cast<uint32_t>(row), draw, 0u), key);
            out[0] = __bfloat162float(e[0]) * noise.inv_temperature + gumbel_from_bits(r.x);
            out[1] = __bfloat162float(e[1]) * noise.inv_temperature + gumbel_from_bits(r.y);
            out[2] = __bfloat162float(e[2]) * noise.inv_temperature + gumbel_from_bits(r.z);
            out[3] = __bfloat162float(e[3]) * noise.inv_temperature + gumbel_from_bits(r.w);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = __bfloat162float(e[j]);
        }
    };
    auto value1 = [&](int i) -> float {
        const float v = __bfloat162float(x[i]);
        if constexpr (NOISY) {
            const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(i >> 2), static_cast<uint32_t>(row), draw, 0u), key);
            const uint32_t bits = (i & 3) == 0 ? r.x : (i & 3) == 1 ? r.y : (i & 3) == 2 ? r.z : r.w;
            return v * noise.inv_temperature + gumbel_from_bits(bits);
        }
        return v;
    };
    const bool aligned = ((reinterpret_cast<uintptr_t>(x + begin) & 15) == 0);
    if (aligned) {
        for (int i = begin + threadIdx.x * 8; i < end; i += blockDim.x * 8) {
            if (i + 8 <= end) {
                const uint4 v = *reinterpret_cast<const uint4*>(x + i);
                const bf16* e = reinterpret_cast<const bf16*>(&v);
                float f[8];
                value4(e, i, f);
                value4(e + 4, i + 4, f + 4);
#pragma unroll
                for (int j = 0; j < 8; ++j) am_better(best, bi, f[j], i + j);
            } else {
                for (int j = i; j < end; ++j) am_better(best, bi, value1(j), j);
            }
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) am_better(best, bi, value1(i), i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        am_better(best, bi, ov, oi);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = (lane < nw) ? sv[lane] : -INFINITY;
        bi = (lane < nw) ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            am_better(best, bi, ov, oi);
        }
        if (lane == 0) {
            pval[row * nchunk + chunk] = best;
            pidx[row * nchunk + chunk] = bi;
        }
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int nchunk,
                                    int32_t* __restrict__ out) {
    grid_dependency_sync();
    const int row = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < nchunk; c += 32) am_better(best, bi, pval[row * nchunk + c], pidx[row * nchunk + c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        am_better(best, bi, ov, oi);
    }
    if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;
}

}  // namespace

void launch_rms_norm(const bf16* x, int ldx, const bf16* w, bf16* y, int ldy, int rows, int dim, float eps,
                     cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0, "rms_norm: dims must be multiples of 8");
    CPM_REQUIRE(dim <= 256 * 8 * 8, "rms_norm: hidden size above 16384 is not supported");
    if (dim <= 256 * 8 * 2) {
        launch_kernel(rms_norm_kernel<false, 2>, dim3(rows), dim3(256), 0, s, const_cast<bf16*>(x), ldx,
                      static_cast<const bf16*>(nullptr), 1.f, w, y, ldy, dim, eps);
    } else {
        launch_kernel(rms_norm_kernel<false, 8>, dim3(rows), dim3(256), 0, s, const_cast<bf16*>(x), ldx,
                      static_cast<const bf16*>(nullptr), 1.f, w, y, ldy, dim, eps);
    }
}

void launch_add_rms_norm(bf16* x, const bf16* delta, float delta_scale, const bf16* w, bf16* y, int rows, int dim,
                         float eps, cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 8 == 0, "rms_norm: dim must be a multiple of 8");
    CPM_REQUIRE(dim <= 256 * 8 * 8, "rms_norm: hidden size above 16384 is not supported");
    if (dim <= 256 * 8 * 2) {
        // 512 threads, one 16-byte vector each: the shorter per-thread chain is worth 0.02 ms on the step
        launch_kernel(rms_norm_kernel<true, 1>, dim3(rows), dim3(512), 0, s, x, dim, delta, delta_scale, w, y, dim, dim, eps);
    } else {
        launch_kernel(rms_norm_kernel<true, 8>, dim3(rows), dim3(256), 0, s, x, dim, delta, delta_scale, w, y, dim, dim, eps);
    }
}

void launch_embedding(const int32_t* ids, const bf16* table, bf16* out, int ld_out, int rows, int dim, float scale,
                      cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 8 == 0 && ld_out % 8 == 0, "embedding: dim must be a multiple of 8");
    launch_kernel(embedding_kernel, dim3(rows), dim3(128), 0, s, ids, table, out, ld_out, dim, scale);
}

void launch_embedding_gather(const int32_t* ids, const bf16* table, bf16* out, int ld_out, int rows, int dim, float scale,
                             const bf16* h_rows, int h_ld, const int32_t* src, bf16* hid_out, int hid_ld,
                             cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 8 == 0 && ld_out % 8 == 0 && h_ld % 8 == 0 && hid_ld % 8 == 0,
                "embedding: dim and row strides must be multiples of 8");
    launch_kernel(embedding_gather_kernel, dim3(rows, 2), dim3(128), 0, s, ids, table, out, ld_out, dim, scale, h_rows, h_ld,
                  src, hid_out, hid_ld);
}

void launch_rope_append(bf16* qkv, int rows, int hq, int hkv, int d, const float* inv_freq, const int32_t* pos,
                        const int32_t* pos_base, int pos_off, int pos_step, bf16* k_cache, bf16* v_cache,
                        const int32_t* kv_len, int kv_off, const int32_t* n_valid, int cache_rows, cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(pos != nullptr || pos_base != nullptr, "rope: no positions given");
    CPM_REQUIRE(d % 4 == 0 && d <= 256, "rope: head_dim must be a multiple of 4 and at most 256");
    launch_kernel(rope_append_kernel, dim3(rows), dim3(256), 0, s, qkv, hq, hkv, d, inv_freq, pos, pos_base, pos_off,
                  pos_step, k_cache, v_cache, kv_len, kv_off, n_valid, cache_rows, runtime().d_error);
}

void launch_silu_gate(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t s, bool interleaved) {
    if (rows <= 0) return;
    CPM_REQUIRE(inter % 8 == 0, "silu_gate: width must be a multiple of 8");
    CPM_REQUIRE(!interleaved || inter % 64 == 0, "silu_gate: interleaved columns come in groups of 64");
    dim3 grid(ceil_div(inter / 8, 256), rows);
    launch_kernel(silu_gate_kernel, grid, dim3(256), 0, s, gate_up, out, inter, interleaved ? 1 : 0);
}

// ---------------------------------------------------------------- tile-major GEMM weights
namespace {

// element offset of (row, k) in a tile-major matrix with K columns
__device__ __forceinline__ size_t tile_major_offset(int row, int k, int K) {
    const size_t block = static_cast<size_t>(row >> 7) * (K >> 6) + (k >> 6);
    return block * (128 * 64) + static_cast<size_t>(row & 127) * 64 + (k & 63);
}

__device__ __forceinline__ int retile_dst_row(int r, int mode, int row_offset) {
    if (mode == 0) return row_offset + r;
    return (r >> 6) * 128 + (mode == 2 ? 64 : 0) + (r & 63);   // gate / up slot of the 64-feature group
}

// one thread per 8 elements (16 bytes) of the source; src holds rows [first_row, first_row + rows) of the matrix
__global__ void retile_rows_kernel(const bf16* __restrict__ src, int first_row, int rows, int src_cols,
                                   bf16* __restrict__ dst, int K, int mode, int row_offset, int k_offset) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int per_row = src_cols / 8;
    if (idx >= static_cast<size_t>(rows) * per_row) return;
    const int r = static_cast<int>(idx / per_row), c8 = static_cast<int>(idx - static_cast<size_t>(r) * per_row);
    const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * src_cols + c8 * 8);
    *reinterpret_cast<uint4*>(dst + tile_major_offset(retile_dst_row(first_row + r, mode, row_offset), k_offset + c8 * 8, K)) = v;
}

__global__ void gather_retiled_kernel(const bf16* __restrict__ src, const int32_t* __restrict__ idx, bf16* __restrict__ dst,
                                      int K) {
    const int d = blockIdx.x, s = idx[d];
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        *reinterpret_cast<uint4*>(dst + tile_major_offset(d, k, K)) = *reinterpret_cast<const uint4*>(src + tile_major_offset(s, k, K));
    }
}

}  // namespace

size_t linear_weight_elems(int N, int K) { return static_cast<size_t>(ceil_div(N, 128)) * 128 * K; }

void retile_weight_rows(const void* src, int rows, int src_cols, bf16* dst, int K, int mode, int row_offset, int k_offset,
                        cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(src_cols % 8 == 0 && K % 64 == 0 && k_offset % 8 == 0 && k_offset + src_cols <= K, "retile: bad column range");
    CPM_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || row_offset == 0), "retile: bad row mapping");
    cudaPointerAttributes attr = {};
    const bool on_device = cudaPointerGetAttributes(&attr, src) == cudaSuccess &&
                           (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
    cudaGetLastError();  // an unregistered host pointer is not an error here
    auto run = [&](const bf16* rows_on_device, int first_row, int n) {
        const size_t threads = static_cast<size_t>(n) * (src_cols / 8);
        retile_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(rows_on_device, first_row, n, src_cols, dst,
                                                                                      K, mode, row_offset, k_offset);
        CUDA_CHECK(cudaGetLastError());
    };
    if (on_device) {
        run(static_cast<const bf16*>(src), 0, rows);
        return;
    }
    // host memory: through a staging buffer, a slab of rows at a time
    const size_t row_bytes = static_cast<size_t>(src_cols) * 2;
    const int slab = static_cast<int>(std::max<size_t>(1, (static_cast<size_t>(64) << 20) / row_bytes));
    bf16* stage = nullptr;
    CUDA_CHECK(cudaMalloc(&stage, static_cast<size_t>(std::min(slab, rows)) * row_bytes));
    for (int r0 = 0; r0 < rows; r0 += slab) {
        const int n = std::min(slab, rows - r0);
        CUDA_CHECK(cudaMemcpyAsync(stage, static_cast<const uint8_t*>(src) + static_cast<size_t>(r0) * row_bytes,
                                   static_cast<size_t>(n) * row_bytes, cudaMemcpyHostToDevice, s));
        run(stage, r0, n);
        CUDA_CHECK(cudaStreamSynchronize(s));   // the staging buffer is reused
    }
    cudaFree(stage);
}

void gather_retiled_rows(const bf16* src, const int32_t* idx, int rows, bf16* dst, int K, cudaStream_t s) {
    if (rows <= 0) return;
    gather_retiled_kernel<<<rows, 128, 0, s>>>(src, idx, dst, K);
    CUDA_CHECK(cudaGetLastError());
}

void launch_add_scaled(bf16* x, const bf16* a, const bf16* b, float scale_b, int rows, int dim, cudaStream_t s) {
    if (rows <= 0) return;
    const size_t n = static_cast<size_t>(rows) * dim;
    launch_kernel(add_scaled_kernel, dim3(static_cast<unsigned>((n / 2 + 255) / 256)), dim3(256), 0, s, x, a, b, scale_b, n);
}

__global__ void add_bias_add_kernel(bf16* __restrict__ x, const bf16* __restrict__ a, const bf16* __restrict__ bias,
                                    const bf16* __restrict__ b, int dim, size_t n) {
    grid_dependency_sync();
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = __bfloat162float(a[i]);
    if (bias != nullptr) v = __bfloat162float(__float2bfloat16(v + __bfloat162float(bias[i % dim])));
    x[i] = __float2bfloat16(v + __bfloat162float(b[i]));
}

void launch_add_bias_add(bf16* x, const bf16* a, const bf16* bias, const bf16* b, int rows, int dim, cudaStream_t s) {
    const size_t n = static_cast<size_t>(rows) * dim;
    if (n == 0) return;
    launch_kernel(add_bias_add_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, x, a, bias, b, dim, n);
}

void launch_scale(bf16* out, const bf16* in, float scale, size_t n, cudaStream_t s) {
    if (n == 0) return;
    launch_kernel(scale_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, out, in, scale, n);
}

size_t argmax_workspace_bytes(int rows, int vocab) {
    return static_cast<size_t>(rows) * ceil_div(vocab, AM_CHUNK) * 8 + 256;
}

void launch_argmax(const bf16* logits, int rows, int vocab, int ld, int32_t* out, void* workspace, cudaStream_t s) {
    launch_sample(logits, rows, vocab, ld, out, workspace, 0.f, 0ull, nullptr, 0, s);
}

void launch_sample(const bf16* logits, int rows, int vocab, int ld, int32_t* out, void* workspace, float temperature,
                   unsigned long long seed, const int32_t* draw, int draw_add, cudaStream_t s) {
    if (rows <= 0) return;
    const int nchunk = ceil_div(vocab, AM_CHUNK);
    float* pval = static_cast<float*>(workspace);
    int* pidx = reinterpret_cast<int*>(pval + static_cast<size_t>(rows) * nchunk);
    PickNoise noise;
    noise.inv_temperature = temperature > 0.f ? 1.0f / temperature : 0.f;
    noise.seed = seed;
    noise.draw = draw;
    noise.draw_add = draw_add;
    if (temperature > 0.f) {
        launch_kernel(argmax_partial_kernel<true>, dim3(nchunk, rows), dim3(256), 0, s, logits, vocab, ld, nchunk, pval, pidx, noise);
    } else {
        launch_kernel(argmax_partial_kernel<false>, dim3(nchunk, rows), dim3(256), 0, s, logits, vocab, ld, nchunk, pval, pidx, noise);
    }
    launch_kernel(argmax_merge_kernel, dim3(rows), dim3(32), 0, s, static_cast<const float*>(pval),
                  static_cast<const int*>(pidx), nchunk, out);
}

// ------------------------------------------------------------------ allocation-free argmax
// Scratch of cpmcu_argmax_noalloc(): the stage-1 (value, index) partials.  It lives in the
// library image, so every GPU that loads the library holds these 16 KB until the process exits.
constexpr int NOALLOC_MAX_ROWS = 64;
constexpr int NOALLOC_MAX_VOCAB = 32 * AM_CHUNK;  // 262144
constexpr size_t NOALLOC_SCRATCH_BYTES = static_cast<size_t>(NOALLOC_MAX_ROWS) * 32 * 8;
static __device__ __align__(256) unsigned char g_argmax_scratch[NOALLOC_SCRATCH_BYTES];

extern "C" int cpmcu_argmax_noalloc(const void* logits, int rows, int vocab, int32_t* out) {
    // In host code `g_argmax_scratch` is only a handle for the symbol, not a device pointer:
    // the address the kernels need is looked up once per device, with that device current.
    static void* scratch_addr[64] = {nullptr};
    if (logits == nullptr || out == nullptr) {
        cpm_set_error("cpmcu_argmax_noalloc: null pointer");
        return -1;
    }
    if (rows < 1 || rows > NOALLOC_MAX_ROWS || vocab < 1 || vocab > NOALLOC_MAX_VOCAB) {
        cpm_set_error("cpmcu_argmax_noalloc: at most 64 rows and 262144 columns fit the built-in scratch; "
                      "use cpmcu_argmax for larger inputs");
        return -1;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        cpm_set_error("cpmcu_argmax_noalloc: no usable CUDA device is current");
        return -1;
    }
    if (scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_argmax_scratch);
        if (e != cudaSuccess || p == nullptr) {
            cpm_set_error((std::string("cpmcu_argmax_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e)).c_str());
            return -1;
        }
        scratch_addr[dev] = p;
    }
    const int nchunk = ceil_div(vocab, AM_CHUNK);
    float* pval = static_cast<float*>(scratch_addr[dev]);
    int* pidx = reinterpret_cast<int*>(pval + static_cast<size_t>(rows) * nchunk);
    // Both stages overwrite every scratch word they later read, so nothing has to be cleared.
    argmax_partial_kernel<false><<<dim3(nchunk, rows), 256, 0, cudaStreamLegacy>>>(static_cast<const bf16*>(logits), vocab,
                                                                                   vocab, nchunk, pval, pidx, PickNoise{});
    argmax_merge_kernel<<<rows, 32, 0, cudaStreamLegacy>>>(pval, pidx, nchunk, out);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(cudaStreamLegacy);
    if (e != cudaSuccess) {
        cpm_set_error((std::string("cpmcu_argmax_noalloc: ") + cudaGetErrorString(e)).c_str());
        return -1;
    }
    return 0;
}
