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
template <bool ADD>
__global__ void rms_norm_kernel(bf16* __restrict__ x, int ldx, const bf16* __restrict__ delta, float delta_scale,
                                const bf16* __restrict__ w, bf16* __restrict__ y, int ldy, int dim, float eps) {
    grid_dependency_sync();
    __shared__ float sh[32];
    const size_t base = static_cast<size_t>(blockIdx.x) * ldx;
    const size_t dbase = static_cast<size_t>(blockIdx.x) * dim;
    const size_t ybase = static_cast<size_t>(blockIdx.x) * ldy;
    float ss = 0.f;
    for (int i = threadIdx.x * 2; i < dim; i += blockDim.x * 2) {
        __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + base + i);
        if (ADD) {
            __nv_bfloat162 dl = *reinterpret_cast<const __nv_bfloat162*>(delta + dbase + i);
            if (delta_scale != 1.0f) {
                dl.x = __float2bfloat16(__bfloat162float(dl.x) * delta_scale);
                dl.y = __float2bfloat16(__bfloat162float(dl.y) * delta_scale);
            }
            v.x = __float2bfloat16(__bfloat162float(v.x) + __bfloat162float(dl.x));
            v.y = __float2bfloat16(__bfloat162float(v.y) + __bfloat162float(dl.y));
            *reinterpret_cast<__nv_bfloat162*>(x + base + i) = v;
        }
        const float a = __bfloat162float(v.x), b = __bfloat162float(v.y);
        ss += a * a + b * b;
    }
    ss = block_sum(ss, sh);
    const float rs = rsqrtf(ss / dim + eps);
    for (int i = threadIdx.x * 2; i < dim; i += blockDim.x * 2) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + base + i);
        const __nv_bfloat162 ww = *reinterpret_cast<const __nv_bfloat162*>(w + i);
        __nv_bfloat162 o;
        o.x = __float2bfloat16(rs * __bfloat162float(v.x) * __bfloat162float(ww.x));
        o.y = __float2bfloat16(rs * __bfloat162float(v.y) * __bfloat162float(ww.y));
        *reinterpret_cast<__nv_bfloat162*>(y + ybase + i) = o;
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

// One CTA per token row.  q heads rotate in place; k heads rotate into the
// cache; v heads are copied into the cache.
__global__ void rope_append_kernel(bf16* __restrict__ qkv, int hq, int hkv, int d, const float* __restrict__ inv_freq,
                                   const int32_t* __restrict__ pos, const int32_t* __restrict__ pos_base, int pos_off,
                                   int pos_step, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                   const int32_t* __restrict__ kv_len, int kv_off,
                                   const int32_t* __restrict__ n_valid) {
    grid_dependency_sync();
    const int r = blockIdx.x;
    const int half = d >> 1;
    const int ld = (hq + 2 * hkv) * d;
    bf16* row = qkv + static_cast<size_t>(r) * ld;
    const int p = (pos != nullptr) ? pos[r] : (*pos_base + pos_off + r * pos_step);
    const bool store_kv = (n_valid == nullptr) || (r < *n_valid);
    const long long kv_row = static_cast<long long>(*kv_len) + kv_off + r;
    const int kv_dim = hkv * d;
    for (int i = threadIdx.x; i < (hq + hkv) * half; i += blockDim.x) {
        const int h = i / half, c = i - h * half;
        const float freq = p * inv_freq[c];
        float sn, cs;
        sincosf(freq, &sn, &cs);
        bf16* hp = row + h * d;
        const float a = __bfloat162float(hp[c]);
        const float b = __bfloat162float(hp[c + half]);
        const bf16 o1 = __float2bfloat16(a * cs - b * sn);
        const bf16 o2 = __float2bfloat16(a * sn + b * cs);
        if (h < hq) {
            hp[c] = o1;
            hp[c + half] = o2;
        } else if (store_kv && kv_row >= 0) {
            bf16* kd = k_cache + kv_row * kv_dim + (h - hq) * d;
            kd[c] = o1;
            kd[c + half] = o2;
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

__global__ void silu_gate_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter) {
    grid_dependency_sync();
    const int r = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (c >= inter) return;
    const bf16* g = gate_up + static_cast<size_t>(r) * 2 * inter;
    const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(g + c);
    const __nv_bfloat162 uv = *reinterpret_cast<const __nv_bfloat162*>(g + inter + c);
    __nv_bfloat162 o;
    {
        const float x = __bfloat162float(gv.x);
        o.x = __float2bfloat16(x * (1.0f / (1.0f + expf(-x))) * __bfloat162float(uv.x));
    }
    {
        const float x = __bfloat162float(gv.y);
        o.y = __float2bfloat16(x * (1.0f / (1.0f + expf(-x))) * __bfloat162float(uv.y));
    }
    *reinterpret_cast<__nv_bfloat162*>(out + static_cast<size_t>(r) * inter + c) = o;
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

// Row argmax over bf16 logits, lowest index wins ties.
__global__ void argmax_kernel(const bf16* __restrict__ logits, int vocab, int ld, int32_t* __restrict__ out) {
    grid_dependency_sync();
    __shared__ float sv[32];
    __shared__ int si[32];
    const bf16* row = logits + static_cast<size_t>(blockIdx.x) * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = __bfloat162float(row[i]);
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
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
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
}

}  // namespace

void launch_rms_norm(const bf16* x, int ldx, const bf16* w, bf16* y, int ldy, int rows, int dim, float eps,
                     cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 2 == 0 && ldx % 2 == 0 && ldy % 2 == 0, "rms_norm: dims must be even");
    launch_kernel(rms_norm_kernel<false>, dim3(rows), dim3(256), 0, s, const_cast<bf16*>(x), ldx, nullptr, 1.f, w, y, ldy, dim, eps);
}

void launch_add_rms_norm(bf16* x, const bf16* delta, float delta_scale, const bf16* w, bf16* y, int rows, int dim,
                         float eps, cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 2 == 0, "rms_norm: dim must be even");
    launch_kernel(rms_norm_kernel<true>, dim3(rows), dim3(256), 0, s, x, dim, delta, delta_scale, w, y, dim, dim, eps);
}

void launch_embedding(const int32_t* ids, const bf16* table, bf16* out, int ld_out, int rows, int dim, float scale,
                      cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(dim % 8 == 0 && ld_out % 8 == 0, "embedding: dim must be a multiple of 8");
    launch_kernel(embedding_kernel, dim3(rows), dim3(128), 0, s, ids, table, out, ld_out, dim, scale);
}

void launch_rope_append(bf16* qkv, int rows, int hq, int hkv, int d, const float* inv_freq, const int32_t* pos,
                        const int32_t* pos_base, int pos_off, int pos_step, bf16* k_cache, bf16* v_cache,
                        const int32_t* kv_len, int kv_off, const int32_t* n_valid, cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(pos != nullptr || pos_base != nullptr, "rope: no positions given");
    launch_kernel(rope_append_kernel, dim3(rows), dim3(256), 0, s, qkv, hq, hkv, d, inv_freq, pos, pos_base, pos_off,
                  pos_step, k_cache, v_cache, kv_len, kv_off, n_valid);
}

void launch_silu_gate(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t s) {
    if (rows <= 0) return;
    CPM_REQUIRE(inter % 2 == 0, "silu_gate: width must be even");
    dim3 grid(ceil_div(inter / 2, 256), rows);
    launch_kernel(silu_gate_kernel, grid, dim3(256), 0, s, gate_up, out, inter);
}

void launch_add_scaled(bf16* x, const bf16* a, const bf16* b, float scale_b, int rows, int dim, cudaStream_t s) {
    if (rows <= 0) return;
    const size_t n = static_cast<size_t>(rows) * dim;
    launch_kernel(add_scaled_kernel, dim3(static_cast<unsigned>((n / 2 + 255) / 256)), dim3(256), 0, s, x, a, b, scale_b, n);
}

void launch_scale(bf16* out, const bf16* in, float scale, size_t n, cudaStream_t s) {
    if (n == 0) return;
    launch_kernel(scale_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, s, out, in, scale, n);
}

void launch_argmax(const bf16* logits, int rows, int vocab, int ld, int32_t* out, cudaStream_t s) {
    if (rows <= 0) return;
    launch_kernel(argmax_kernel, dim3(rows), dim3(1024), 0, s, logits, vocab, ld, out);
}
