// TEST INFRASTRUCTURE, not product code: C entry points around the reference project's OWN attention
// code, src/flash_attn (its FlashAttention fork: split-KV kernel with the 64-bit tree mask, block-window
// iterator, block-sparse head-group mode and the stage-1 scoring kernel).  oracle/build_ref.py compiles the
// reference's four head_dim-128 bf16 translation units and src/flash_attn/flash_api.hpp where they lie,
// with the CUTLASS headers that ship inside this image's Python packages standing in for the reference's
// empty src/cutlass submodule, into oracle/_ref/libcpmcu_ref_flash.so.  Nothing is copied into this tree.
//
//   refk_mha_fwd_kvcache   mha_fwd_kvcache   (src/flash_attn/flash_api.hpp:292-392) with the argument
//                          values of Attention::decode / ::prefill (src/model/attn.cuh:135-234) and of
//                          MiniCPM4Attention::decode (src/model/minicpm4/minicpm4_attn.cuh:291-318)
//   refk_mha_fwd_stage1    mha_fwd_stage1    (flash_api.hpp:204-290) as called at minicpm4_attn.cuh:236-258
//
// Every function takes device pointers, runs on the default stream, synchronises and returns the CUDA
// error code (0 = success).
#include <cstdint>
#include <cuda_runtime.h>

#include "flash_attn/flash_api.hpp"

namespace {
int finish() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return int(e);
}
// scratch of the split kernel, sized as Attention::init_output_ptr does (src/model/attn.cuh:101-111)
struct Scratch {
    float *lse = nullptr, *lse_accum = nullptr, *oaccum = nullptr;
    size_t rows = 0;
};
Scratch& scratch(int tokens, int heads, int head_dim) {
    static Scratch s;
    const size_t need = size_t(tokens > 128 * 64 ? tokens : 128 * 64) * heads;
    if (need > s.rows) {
        cudaFree(s.lse);
        cudaFree(s.lse_accum);
        cudaFree(s.oaccum);
        cudaMalloc(&s.lse, need * sizeof(float));
        cudaMalloc(&s.lse_accum, need * sizeof(float));
        cudaMalloc(&s.oaccum, need * head_dim * sizeof(float));
        s.rows = need;
    }
    return s;
}
}  // namespace

extern "C" {

// q [tokens, hq, 128] contiguous; k_cache / v_cache [>= seqlen_k, hkv, 128]; out [tokens, hq, 128].
// cache_length: device int32 (keys visible, the new rows included) or null — with null the kernel runs
// unsplit over seqlen_k keys (the prefill call), otherwise with the reference's fixed 16 splits.
// mask: device uint64[tokens] tree mask over the last mask_k keys (the verify pass gives mask_k = tokens, a
// draft level k * level: Mask(ptr, q_range, k_range) at src/model/model.cuh:156 and
// src/model/minicpm4/minicpm4_eagle.cuh:359) or null; blockmask: device uint64 block masks or null;
// block_window_size: the draft layer's sliding window in tokens when blockmask is null, the local window in
// 64-key blocks when it is not.
int refk_mha_fwd_kvcache(int tokens, int seqlen_k, int hq, int hkv, void* q, void* k_cache, void* v_cache,
                         int32_t* cache_length, uint64_t* mask, int mask_k, void* out, uint64_t* blockmask,
                         int block_window_size) {
    Scratch& s = scratch(tokens, hq, 128);
    mha_fwd_kvcache(true, 1, tokens, seqlen_k, hq, hkv, 128, q, k_cache, v_cache, cache_length,
                    Mask(mask, tokens, mask_k), out, s.lse, s.lse_accum, s.oaccum, rsqrtf(128.f), true, -1, -1, 0,
                    nullptr, blockmask, block_window_size);
    return finish();
}

// q [tokens, hq, 128]; c1 [c1_len, hkv, 128] (keys that are scored); c2 [c2_len, hkv, 128] (keys that give
// the softmax normaliser; pass c1 again for apply_compress_lse = false).  scores: bf16
// [hkv, q_round, k_round]; the two rounded extents are returned through q_round / k_round.
int refk_mha_fwd_stage1(int tokens, int c1_len, int c2_len, int hq, int hkv, void* q, void* c1, void* c2,
                        void* scores, int* q_round, int* k_round) {
    int qr = 0, kr = 0;
    mha_fwd_stage1(true, 1, tokens, c1_len, c2_len, hq, hkv, 128, q, c1, c2, nullptr, scores, rsqrtf(128.f), false,
                   -1, -1, 0, nullptr, qr, kr);
    *q_round = qr;
    *k_round = kr;
    return finish();
}

// Timed loop of the decode-shaped call for the per-kernel timing table (same launch repeated; the K/V
// tensors of one layer stay in L2 as they do between the layers' own launches only partly, so the caller
// passes `copies` separate caches that are visited round robin).
int refk_bench_mha_fwd_kvcache(int tokens, int seqlen_k, int hq, int hkv, void* q, void** k_caches, void** v_caches,
                               int copies, int32_t* cache_length, uint64_t* mask, void* out, int iters, float* avg_us) {
    Scratch& s = scratch(tokens, hq, 128);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int it = -3; it < iters; ++it) {
        if (it == 0) cudaEventRecord(e0, nullptr);
        const int c = ((it % copies) + copies) % copies;
        mha_fwd_kvcache(true, 1, tokens, seqlen_k, hq, hkv, 128, q, k_caches[c], v_caches[c], cache_length,
                        Mask(mask, tokens, tokens), out, s.lse, s.lse_accum, s.oaccum, rsqrtf(128.f), true, -1, -1, 0,
                        nullptr, nullptr, 0);
    }
    cudaEventRecord(e1, nullptr);
    int rc = finish();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    *avg_us = ms * 1000.f / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

}  // extern "C"
