// InfLLM-v2 block selection (sparse_select.cu): buffers and launchers.
#pragma once
#include "common.cuh"

// Arguments of init_minicpm4_model (reference src/entry.cu:138-158).
struct SparseConfig {
    bool enabled = false;
    int sink_blocks = 1;      // sink_window_size: leading 64-token blocks always selected
    int window_blocks = 32;   // block_window_size: trailing 64-token blocks always visited
    int topk = 64;            // sparse_topk_k
    int sparse_switch = 8192; // selection starts once the compressed cache covers this many tokens
    bool compress_lse = true; // normalise stage-1 scores by the log-sum-exp over the c2 cache
};

struct SparseBuffers {
    bf16* c1 = nullptr;          // [layers][budget / 16][kv_dim]  means of 32 keys every 16
    size_t c1_layer_stride = 0;  // elements
    bf16* c2 = nullptr;          // [layers][budget / 64][kv_dim]  means of 128 keys every 64 (compress_lse only)
    size_t c2_layer_stride = 0;
    int32_t* done = nullptr;     // [2] entries of c1 / c2 computed so far (same for every layer)
    float2* lse = nullptr;       // [hkv][max_tokens][16][score_ld / 128]  (max, exp-sum) per 128-key chunk of the LSE keys
    bf16* scores = nullptr;      // [hkv][max_tokens][score_ld]  stage-1 scores of the layer being run
    int score_ld = 0;
    uint64_t* blockmask = nullptr;  // [hkv][max_tokens][bm_words]
    int bm_words = 0;
    int max_tokens = 0;
};

// Bring the compressed caches of all layers up to the L = *kv_len + kv_add accepted rows
// (max_new = upper bound on entries added since the previous call).
void launch_sparse_compress(const SparseBuffers& b, bf16* const* caches, int layers, int kv_dim, const int32_t* kv_len,
                            int kv_add, int max_new, cudaStream_t s);

// Stage-1 scores of `T` query rows against the layer's compressed keys, then max-pool / top-k /
// bitmask into b.blockmask ([hkv][T][bm_words], all ones while selection is not active).
void launch_sparse_select(const SparseBuffers& b, const SparseConfig& cfg, int layer, const bf16* q, int q_ld, int T,
                          int hq, int hkv, const int32_t* kv_len, int kv_add, const int32_t* n_valid, cudaStream_t s);
