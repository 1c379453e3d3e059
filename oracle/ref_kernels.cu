// TEST INFRASTRUCTURE, not product code: C entry points around the reference project's OWN device
// kernels, compiled from the reference's headers where they lie (never copied into this tree) by
// oracle/build_ref.py into oracle/_ref/libcpmcu_ref_kernels.so.  The parity tests run these on the
// same inputs as the library and as the CPU oracle, which pins both against the reference itself
// for every stage whose source compiles from the reference's own files:
//
//   draft tree from given logits   log_softmax, TopK (bitonic), cumsum, set_parent, update_tree,
//                                  remap_id(_fr), build_dynamic_tree — composed in the order of
//                                  MiniCPM4EagleImpl::draft (src/model/minicpm4/minicpm4_eagle.cuh:304-398)
//   verify + KV compaction         verify_draft, fix_kv_cache (src/model/tree_drafter.cuh:5-101),
//                                  composed as MiniCPM4EagleImpl::verify (minicpm4_eagle.cuh:400-418)
//   block selection, integer part  meanpooling, maxpooling_func, TopK, topk_to_uint64_func
//                                  (src/model/minicpm4/minicpm4_kvcache.cuh), composed as
//                                  MiniCPM4Attention::decode (minicpm4_attn.cuh:226-290)
//   row-wise float kernels         rms_norm / add_and_rms_norm (norm.cuh), rotary_embedding (rotary.cuh),
//                                  gated_silu_interleaved (activation.cuh), embedding (embedding.cuh)
//   linear                         linear<T> = cublasGemmEx (linear.cuh:8-37)
//
// Attention (src/flash_attn) is not here: it needs the un-vendored CUTLASS tree.
// eagle.cuh's own #include list pulls that attention code in, so its kernel section (everything
// before `struct Skip`) is cut out at build time into the build folder as eagle_kernels.inc.
//
// Every function takes device pointers, runs on the default stream, synchronises and returns the
// CUDA error code (0 = success).
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>
#include <cassert>
#include "utils.cuh"
#include "trait.cuh"
#include "model/memory.cuh"
#include "model/tree_drafter.cuh"
#include "model/topk.cuh"
#include "model/norm.cuh"
#include "model/rotary.cuh"
#include "model/activation.cuh"
#include "model/embedding.cuh"
#include "model/elementwise.cuh"
#include "model/linear.cuh"
#include "model/minicpm4/minicpm4_kvcache.cuh"
#include "eagle_kernels.inc"

using bf16 = __nv_bfloat16;

namespace {

Stream ref_stream() {
    static Stream s = [] {
        Stream t;
        t.stream = nullptr;
        cublasCreate(&t.cublas_handle);
        return t;
    }();
    return s;
}

// The reference's functors carve their buffers out of its Memory pool; one small pool serves all calls
// (re-carved from offset 0 by every call).
Memory* ref_pool() {
    static Memory* m = new Memory(0.004f);
    return m;
}

int finish() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return int(e);
}

template <typename T>
int64_t carve(Memory* m, T** p, int64_t off, size_t count) {
    return m->allocate((void**)p, off, count * sizeof(T));
}

}  // namespace

extern "C" {

// Same argument list as the library's cpmcu_draft_tree_from_logits.  logits: [1 + (num_iter-1)*k, vocab]
// bf16 (row 0 = level 0; level d uses rows 1 + (d-1)*k ..).  A copy is log-softmaxed in place as the
// reference does with its eagle_logits buffer.
int refk_draft_tree_from_logits(const void* logits, int vocab, int k, int num_iter, int tree_size,
                                const int32_t* token_id_remap, const int32_t* cache_length, int32_t* tree_ids,
                                int32_t* tree_pos, uint64_t* tree_mask, int32_t* tree_parent, void* tried_val_out,
                                int32_t* tried_pos, int32_t* tried_parent) {
    const Stream S = ref_stream();
    Memory* mem = ref_pool();
    const int total_tried = k * k * (num_iter - 1) + k;
    const int rows = 1 + (num_iter - 1) * k;
    bf16* tried_val = (bf16*)tried_val_out;
    functions::TopK<bf16> t1(vocab, k), t2(total_tried, tree_size - 1);
    bf16* lg;
    uint64_t *mask_2d, *tmp_mask_2d;
    char* spill;
    int64_t off = 0;
    off = carve(mem, &lg, off, size_t(rows) * vocab);
    off = carve(mem, &mask_2d, off, 64);
    off = carve(mem, &tmp_mask_2d, off, 64);
    off = t1.init_output_ptr(mem, k, off);
    off = t2.init_output_ptr(mem, 1, off);
    off = carve(mem, &spill, off, 1024);   // the second 32-wide pass of TopK writes up to entry 63 of 59-entry outputs
    if (off < 0) return -1;
    int32_t L = 0;
    cudaMemcpy(&L, cache_length, sizeof(int32_t), cudaMemcpyDeviceToHost);
    cudaMemcpy(lg, logits, size_t(rows) * vocab * sizeof(bf16), cudaMemcpyDeviceToDevice);
    const bool fr = token_id_remap != nullptr;
    {   // d = 0
        log_softmax(S, 1, vocab, lg);
        t1.prefill(S, 1, lg);
        cudaMemcpy(tried_val, t1.topk_val, k * sizeof(bf16), cudaMemcpyDeviceToDevice);
        cudaMemcpy(tried_pos, t1.topk_pos, k * sizeof(int32_t), cudaMemcpyDeviceToDevice);
        if (fr) remap(S, k, t1.topk_pos, t2.topk_pos, token_id_remap);
        else cudaMemcpy(t2.topk_pos, t1.topk_pos, k * sizeof(int32_t), cudaMemcpyDeviceToDevice);
        cudaMemcpy(t2.topk_val, t1.topk_val, k * sizeof(bf16), cudaMemcpyDeviceToDevice);
        init_tree(S, k, mask_2d);
    }
    for (int d = 1; d < num_iter; ++d) {
        bf16* lrow = lg + size_t(1 + (d - 1) * k) * vocab;
        log_softmax(S, k, vocab, lrow);
        t1.prefill(S, k, lrow);
        cumsum(S, k, k, t1.topk_val, t2.topk_val);
        cudaMemcpy(tried_val + k + (d - 1) * k * k, t1.topk_val, k * k * sizeof(bf16), cudaMemcpyDeviceToDevice);
        cudaMemcpy(tried_pos + k + (d - 1) * k * k, t1.topk_pos, k * k * sizeof(int32_t), cudaMemcpyDeviceToDevice);
        t2.prefill(S, 1, t1.topk_val, k * k, k);
        cudaMemcpy(tmp_mask_2d, mask_2d, k * sizeof(uint64_t), cudaMemcpyDeviceToDevice);
        set_parent(S, k, tried_parent + (d - 1) * k, t2.topk_pos, k + (d - 1) * k * k);
        update_tree(S, k, k * d, mask_2d, tmp_mask_2d, t2.topk_pos);
        if (fr) remap_id_fr(S, k, t2.topk_pos, t1.topk_pos, token_id_remap);
        else remap_id(S, k, t2.topk_pos, t1.topk_pos);
    }
    t2.prefill(S, 1, tried_val);
    try {
        build_dynamic_tree(S, tree_size, L, k, tried_parent, t2.topk_pos, tree_pos, tree_mask, tree_parent);
    } catch (const std::exception&) {
        return -2;
    }
    if (fr) remap_id_fr(S, tree_size - 1, t2.topk_pos, tried_pos, token_id_remap, tree_ids + 1);
    else remap_id(S, tree_size - 1, t2.topk_pos, tried_pos, tree_ids + 1);
    return finish();
}

// Same argument list as the library's cpmcu_verify_and_compact.  result (device, 2 + max_accept ints):
// [0] accept length, [1] best node, [2..] accepted path (tree indices, root first); pred[0:n] receives
// the emitted tokens as fix_kvcache_kernel_2 leaves them.
int refk_verify_and_compact(int tree_size, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                            const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent,
                            void* const* caches, int num_caches, int kv_dim, int max_accept, int32_t* result) {
    const Stream S = ref_stream();
    Memory* mem = ref_pool();
    int32_t* d_best;
    bf16* tmp;
    int64_t off = 0;
    off = carve(mem, &d_best, off, 4);
    off = carve(mem, &tmp, off, size_t(64) * num_caches * kv_dim);
    if (off < 0) return -1;
    verify_draft(S, tree_size, pred, gt, position_ids, cache_length, attn_mask, tree_parent, d_best);
    int32_t h_best[2] = {0, 0};
    cudaMemcpy(h_best, d_best, sizeof(h_best), cudaMemcpyDeviceToHost);
    const int n = h_best[0];
    if (n < 1 || n > max_accept || n > 64) return -3;
    cudaMemcpy(result, d_best, 2 * sizeof(int32_t), cudaMemcpyDeviceToDevice);
    cudaMemcpy(result + 2, pred, n * sizeof(int32_t), cudaMemcpyDeviceToDevice);
    fix_kv_cache<bf16>(S, n, num_caches, kv_dim, pred, gt, cache_length, (bf16**)caches, tmp);
    return finish();
}

// MiniCPM4KVCache::compress from an empty compressed cache: c1 = mean over 32 keys every 16,
// c2 = mean over 128 keys every 64 (c2 may be null).  Returns the error code; lengths follow
// max((kv_len - stride) / stride, 0).
int refk_compress(const void* k_cache, int kv_len, int kv_dim, void* c1, void* c2) {
    const Stream S = ref_stream();
    const int n1 = max((kv_len - 16) / 16, 0), n2 = max((kv_len - 64) / 64, 0);
    meanpooling<bf16>(S, 0, n1, kv_dim, (bf16*)c1, (const bf16*)k_cache, 16);
    if (c2) meanpooling<bf16>(S, 0, n2, kv_dim, (bf16*)c2, (const bf16*)k_cache, 64);
    return finish();
}

// The integer part of the block selection, from stage-1 scores [hkv][q_round][k_round] (bf16):
// maxpooling_func -> TopK(4096, topk)::prefill(dim = out_len) -> topk_to_uint64_func, with the arguments
// MiniCPM4Attention::decode passes.  pool_out: [hkv][tq][out_len] bf16 (out_len = ceil(cache_len / 64));
// blockmask: [hkv * tq][ceil(ceil(padded_length / 64) / 64)] uint64.
int refk_select_from_scores(const void* scores, int hkv, int tq, int q_round, int k_round, int cache_len,
                            int sink_blocks, int window_blocks, int topk, int padded_length, void* pool_out,
                            uint64_t* blockmask) {
    const Stream S = ref_stream();
    Memory* mem = ref_pool();
    int out_len = 0;
    const int max_blocks = max(4096, (cache_len + 63) / 64);
    functions::TopK<bf16> tk(max_blocks, topk);
    char* spill;
    int64_t off = tk.init_output_ptr(mem, hkv * tq, 0);
    off = carve(mem, &spill, off, 1024);
    if (off < 0) return -1;
    maxpooling_func<bf16>(S.stream, (const bf16*)scores, (bf16*)pool_out, hkv, tq, q_round, k_round, cache_len,
                          sink_blocks, window_blocks, out_len);
    tk.prefill(S, hkv * tq, (const bf16*)pool_out, out_len);
    topk_to_uint64_func(S.stream, tk.topk_pos, blockmask, hkv * tq, tk.top, padded_length);
    return finish();
}

int refk_rms_norm(const void* input, const void* weight, void* output, int rows, int dim, float eps) {
    rms_norm<bf16>(ref_stream(), rows, dim, (const bf16*)input, (const bf16*)weight, (bf16*)output, eps);
    return finish();
}

// input += prev_output (kept), output = norm(input) * weight
int refk_add_and_rms_norm(void* input, const void* prev_output, const void* weight, void* output, int rows, int dim,
                          float eps) {
    add_and_rms_norm<bf16>(ref_stream(), rows, dim, (bf16*)input, (const bf16*)prev_output, (const bf16*)weight,
                           (bf16*)output, eps);
    return finish();
}

// q: [rows][hq*head_dim], k: [rows][hkv*head_dim], both contiguous, rotated in place
int refk_rotary(void* q, void* k, int rows, int hq, int hkv, int head_dim, const float* inv_freq, const int32_t* pos) {
    rotary_embedding<bf16>(ref_stream(), rows, hq, hkv, head_dim / 2, inv_freq, pos, (bf16*)q, (bf16*)k);
    return finish();
}

// gate_up: [rows][2*inter] (gate columns first), out: [rows][inter]
int refk_gated_silu(const void* gate_up, void* out, int rows, int inter) {
    gated_silu_interleaved<bf16>(ref_stream(), rows, inter, (const bf16*)gate_up, (bf16*)out);
    return finish();
}

int refk_embedding(const int32_t* ids, const void* table, void* out, int rows, int hidden) {
    embedding<bf16>(ref_stream(), rows, hidden, ids, (const bf16*)table, (bf16*)out);
    return finish();
}

// y[M][N] = x[M][K] * w[N][K]^T through the reference's cuBLAS call
int refk_linear(const void* x, const void* w, void* y, int M, int N, int K) {
    linear<bf16>(ref_stream(), M, K, N, (const bf16*)x, (const bf16*)w, (bf16*)y);
    return finish();
}

// Times `iters` back-to-back calls of the reference's linear<T> (cuBLAS) with CUDA events, cycling through
// `copies` weight buffers so that the weights come from HBM and not from L2.  avg_us: host float.
int refk_bench_linear(int M, int N, int K, int copies, int iters, float* avg_us) {
    const Stream S = ref_stream();
    bf16 *x = nullptr, *y = nullptr, *w = nullptr;
    const size_t wn = size_t(N) * K;
    if (cudaMalloc(&x, size_t(M) * K * 2) != cudaSuccess || cudaMalloc(&y, size_t(M) * N * 2) != cudaSuccess ||
        cudaMalloc(&w, wn * copies * 2) != cudaSuccess)
        return int(cudaGetLastError());
    cudaMemset(x, 0x3c, size_t(M) * K * 2);
    cudaMemset(w, 0x3c, wn * copies * 2);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int i = 0; i < 3; ++i) linear<bf16>(S, M, K, N, x, w + wn * (i % copies), y);
    cudaEventRecord(e0, S.stream);
    for (int i = 0; i < iters; ++i) linear<bf16>(S, M, K, N, x, w + wn * (i % copies), y);
    cudaEventRecord(e1, S.stream);
    const int rc = finish();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    *avg_us = ms * 1000.f / iters;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(x);
    cudaFree(y);
    cudaFree(w);
    return rc;
}

// In-place log-softmax over rows of `dim` bf16 values, then the reference's top-k of each row.
int refk_log_softmax_topk(void* logits, int rows, int dim, int top, void* out_val, int32_t* out_pos) {
    const Stream S = ref_stream();
    Memory* mem = ref_pool();
    functions::TopK<bf16> tk(dim, top);
    char* spill;
    int64_t off = tk.init_output_ptr(mem, rows, 0);
    off = carve(mem, &spill, off, 1024);
    if (off < 0) return -1;
    log_softmax(S, rows, dim, (bf16*)logits);
    tk.prefill(S, rows, (const bf16*)logits);
    cudaMemcpy(out_val, tk.topk_val, size_t(rows) * top * sizeof(bf16), cudaMemcpyDeviceToDevice);
    cudaMemcpy(out_pos, tk.topk_pos, size_t(rows) * top * sizeof(int32_t), cudaMemcpyDeviceToDevice);
    return finish();
}

}  // extern "C"
