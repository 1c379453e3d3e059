/* C ABI of libcpmcu_b200.so: the speculative-decoding hot path of CPM.cu
 * (EAGLE draft loop -> tree build -> tree-verify forward -> greedy acceptance
 * with KV compaction) as sm_100a CUDA.
 *
 * Part 1 declares, one for one, the functions the reference binds into its
 * `cpmcu.C` Python module (src/entry.cu:510-535).  Arguments keep the
 * reference's order and meaning; pointers that the reference passes as
 * uintptr_t are plain pointers here.  Unless stated otherwise pointers are
 * DEVICE memory.  Functions that return void in the reference return 0 on
 * success and -1 on failure here (message via cpmcu_last_error()).
 *
 * Part 2 is the fused step (one CUDA graph per speculative step, no host
 * round trips inside the step).  Part 3 exposes the individual kernels so each
 * can be checked in isolation against the CPU oracle.
 *
 * bf16 values are passed as void* (16-bit storage, row-major).
 * There is no CPU path: every call fails with an error if no sm_100 device is
 * visible.
 */
#ifndef CPMCU_B200_H
#define CPMCU_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ part 1 */

/* Message of the last failure on the calling thread ("" if none). */
const char* cpmcu_last_error(void);

/* reference: init_base_model, src/entry.cu:100-136.  torch_dtype: 1 = bf16
 * (0 = fp16 is rejected: this library computes in bf16 only). */
int cpmcu_init_base_model(float memory_limit, int vocab_size, int num_hidden_layers, int hidden_size,
                          int intermediate_size, int num_attention_heads, int num_key_value_heads, int head_dim,
                          float rms_norm_eps, int torch_dtype, int chunk_length, float scale_embed,
                          float scale_lmhead, float scale_residual);

/* reference: init_minicpm4_model, src/entry.cu:138-184 (InfLLM-v2 sparse target).
 * Target layers keep compressed key caches (means of 32 keys every 16, of 128 every 64) and, once
 * they cover sparse_switch tokens, every query token attends only to its sparse_topk_k best
 * 64-token blocks, the first sink_window_size blocks and the last block_window_size blocks.
 * At most 16 query heads per KV head and 262144 tokens of context. */
int cpmcu_init_minicpm4_model(float memory_limit, int vocab_size, int num_hidden_layers, int hidden_size,
                              int intermediate_size, int num_attention_heads, int num_key_value_heads,
                              int head_dim, float rms_norm_eps, int torch_dtype, int chunk_length,
                              float scale_embed, float scale_lmhead, float scale_residual, int sink_window_size,
                              int block_window_size, int sparse_topk_k, int sparse_switch, int apply_compress_lse);

/* reference: init_w4a16_gptq_marlin_base_model, src/entry.cu:186-225.  Target whose linears
 * arrive as GPTQ-Marlin tensors (`...qkv_proj|o_proj|gate_up_proj|down_proj.{qweight,scales}`,
 * int32 in Marlin tile order + model-dtype scales, group_size 128).  They are re-tiled when
 * loaded (k-contiguous nibbles, group-major scales) and streamed as 4-bit by the W4A16 GEMM,
 * which dequantises w = (q - 8) * scale on the way into the tensor cores.
 * init_w4a16_gptq_marlin_minicpm4_model (:227-275) is the same target with the InfLLM-v2 block
 * selection of init_minicpm4_model. */
int cpmcu_init_w4a16_gptq_marlin_base_model(float memory_limit, int vocab_size, int num_hidden_layers,
                                            int hidden_size, int intermediate_size, int num_attention_heads,
                                            int num_key_value_heads, int head_dim, float rms_norm_eps,
                                            int group_size, int torch_dtype, int chunk_length, float scale_embed,
                                            float scale_lmhead, float scale_residual);
int cpmcu_init_w4a16_gptq_marlin_minicpm4_model(float memory_limit, int vocab_size, int num_hidden_layers,
                                                int hidden_size, int intermediate_size, int num_attention_heads,
                                                int num_key_value_heads, int head_dim, float rms_norm_eps,
                                                int group_size, int torch_dtype, int chunk_length,
                                                float scale_embed, float scale_lmhead, float scale_residual,
                                                int sink_window_size, int block_window_size, int sparse_topk_k,
                                                int sparse_switch, int apply_compress_lse);

/* reference: init_eagle_model, src/entry.cu:278-301 (plain EAGLE head: no input
 * norms, no attention norm in the draft layer, fc bias, full-vocabulary head). */
int cpmcu_init_eagle_model(int num_layers, int num_iter, int topk_per_iter, int tree_size, int torch_dtype);

/* reference: init_minicpm4_eagle_model, src/entry.cu:303-341 (optional input
 * norms / attention norm, FR-Spec reduced draft vocabulary, draft sliding
 * window, residual scale).  apply_eagle_quant: fc1, fc2 and the draft layer's linears are W4A16 GPTQ-Marlin
 * tensors (group_size 128), src/entry.cu:83-96, src/model/minicpm4/minicpm4_eagle.cuh:77-94. */
int cpmcu_init_minicpm4_eagle_model(int num_layers, int num_iter, int topk_per_iter, int tree_size, int torch_dtype,
                                    int apply_eagle_quant, int group_size, int eagle_window_size,
                                    int frspec_vocab_size, float residual_scale, int use_input_norm,
                                    int use_attn_norm);

/* reference: the three spec / hierarchical initialisers, src/entry.cu:344-459.
 * Out of scope for this library: always fail. */
int cpmcu_init_w4a16_gm_spec_w4a16_gm_model(void);
int cpmcu_init_hier_eagle_w4a16_gm_spec_w4a16_gm_model(void);
int cpmcu_init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model(void);

/* reference: init_storage, src/entry.cu:462.  Allocates the device pool and
 * returns the number of tokens the KV caches hold, or -1. */
int cpmcu_init_storage(void);

/* reference: load_model, src/entry.cu:466.  `param` may be host or device
 * memory holding the tensor in the model dtype (fp32 for *rotary_emb.inv_freq,
 * int32 for eagle.token_id_remap).  Names as in the reference
 * (src/model/model.cuh:116-137, src/model/minicpm4/minicpm4_eagle.cuh:187-221). */
int cpmcu_load_model(const char* name, const void* param);

/* reference: prefill, src/entry.cu:470.  `output` receives the logits of the
 * last token (row 0 of a [>=1, vocab] bf16 buffer). */
int cpmcu_prefill(int input_length, int history_length, const int32_t* input, const int32_t* position_ids,
                  void* output);

/* reference: decode, src/entry.cu:474-496.  *cache_length must already include
 * input_length (reference cpmcu/llm.py:263-283); mask_2d may be NULL (causal).
 * `output` is [input_length, vocab] bf16.  padded_length and cuda_graph are
 * accepted for compatibility and ignored. */
int cpmcu_decode(int input_length, int padded_length, const int32_t* input, const int32_t* position_ids,
                 const int32_t* cache_length, const uint64_t* mask_2d, void* output, int cuda_graph);

/* reference: draft, src/entry.cu:498.  Reads tree_draft_ids[0] (root) and
 * *cache_length; writes tree_draft_ids[1:], positions, masks, parents. */
int cpmcu_draft(int32_t* tree_draft_ids, int32_t* tree_position_ids, const int32_t* cache_length,
                uint64_t* attn_mask, int32_t* tree_parent);

/* reference: verify_and_fix, src/entry.cu:502.  Returns the accept length n
 * (>= 1) or -1; pred[0:n] then holds the emitted tokens. */
int cpmcu_verify_and_fix(int num_tokens, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                         const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent);

/* reference: print_perf_summary, src/entry.cu:506.  Prints launch counts. */
void cpmcu_print_perf_summary(void);

/* ------------------------------------------------------------------ part 2 */

/* Start fused generation after prefill: prefix_length tokens are cached and
 * root_token is the first generated token.  No counterpart in the reference
 * (its loop lives in cpmcu/speculative/tree_drafter.py:215-252). */
int cpmcu_begin_generation(int prefix_length, int32_t root_token);

/* Sampling mode of the fused step (temperature 0 = greedy, the default): with a temperature the step picks the
 * target's token at every tree node as cpmcu_sample does, inside the captured step, draw index = number of steps
 * since cpmcu_begin_generation (the root token is draw 0: cpmcu_sample on the prefill logits).  Call it before
 * cpmcu_begin_generation; a change re-captures the step.  No counterpart in the reference's C module (its
 * sampling is torch code in the Python loop). */
int cpmcu_set_sampling(float temperature, unsigned long long seed);

/* One speculative step on engine-owned buffers.  Writes the n emitted tokens
 * to out_tokens (HOST memory, at most max_tokens) and returns n, or -1. */
int cpmcu_spec_step(int32_t* out_tokens, int max_tokens);

/* Runs one more speculative step eagerly (not from the graph) with every launch
 * bracketed by CUDA events on its stream.  class_ms / class_launches receive 3
 * entries (HOST memory): [0] linear layers, [1] attention, [2] InfLLM-v2 block
 * selection (zero for a dense target); total_ms the whole step.  The step's tokens are consumed (generation advances). */
int cpmcu_profile_step(float* class_ms, int* class_launches, float* total_ms);

/* Device time of the last cpmcu_spec_step in milliseconds (CUDA events). */
double cpmcu_last_step_ms(void);
/* The same step in its two halves, split by an event node inside the captured step: the draft half (state
 * advance, EAGLE draft loop, tree build) and the verify half, which is what the reference's C.decode +
 * argmax + C.verify_and_fix cover (tree embedding, target layers, LM head, argmax, acceptance, K/V
 * compaction and gathers, publishing the result). */
double cpmcu_last_draft_ms(void);
double cpmcu_last_verify_ms(void);
/* Kernels in one captured step / launched by this library so far. */
long cpmcu_launches_per_step(void);
long cpmcu_total_launches(void);
/* Test hook (sparse target): from now on every forward pass also copies each target layer's block
 * mask, [hkv][rows][words] packed per layer at stride hkv * max(chunk_length, 64) * words, into
 * device_buf (caller-owned device memory; NULL stops it).  Returns words per mask row. */
int cpmcu_capture_blockmasks(uint64_t* device_buf);

/* Copies the engine-owned tree of the last step to HOST arrays of 64 entries
 * (any pointer may be NULL). */
int cpmcu_get_tree(int32_t* ids, int32_t* pos, int32_t* parent, int32_t* gt, uint64_t* mask, int32_t* state);
/* Drops the current model (frees the device pool). */
void cpmcu_release(void);

/* ------------------------------------------------------------------ part 3 */

/* Y[M,N] = X[M,K] W[N,K]^T (+ bias[N]).  reference: linear<T>,
 * src/model/linear.cuh:8-37 (cuBLAS).  K % 64 == 0.  grid_limit <= 0 uses one
 * CTA per SM; smaller values force split-K pieces (tests). */
int cpmcu_linear_bf16(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                      int grid_limit);

/* W4A16 linear: Y[M,N] = X[M,K] dequant(Wq)^T with w = (q - 8) * scale.  reference:
 * gptq_marlin_gemm, src/qgemm/gptq_marlin/gptq_marlin.cu:2093-2138.  qweight: int32 [K/16, 2N] in
 * Marlin tile order, scales: bf16 [K/128, N] in Marlin scale order (both as written by
 * model_convert/convert_w4a16.py); they are re-tiled for the streaming kernel inside the call.
 * K % 256 == 0, N % 128 == 0. */
int cpmcu_linear_w4a16(const void* x, const void* qweight, const void* scales, void* y, int M, int N, int K,
                       int grid_limit);

/* Host only, no GPU needed: the work distribution of cpmcu_linear_bf16(M, N, K, grid_limit) as the kernels walk it
 * (the iterator and raster code of the kernels compiled for the host; a launch that uses the cluster variant cuts
 * every tile into equal pieces instead).  out: HOST int32[cap][6] = (cta, tile, token tile, feature tile, first
 * k-block, end k-block) per segment, in each CTA's execution order.  Returns the segment count, -1 on error or
 * when cap is too small. */
int cpmcu_debug_linear_schedule(int M, int N, int K, int grid_limit, int32_t* out, int cap);

/* Times `iters` back-to-back launches of the linear kernel on the library's
 * stream with CUDA events, cycling through `copies` separate weight buffers so
 * that the weights come from HBM and not from L2.  avg_us: HOST float. */
int cpmcu_bench_linear(int M, int N, int K, int copies, int iters, int grid_limit, float* avg_us);
/* The same for the W4A16 kernel: the buffers are read as 4-bit blocks (any bit pattern is a valid weight). */
int cpmcu_bench_linear_w4(int M, int N, int K, int copies, int iters, int grid_limit, float* avg_us);
/* The same for the gate/up projection with the SwiGLU epilogue (cpmcu_linear_swiglu_bf16): 2 * inter weight rows. */
int cpmcu_bench_linear_swiglu(int M, int inter, int K, int copies, int iters, int grid_limit, float* avg_us);

/* reference: mha_fwd_kvcache, src/flash_attn/flash_api.hpp:292-392.
 * q: token t, head h at q + t*q_ld + h*128; caches [budget, hkv*128]; keys
 * visible = *kv_len + kv_len_add; n_valid (device, may be NULL) = number of
 * real query rows; mask (may be NULL) covers the last mask_k keys. */
int cpmcu_tree_attention(const void* q, int q_ld, const void* k_cache, const void* v_cache, int budget, int tq,
                         int hq, int hkv, const int32_t* kv_len, int kv_len_add, const int32_t* n_valid,
                         const uint64_t* mask, int mask_k, int window, int splits, void* out, int out_ld);

/* Block-sparse form of cpmcu_tree_attention for the InfLLM-v2 target layers.  reference:
 * mha_fwd_kvcache with a blockmask, src/flash_attn/flash_api.hpp:292-392 and
 * src/flash_attn/src/flash_blockmask.h.  blockmask: [hkv][tq][bm_words] bits over 64-key blocks;
 * token t also sees every block >= ceil((t + kv_total - tq) / 64) - block_window. */
int cpmcu_sparse_attention(const void* q, int q_ld, const void* k_cache, const void* v_cache, int budget, int tq,
                           int hq, int hkv, const int32_t* kv_len, int kv_len_add, const uint64_t* mask, int mask_k,
                           const uint64_t* blockmask, int bm_words, int block_window, int splits, void* out,
                           int out_ld);

/* InfLLM-v2 block selection of one layer.  reference: MiniCPM4KVCache::compress, mha_fwd_stage1,
 * maxpooling_func, TopK::prefill, topk_to_uint64_func as called from MiniCPM4Attention::decode,
 * src/model/minicpm4/minicpm4_attn.cuh:226-290.  L = *kv_len + kv_len_add accepted key rows.
 * Outputs (device): c1_out [budget/16, hkv*128], c2_out [budget/64, hkv*128] (may be NULL),
 * scores_out [hkv, tq, score_ld] (may be NULL), blockmask_out [hkv, tq, bm_words]. */
int cpmcu_sparse_select(const void* q, int q_ld, int tq, int hq, int hkv, const void* k_cache, int budget,
                        const int32_t* kv_len, int kv_len_add, int sink_window_size, int block_window_size,
                        int sparse_topk_k, int sparse_switch, int apply_compress_lse, void* c1_out, void* c2_out,
                        void* scores_out, int score_ld, uint64_t* blockmask_out, int bm_words);

/* Times `iters` back-to-back tree-attention launches (split kernel + merge) with
 * CUDA events on the library's stream, rotating over 8 separate KV caches. */
int cpmcu_bench_attention(int tq, int hq, int hkv, int kv_total, int splits, int with_mask, int iters,
                          float* avg_us);

/* reference: rms_norm / add_and_rms_norm, src/model/norm.cuh:8-99.
 * delta may be NULL; otherwise x += round(delta * delta_scale) in place first. */
int cpmcu_rms_norm(void* x, const void* delta, float delta_scale, const void* weight, void* y, int rows, int dim,
                   float eps);

/* reference: rotary_embedding + copy_to_kvcache, src/model/rotary.cuh:7-34,
 * src/model/attn.cuh:14-21.  qkv [rows, (hq+2hkv)*128] is rotated in place
 * (q part); k (rotated) and v go to cache row *kv_len + kv_off + r. */
int cpmcu_rope_append(void* qkv, int rows, int hq, int hkv, const float* inv_freq, const int32_t* pos,
                      void* k_cache, void* v_cache, const int32_t* kv_len, int kv_off);

/* reference: gated_silu_interleaved, src/model/activation.cuh:7-18. */
int cpmcu_silu_gate(const void* gate_up, void* out, int rows, int inter);

/* The gate/up projection and the activation of GatedFFN::prefill (src/model/ffn.cuh:72-86) in one launch, for
 * prefill-sized row counts: out[rows, inter] = silu(x Wg^T) * (x Wu^T), w = [gate rows ; up rows] of K columns,
 * both projections rounded to bf16 before the product: bit-identical to cpmcu_linear_bf16 followed by
 * cpmcu_silu_gate.  inter % 64 == 0, K % 64 == 0. */
int cpmcu_linear_swiglu_bf16(const void* x, const void* w, void* out, int rows, int inter, int K, int grid_limit);

/* Row argmax (lowest index wins ties); reference: torch argmax in
 * cpmcu/speculative/tree_drafter.py:233. */
int cpmcu_argmax(const void* logits, int rows, int vocab, int32_t* out);

/* One token per row drawn from softmax(logits[r] / temperature); reference: torch.multinomial over
 * F.softmax(logits / temperature), cpmcu/speculative/tree_drafter.py:99-100,230-231.  The draw is
 * argmax(logit / temperature + Gumbel noise) with Philox4x32-10 noise keyed by (seed, row, draw, column), so it
 * is a pure function of its arguments; temperature == 0 is cpmcu_argmax. */
int cpmcu_sample(const void* logits, int rows, int vocab, float temperature, unsigned long long seed, int draw,
                 int32_t* out);

/* Row argmax like cpmcu_argmax, but without any device allocation.  It has no
 * counterpart in the reference.  cpmcu_argmax takes its two-stage scratch from
 * cudaMalloc on every call and frees it again.  Once cpmcu_init_storage has
 * handed memory_limit of the device to the model pool that allocation can fail,
 * and some callers may not allocate at all: a serving loop that picks tokens
 * from logits it owns while the engine is live, or code running under a memory
 * budget that was fixed at start-up.  For them the scratch is a 16 KB array
 * inside the library image, which every GPU that loads the library keeps until
 * exit; the call makes no cudaMalloc / cudaFree and cannot fail for lack of
 * memory.
 *   - rows <= 64 and vocab <= 262144, otherwise -1 with a message.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current).
 *   - EVERY call launches on the legacy default stream and returns after that
 *     stream has drained.  The library's own stream is a blocking stream, so
 *     the call orders itself after work already queued there (a speculative
 *     step in flight finishes first) and before work queued later: it does not
 *     run beside a step.  For the same reason no call, first or later, may be
 *     made while any stream of the process is being captured into a CUDA graph.
 *   - All calls share the one array, which keeps the previous call's partials
 *     (each call overwrites what it reads, nothing needs clearing); two calls
 *     that overlap on the GPU, from different host threads or processes sharing
 *     a context, race on it.  The per-device address cache is written without a
 *     lock: concurrent first calls store the same value. */
int cpmcu_argmax_noalloc(const void* logits, int rows, int vocab, int32_t* out);

/* Draft tree from given logits: level 0 uses row 0 of `logits`, level d >= 1
 * rows 1 + (d-1)*k .. (k rows).  logits: [1 + (num_iter-1)*k, vocab] bf16.
 * Runs log-softmax, top-k, frontier expansion and the final tree build exactly
 * as the draft loop does (reference src/model/eagle.cuh:436-498, 188-218).
 * Outputs (device): tree ids[1:], positions, masks, parents (tree_size
 * entries each; ids[0] is left untouched) and, if not NULL, the candidate
 * history tried_val (bf16) / tried_pos / tried_parent. */
int cpmcu_draft_tree_from_logits(const void* logits, int vocab, int k, int num_iter, int tree_size,
                                 const int32_t* token_id_remap, const int32_t* cache_length, int32_t* tree_ids,
                                 int32_t* tree_pos, uint64_t* tree_mask, int32_t* tree_parent, void* tried_val,
                                 int32_t* tried_pos, int32_t* tried_parent);

/* reference: verify_kernel + fix_kvcache_kernel_1/2, src/model/tree_drafter.cuh:5-101.
 * caches: device array of num_caches row-major [rows, kv_dim] bf16 buffers.
 * result (device, 18 ints): [0] accept length, [1] best node, [2..] path. */
int cpmcu_verify_and_compact(int tree_size, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                             const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent,
                             void* const* caches, int num_caches, int kv_dim, int max_accept, int32_t* result);

/* The whole tail of a speculative step in its one launch: acceptance and K/V compaction as above plus, when
 * hidden > 0, what the reference's verify does next (src/model/minicpm4/minicpm4_eagle.cuh:398-418,
 * remap_hidden src/model/eagle.cuh:108-115): prev_hidden[i] = norm_out[path[i]] (rows of `hidden` bf16),
 * prev_embed[i] = embed_table[emitted token i] * embed_scale, eagle_pos[i] = cache_length + i, for i < n
 * (eagle_pos for all i < max_accept).  cache_rows: rows every cache holds; a compaction that would touch a
 * row at or beyond it is skipped and reported as an error.  With hidden == 0 the five buffers may be NULL. */
int cpmcu_accept_fixup(int tree_size, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                       const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent,
                       void* const* caches, int num_caches, int kv_dim, int cache_rows, int max_accept, int hidden,
                       const void* norm_out, void* prev_hidden, const void* embed_table, float embed_scale,
                       void* prev_embed, int32_t* eagle_pos, int32_t* result);

#ifdef __cplusplus
}
#endif
#endif /* CPMCU_B200_H */
