// Host-side model state for the speculative-decoding path: weights, KV caches,
// activation buffers, pre-built kernel plans and the captured step graph.
// Mirrors the reference's `Model` interface (src/model/model.cuh:14-23:
// init_storage / load_to_storage / prefill / decode / draft / verify) for the
// Llama-format target (ModelImpl, src/model/model.cuh:25-173) and the EAGLE
// drafters (EagleImpl src/model/eagle.cuh:262-516, MiniCPM4EagleImpl
// src/model/minicpm4/minicpm4_eagle.cuh:10-418).
#pragma once
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "draft_tree.cuh"
#include "sparse_select.cuh"

struct ModelConfig {
    float memory_limit = 0.8f;
    int vocab = 0, layers = 0, hidden = 0, inter = 0, hq = 0, hkv = 0, head_dim = 128;
    float eps = 1e-5f;
    int chunk_length = 1024;
    float scale_embed = 1.f, scale_lmhead = 1.f, scale_residual = 1.f;
    bool w4a16 = false;  // target linears arrive as GPTQ-Marlin int4 + scales (embeddings / LM head stay bf16)
    int group_size = 128;
    SparseConfig sparse;  // InfLLM-v2 block selection in the target layers (init_minicpm4_model)
};

struct EagleConfig {
    int num_layers = 1, num_iter = 6, topk = 10, tree_size = 60;
    int window = 0;        // draft sliding window (tokens), 0 = off
    int frspec_vocab = 0;  // 0 = full vocabulary
    float residual_scale = 1.f;
    bool use_input_norm = false, use_attn_norm = false;
    bool minicpm4_variant = false;  // draft LM head skips scale_lmhead (reference quirk)
    // W4A16 drafter (reference apply_eagle_quant, src/entry.cu:83-96): fc1, fc2 and the draft layer's four linears
    // arrive as GPTQ-Marlin int4 tensors; fc1 and fc2 are then two GEMMs (the bf16 drafter runs them as one)
    bool quant = false;
    int group_size = 128;
};

struct LayerWeights {
    bf16* qkv = nullptr;      // [(hq + 2 hkv) * d, hidden]  rows: q | k | v
    bf16* o = nullptr;        // [hidden, hq * d]
    bf16* gate_up = nullptr;  // [2 * inter, hidden]          rows: gate | up
    bf16* down = nullptr;     // [hidden, inter]
    bf16* ln_attn = nullptr;  // [hidden]
    bf16* ln_ffn = nullptr;   // [hidden]
    // W4A16 layers: 4-bit blocks in the streaming layout of the W4A16 GEMM instead of the bf16 matrices
    uint8_t *qkv_q = nullptr, *o_q = nullptr, *gate_up_q = nullptr, *down_q = nullptr;
};
struct KVLayer {
    bf16* k = nullptr;  // [budget, hkv * d]
    bf16* v = nullptr;
};

// How a batch of rows walks through a decoder layer.
struct RowCtx {
    int rows = 0;
    const int32_t* pos = nullptr;       // explicit positions, or
    const int32_t* pos_base = nullptr;  // *pos_base + pos_off + r * pos_step
    int pos_off = 0, pos_step = 0;
    const int32_t* kv_len = nullptr;    // KV row of r = *kv_len + kv_append_off + r
    int kv_append_off = 0;
    int attn_kv_add = 0;                // keys visible = *kv_len + attn_kv_add
    const int32_t* n_valid = nullptr;
    const uint64_t* mask = nullptr;
    int mask_k = 0;
    int window = 0;
};

struct LayerPlans {
    LinearPlan qkv, o, gate_up, down;
    AttnPlan attn;
};
struct ForwardPlans {
    int rows = 0;
    bool lazy = false;   // layers[l] is built by target_forward right before layer l is launched
    std::vector<LayerPlans> layers;
};

class Engine {
public:
    explicit Engine(const ModelConfig& mc);
    ~Engine();
    void attach_eagle(const EagleConfig& ec);
    int init_storage();
    void load(const std::string& name, const void* src);

    // reference-compatible entry points (device pointers owned by the caller)
    void prefill(int n, int history, const int32_t* ids, const int32_t* pos, bf16* logits_out);
    void decode(int n, int padded_len, const int32_t* ids, const int32_t* pos, const int32_t* cache_length,
                const uint64_t* mask, bf16* logits_out, bool cuda_graph);
    void draft(int32_t* tree_ids, int32_t* tree_pos, const int32_t* cache_length, uint64_t* tree_mask,
               int32_t* tree_parent);
    int verify_and_fix(int T, int32_t* pred, const int32_t* gt, const int32_t* pos, const int32_t* cache_length,
                       const uint64_t* mask, const int32_t* parent);

    // fused step: draft -> tree -> verify -> accept in one CUDA graph, state on the device.
    // begin_generation() is called once after prefill with the first root token.
    void begin_generation(int prefix_length, int32_t root_token);
    // temperature > 0: the fused step picks the target's token at every tree node by sampling from
    // softmax(logits / temperature) instead of argmax (reference cpmcu/speculative/tree_drafter.py:230-231), on the
    // device and inside the captured step; the draw index advances with every step, so a run is a function of the seed
    void set_sampling(float temperature, unsigned long long seed);
    int spec_step(int32_t* out_tokens, int max_tokens);  // returns accept length n; out_tokens[0:n]
    void profile_step(float* ms, int* counts, float* total_ms);
    double last_step_device_ms() const { return last_step_ms_; }
    // device time of the two halves of the last captured step: state advance + draft loop + tree build, and
    // the target's verify pass (tree embedding .. LM head .. argmax .. acceptance and fix-up .. publish)
    double last_draft_ms() const { return last_draft_ms_; }
    double last_verify_ms() const { return last_verify_ms_; }
    long launches_per_step() const { return launches_per_step_; }

    const ModelConfig& config() const { return mc_; }
    bool has_eagle() const { return has_eagle_; }
    int budget() const { return budget_; }
    const bf16* norm_out() const { return norm_out_; }
    const int32_t* tree_buffers(int which) const;

    // ---- test hook: copy every target layer's block mask of each forward pass to `buf`
    // ([layers][hkv][max_rows][bm_words], device memory owned by the caller; null stops it)
    void capture_blockmasks(uint64_t* buf) { bm_capture_ = buf; }
    int blockmask_words() const { return sp_.bm_words; }
    int max_rows() const { return max_rows_; }

private:
    // ---- memory
    struct Pool {
        uint8_t* base = nullptr;
        size_t used = 0, cap = 0;
        bool counting = true;
        void* take(size_t bytes);
    };
    void lay_out(Pool& pool);
    template <typename T>
    T* take(Pool& pool, size_t count) { return reinterpret_cast<T*>(pool.take(count * sizeof(T))); }

    // ---- building blocks
    void build_layer_plans(LayerPlans& lp, const LayerWeights& w, const KVLayer& kv, int rows, int attn_splits);
    ForwardPlans& target_plans(int rows);
    // plans of the draft layer; without an attention norm its q/k/v GEMM reads the fc output in place
    void build_draft_plans(LayerPlans& lp, int rows, int attn_splits);
    // sparse_layer >= 0: target layer with InfLLM-v2 block selection (index into the compressed caches)
    void layer_forward(LayerPlans& lp, const LayerWeights& w, const KVLayer& kv, const RowCtx& c, bf16* x,
                       const bf16* pending, float pending_scale, bool first_norm, float res_scale, cudaStream_t s,
                       int sparse_layer = -1);
    void sparse_prepare(const RowCtx& c, cudaStream_t s);
    void target_forward(ForwardPlans& fp, const RowCtx& c, const int32_t* ids, bool all_logits, bf16* logits_out,
                        int logits_ld, cudaStream_t s);
    void lm_head_rows(const bf16* x, int x_rows, int rows, bf16* logits_out, int ld, cudaStream_t s);
    void draft_forward(const RowCtx& c, int rows, LayerPlans& lp, cudaStream_t s);
    void draft_first(int history, cudaStream_t s);
    void draft_catchup(cudaStream_t s);
    void draft_levels(int32_t* tree_ids, int32_t* tree_pos, const int32_t* cache_length, uint64_t* tree_mask,
                      int32_t* tree_parent, bool first, cudaStream_t s);
    void accept_and_fix(int T, int32_t* pred, const int32_t* gt, const int32_t* pos, const int32_t* cache_length,
                        const uint64_t* mask, const int32_t* parent, cudaStream_t s);
    void enqueue_step(bool first, cudaStream_t s);
    void check_errors(const char* where);
    int attn_splits_for(int rows) const;
    // bf16 gate/up weights: gate and up rows of a 64-feature group share one 128-row tile when the width is a multiple
    // of 64; otherwise [gate ; up] as in the checkpoint
    bool gate_up_interleaved() const { return mc_.inter % 64 == 0; }
    size_t gate_up_elems() const { return linear_weight_elems(2 * mc_.inter, mc_.hidden); }

    ModelConfig mc_;
    EagleConfig ec_;
    bool has_eagle_ = false;
    bool storage_ready_ = false;
    Pool pool_;
    int budget_ = 0;
    int max_rows_ = 0;
    int qkv_dim_ = 0;

    // weights
    bf16* embed_ = nullptr;
    bf16* lm_head_ = nullptr;
    bf16* final_norm_ = nullptr;
    float* inv_freq_ = nullptr;
    std::vector<LayerWeights> layers_;
    std::vector<KVLayer> kv_;
    // draft weights
    bf16* fc_ = nullptr;       // [hidden, 2*hidden]: columns [0,H) act on the token embedding, [H,2H) on the hidden state
    bf16* fc_bias_ = nullptr;
    uint8_t *fc1_q_ = nullptr, *fc2_q_ = nullptr;  // W4A16 drafter: [H -> H] each, streaming 4-bit layout
    bf16* in_norm1_ = nullptr;
    bf16* in_norm2_ = nullptr;
    LayerWeights elayer_;
    KVLayer ekv_;
    bf16* draft_lm_head_ = nullptr;  // FR-Spec gathered rows, or alias of lm_head_
    int32_t* token_id_remap_ = nullptr;
    int draft_vocab_ = 0;
    bool remap_loaded_ = false;
    // W4A16 loading: whichever of (qweight, scales) arrives first waits here for the other
    struct PendingQuant {
        void* qweight = nullptr;
        void* scales = nullptr;
    };
    std::map<std::string, PendingQuant> pending_quant_;
    void load_quantized(const std::string& key, bool is_scales, const void* src, int K, int N, uint8_t* wq);

    // activations
    bf16 *x_ = nullptr, *normed_ = nullptr, *qkv_ = nullptr, *attn_out_ = nullptr, *delta_ = nullptr,
         *gate_up_ = nullptr, *act_ = nullptr, *norm_out_ = nullptr, *lm_in_ = nullptr;
    bf16 *e_in_ = nullptr, *e_x_ = nullptr, *e_h_ = nullptr, *e_hid_ = nullptr, *e_emb_ = nullptr;
    bf16 *prev_embed_ = nullptr, *prev_hidden_ = nullptr;
    bf16* e_logits_ = nullptr;   // [16, draft_vocab]
    bf16* logits_ = nullptr;     // [64, vocab] (fused mode)
    float* gemm_ws_ = nullptr;
    int* tickets_ = nullptr;
    float *attn_ws_o_ = nullptr, *attn_ws_ml_ = nullptr;
    void* scan_ws_ = nullptr;
    void* argmax_ws_ = nullptr;
    bf16** d_cache_ptrs_ = nullptr;
    uint64_t* bm_capture_ = nullptr;
    SparseBuffers sp_;  // InfLLM-v2 compressed caches, scores and block masks (sparse target only)
    // device state words
    int32_t* st_ = nullptr;
    enum { S_L = 0, S_NPREV = 1, S_BASE = 2, S_LASTROW = 3, S_ACCEPT = 4, S_ZERO = 5, S_DRAW = 8, S_COUNT = 16 };
    int32_t* eagle_pos_ = nullptr;
    int32_t* accept_result_ = nullptr;  // [2 + 16]
    int32_t* d_publish_ = nullptr;      // [32]: n, tokens, error word (copied to the host)
    DraftTreeState tree_;
    // engine-owned tree buffers (fused mode)
    int32_t *t_ids_ = nullptr, *t_pos_ = nullptr, *t_parent_ = nullptr, *t_gt_ = nullptr;
    uint64_t* t_mask_ = nullptr;
    int32_t* h_result_ = nullptr;  // pinned: [0]=n, [1..] tokens

    // host-side draft bookkeeping (reference: num_prev, num_history_tokens, is_first_draft)
    int num_prev_ = 0, num_history_ = 0;
    bool first_draft_ = true;
    int catchup_rows_ = 0;

    std::map<int, std::unique_ptr<ForwardPlans>> plans_;
    LayerPlans eplan_level_, eplan_catchup_;
    LinearPlan fc_plan_level_, fc_plan_catchup_, dlm_plan_level_, dlm_plan_catchup_;
    LinearPlan fc2_plan_level_, fc2_plan_catchup_;  // W4A16 drafter: the hidden-state half of fc
    // Where the drafter's fc input rows live: bf16 drafter [rows, 2H] (embedding | hidden state side by side, one
    // GEMM over K = 2H); W4A16 drafter two [rows, H] matrices (the int4 kernel wants densely packed rows).
    int ein_ld() const { return ec_.quant ? mc_.hidden : 2 * mc_.hidden; }
    bf16* ein_hidden() const { return ec_.quant ? e_in_ + static_cast<size_t>(max_rows_) * mc_.hidden : e_in_ + mc_.hidden; }
    void draft_fc(int rows, const LinearPlan& fc, const LinearPlan& fc2, cudaStream_t s);
    LinearPlan lm_plan_tree_;

    cudaGraphExec_t step_graph_ = nullptr;
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr, ev_mid_ = nullptr;
    double last_step_ms_ = 0.0, last_draft_ms_ = 0.0, last_verify_ms_ = 0.0;
    // tokens whose target K/V rows are final, as far as the host knows (prefill, then every accepted length);
    // -1 before the first prefill.  Guards every pass against writing K/V rows beyond the budget.
    long host_len_ = -1;
    float temperature_ = 0.f;
    unsigned long long sample_seed_ = 0;
    void require_room(long rows_after_len, const char* where) const;
    long launches_per_step_ = 0;
    long launch_counter_ = 0;
};
