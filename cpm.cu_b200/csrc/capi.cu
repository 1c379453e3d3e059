// extern "C" surface of libcpmcu_b200.so (declared in include/cpmcu_b200.h).
// Holds the single global model the reference keeps in src/entry.cu:98 and
// turns C++ exceptions into return codes + a thread-local message.
#include <cstdio>
#include <memory>
#include <vector>

#include "../../include/cpmcu_b200.h"
#include "engine.cuh"
#include "sparse_select.cuh"

namespace {

thread_local std::string g_error;
std::unique_ptr<Engine> g_engine;

template <typename F>
int guarded(F&& f) {
    try {
        g_error.clear();
        return f();
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    } catch (...) {
        g_error = "unknown error";
        return -1;
    }
}

Engine& engine() {
    if (!g_engine) throw std::runtime_error("cpmcu_b200: no model initialised");
    return *g_engine;
}

void require_bf16(int torch_dtype) {
    if (torch_dtype != 1) throw std::invalid_argument("cpmcu_b200: only torch_dtype 1 (bfloat16) is supported");
}

int not_built(const char* what) {
    g_error = std::string("cpmcu_b200: ") + what + " is not built in this library";
    return -1;
}

struct DeviceBuf {
    void* p = nullptr;
    explicit DeviceBuf(size_t bytes) { CUDA_CHECK(cudaMalloc(&p, bytes ? bytes : 1)); }
    ~DeviceBuf() { cudaFree(p); }
    DeviceBuf(const DeviceBuf&) = delete;
    DeviceBuf& operator=(const DeviceBuf&) = delete;
};

void sync_and_check(const char* where) {
    const int e = read_and_clear_error();
    if (e != 0) throw std::runtime_error(std::string("cpmcu_b200: kernel error flags ") + std::to_string(e) + " in " + where);
}

}  // namespace

void cpm_set_error(const char* msg) { g_error = msg ? msg : ""; }

extern "C" {

const char* cpmcu_last_error(void) { return g_error.c_str(); }

namespace {
struct SparseArgs {
    int sink_window_size, block_window_size, sparse_topk_k, sparse_switch, apply_compress_lse;
};

// The four target initialisers differ only in two switches: int4 linears (group_size > 0) and block selection.
int init_target(float memory_limit, int vocab_size, int num_hidden_layers, int hidden_size, int intermediate_size,
                int num_attention_heads, int num_key_value_heads, int head_dim, float rms_norm_eps, int torch_dtype,
                int chunk_length, float scale_embed, float scale_lmhead, float scale_residual, int group_size,
                const SparseArgs* sp) {
    return guarded([&] {
        require_bf16(torch_dtype);
        ModelConfig mc;
        mc.memory_limit = memory_limit;
        mc.vocab = vocab_size;
        mc.layers = num_hidden_layers;
        mc.hidden = hidden_size;
        mc.inter = intermediate_size;
        mc.hq = num_attention_heads;
        mc.hkv = num_key_value_heads;
        mc.head_dim = head_dim;
        mc.eps = rms_norm_eps;
        mc.chunk_length = chunk_length;
        mc.scale_embed = scale_embed;
        mc.scale_lmhead = scale_lmhead;
        mc.scale_residual = scale_residual;
        if (group_size > 0) {
            mc.w4a16 = true;
            mc.group_size = group_size;
        }
        if (sp != nullptr) {
            CPM_REQUIRE(sp->sink_window_size >= 0 && sp->block_window_size >= 1 && sp->sparse_topk_k >= 1 &&
                            sp->sparse_switch >= 0,
                        "init_minicpm4_model: bad block-selection arguments");
            CPM_REQUIRE(num_key_value_heads >= 1 && num_attention_heads / num_key_value_heads <= 16,
                        "init_minicpm4_model: at most 16 query heads per KV head");
            mc.sparse.enabled = true;
            mc.sparse.sink_blocks = sp->sink_window_size;
            mc.sparse.window_blocks = sp->block_window_size;
            mc.sparse.topk = sp->sparse_topk_k;
            mc.sparse.sparse_switch = sp->sparse_switch;
            mc.sparse.compress_lse = sp->apply_compress_lse != 0;
        }
        g_engine.reset();  // one model per process, like the reference's global
        g_engine = std::make_unique<Engine>(mc);
        return 0;
    });
}
}  // namespace

int cpmcu_init_base_model(float memory_limit, int vocab_size, int num_hidden_layers, int hidden_size,
                          int intermediate_size, int num_attention_heads, int num_key_value_heads, int head_dim,
                          float rms_norm_eps, int torch_dtype, int chunk_length, float scale_embed,
                          float scale_lmhead, float scale_residual) {
    return init_target(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
                       num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed, scale_lmhead,
                       scale_residual, 0, nullptr);
}

int cpmcu_init_minicpm4_model(float memory_limit, int vocab_size, int num_hidden_layers, int hidden_size,
                              int intermediate_size, int num_attention_heads, int num_key_value_heads,
                              int head_dim, float rms_norm_eps, int torch_dtype, int chunk_length,
                              float scale_embed, float scale_lmhead, float scale_residual, int sink_window_size,
                              int block_window_size, int sparse_topk_k, int sparse_switch, int apply_compress_lse) {
    const SparseArgs sp = {sink_window_size, block_window_size, sparse_topk_k, sparse_switch, apply_compress_lse};
    return init_target(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
                       num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed, scale_lmhead,
                       scale_residual, 0, &sp);
}

int cpmcu_init_w4a16_gptq_marlin_base_model(float memory_limit, int vocab_size, int num_hidden_layers,
                                            int hidden_size, int intermediate_size, int num_attention_heads,
                                            int num_key_value_heads, int head_dim, float rms_norm_eps,
                                            int group_size, int torch_dtype, int chunk_length, float scale_embed,
                                            float scale_lmhead, float scale_residual) {
    if (group_size <= 0) return guarded([&]() -> int { throw std::invalid_argument("cpmcu_b200: W4A16: only group_size 128 is supported"); });
    return init_target(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
                       num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed, scale_lmhead,
                       scale_residual, group_size, nullptr);
}

int cpmcu_init_w4a16_gptq_marlin_minicpm4_model(float memory_limit, int vocab_size, int num_hidden_layers,
                                                int hidden_size, int intermediate_size, int num_attention_heads,
                                                int num_key_value_heads, int head_dim, float rms_norm_eps,
                                                int group_size, int torch_dtype, int chunk_length, float scale_embed,
                                                float scale_lmhead, float scale_residual, int sink_window_size,
                                                int block_window_size, int sparse_topk_k, int sparse_switch,
                                                int apply_compress_lse) {
    // the W4A16 target with InfLLM-v2 block selection: both features are independent in the engine
    if (group_size <= 0) return guarded([&]() -> int { throw std::invalid_argument("cpmcu_b200: W4A16: only group_size 128 is supported"); });
    const SparseArgs sp = {sink_window_size, block_window_size, sparse_topk_k, sparse_switch, apply_compress_lse};
    return init_target(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
                       num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed, scale_lmhead,
                       scale_residual, group_size, &sp);
}

int cpmcu_init_eagle_model(int num_layers, int num_iter, int topk_per_iter, int tree_size, int torch_dtype) {
    return guarded([&] {
        require_bf16(torch_dtype);
        EagleConfig ec;
        ec.num_layers = num_layers;
        ec.num_iter = num_iter;
        ec.topk = topk_per_iter;
        ec.tree_size = tree_size;
        ec.minicpm4_variant = false;
        engine().attach_eagle(ec);
        return 0;
    });
}

int cpmcu_init_minicpm4_eagle_model(int num_layers, int num_iter, int topk_per_iter, int tree_size, int torch_dtype,
                                    int apply_eagle_quant, int group_size, int eagle_window_size,
                                    int frspec_vocab_size, float residual_scale, int use_input_norm,
                                    int use_attn_norm) {
    return guarded([&] {
        require_bf16(torch_dtype);
        EagleConfig ec;
        ec.quant = apply_eagle_quant != 0;
        if (ec.quant) {
            CPM_REQUIRE(group_size == 128, "W4A16 drafter: only group_size 128 is supported");
            ec.group_size = group_size;
        }
        ec.num_layers = num_layers;
        ec.num_iter = num_iter;
        ec.topk = topk_per_iter;
        ec.tree_size = tree_size;
        ec.window = eagle_window_size;
        ec.frspec_vocab = frspec_vocab_size;
        ec.residual_scale = residual_scale;
        ec.use_input_norm = use_input_norm != 0;
        ec.use_attn_norm = use_attn_norm != 0;
        ec.minicpm4_variant = true;
        engine().attach_eagle(ec);
        return 0;
    });
}

int cpmcu_init_w4a16_gm_spec_w4a16_gm_model(void) { return not_built("sequence speculative decoding with a quantised draft LLM"); }
int cpmcu_init_hier_eagle_w4a16_gm_spec_w4a16_gm_model(void) { return not_built("hierarchical speculative decoding"); }
int cpmcu_init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model(void) { return not_built("hierarchical speculative decoding"); }

int cpmcu_init_storage(void) {
    return guarded([&] { return engine().init_storage(); });
}

int cpmcu_load_model(const char* name, const void* param) {
    return guarded([&] {
        engine().load(name, param);
        return 0;
    });
}

int cpmcu_prefill(int input_length, int history_length, const int32_t* input, const int32_t* position_ids,
                  void* output) {
    return guarded([&] {
        engine().prefill(input_length, history_length, input, position_ids, static_cast<bf16*>(output));
        return 0;
    });
}

int cpmcu_decode(int input_length, int padded_length, const int32_t* input, const int32_t* position_ids,
                 const int32_t* cache_length, const uint64_t* mask_2d, void* output, int cuda_graph) {
    return guarded([&] {
        engine().decode(input_length, padded_length, input, position_ids, cache_length, mask_2d,
                        static_cast<bf16*>(output), cuda_graph != 0);
        return 0;
    });
}

int cpmcu_draft(int32_t* tree_draft_ids, int32_t* tree_position_ids, const int32_t* cache_length,
                uint64_t* attn_mask, int32_t* tree_parent) {
    return guarded([&] {
        engine().draft(tree_draft_ids, tree_position_ids, cache_length, attn_mask, tree_parent);
        return 0;
    });
}

int cpmcu_verify_and_fix(int num_tokens, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                         const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent) {
    return guarded([&] {
        return engine().verify_and_fix(num_tokens, pred, gt, position_ids, cache_length, attn_mask, tree_parent);
    });
}

void cpmcu_print_perf_summary(void) {
    try {
        printf("cpmcu_b200: %ld kernels launched so far", runtime().launches);
        if (g_engine && g_engine->launches_per_step() > 0) {
            printf(", %ld kernels per captured speculative step, last step %.3f ms", g_engine->launches_per_step(),
                   g_engine->last_step_device_ms());
        }
        printf("\n");
    } catch (...) {
    }
}

int cpmcu_begin_generation(int prefix_length, int32_t root_token) {
    return guarded([&] {
        engine().begin_generation(prefix_length, root_token);
        return 0;
    });
}

int cpmcu_set_sampling(float temperature, unsigned long long seed) {
    return guarded([&] {
        engine().set_sampling(temperature, seed);
        return 0;
    });
}

int cpmcu_spec_step(int32_t* out_tokens, int max_tokens) {
    return guarded([&] { return engine().spec_step(out_tokens, max_tokens); });
}

int cpmcu_profile_step(float* class_ms, int* class_launches, float* total_ms) {
    return guarded([&] {
        engine().profile_step(class_ms, class_launches, total_ms);
        return 0;
    });
}

double cpmcu_last_step_ms(void) { return g_engine ? g_engine->last_step_device_ms() : 0.0; }
double cpmcu_last_draft_ms(void) { return g_engine ? g_engine->last_draft_ms() : 0.0; }
double cpmcu_last_verify_ms(void) { return g_engine ? g_engine->last_verify_ms() : 0.0; }
long cpmcu_launches_per_step(void) { return g_engine ? g_engine->launches_per_step() : 0; }
long cpmcu_total_launches(void) {
    try {
        return runtime().launches;
    } catch (...) {
        return 0;
    }
}

int cpmcu_get_tree(int32_t* ids, int32_t* pos, int32_t* parent, int32_t* gt, uint64_t* mask, int32_t* state) {
    return guarded([&] {
        Engine& e = engine();
        cudaStream_t s = runtime().stream;
        void* dst[6] = {ids, pos, parent, gt, mask, state};
        const size_t bytes[6] = {256, 256, 256, 256, 512, 64};
        for (int i = 0; i < 6; ++i) {
            if (dst[i]) CUDA_CHECK(cudaMemcpyAsync(dst[i], e.tree_buffers(i), bytes[i], cudaMemcpyDeviceToHost, s));
        }
        CUDA_CHECK(cudaStreamSynchronize(s));
        return 0;
    });
}

int cpmcu_capture_blockmasks(uint64_t* device_buf) {
    return guarded([&] {
        Engine& e = engine();
        e.capture_blockmasks(device_buf);
        return e.blockmask_words();
    });
}

void cpmcu_release(void) { g_engine.reset(); }

// ------------------------------------------------------------------ kernel-level entry points
int cpmcu_linear_bf16(const void* x, const void* w, const void* bias, void* y, int M, int N, int K, int grid_limit) {
    return guarded([&] {
        Runtime& rt = runtime();
        const int limit = (grid_limit > 0) ? grid_limit : rt.num_sms;
        const int mt = linear_pick_mt(M);
        DeviceBuf ws(linear_workspace_bytes(mt, limit));
        const size_t tiles = static_cast<size_t>(ceil_div(N, 128)) * ceil_div(M, mt);
        DeviceBuf tickets(2 * tiles * sizeof(int));
        CUDA_CHECK(cudaMemsetAsync(tickets.p, 0, 2 * tiles * sizeof(int), rt.stream));
        // the caller's row-major W in the kernels' tile-major layout
        DeviceBuf wt(linear_weight_elems(N, K) * sizeof(bf16));
        CUDA_CHECK(cudaMemsetAsync(wt.p, 0, linear_weight_elems(N, K) * sizeof(bf16), rt.stream));
        retile_weight_rows(w, N, K, static_cast<bf16*>(wt.p), K, 0, 0, 0, rt.stream);
        LinearPlan p = make_linear_plan(static_cast<const bf16*>(x), M, static_cast<const bf16*>(wt.p), M, N, K,
                                        static_cast<bf16*>(y), N, static_cast<const bf16*>(bias),
                                        static_cast<float*>(ws.p), static_cast<int*>(tickets.p), limit);
        launch_linear(p, rt.stream);
        sync_and_check("linear");
        return 0;
    });
}

int cpmcu_debug_linear_schedule(int M, int N, int K, int grid_limit, int32_t* out, int cap) {
    int n = -1;
    const int rc = guarded([&] {
        CPM_REQUIRE(M >= 1 && N >= 1 && K >= 64 && K % 64 == 0 && grid_limit >= 1 && out != nullptr && cap >= 1,
                    "debug_linear_schedule: bad arguments");
        n = linear_schedule_dump(M, N, K, grid_limit, out, cap);
        return 0;
    });
    return rc < 0 ? rc : n;
}

int cpmcu_linear_swiglu_bf16(const void* x, const void* w, void* out, int rows, int inter, int K, int grid_limit) {
    return guarded([&] {
        Runtime& rt = runtime();
        const int limit = (grid_limit > 0) ? grid_limit : rt.num_sms;
        // gate rows and up rows into the tiles of their 64-feature groups
        DeviceBuf wt(linear_weight_elems(2 * inter, K) * sizeof(bf16));
        retile_weight_rows(w, inter, K, static_cast<bf16*>(wt.p), K, 1, 0, 0, rt.stream);
        retile_weight_rows(static_cast<const bf16*>(w) + static_cast<size_t>(inter) * K, inter, K, static_cast<bf16*>(wt.p), K, 2, 0,
                           0, rt.stream);
        LinearPlan p = make_linear_swiglu_plan(static_cast<const bf16*>(x), rows, static_cast<const bf16*>(wt.p), rows, inter, K,
                                               static_cast<bf16*>(out), inter, limit);
        launch_linear(p, rt.stream);
        sync_and_check("linear_swiglu");
        return 0;
    });
}

int cpmcu_linear_w4a16(const void* x, const void* qweight, const void* scales, void* y, int M, int N, int K,
                       int grid_limit) {
    return guarded([&] {
        Runtime& rt = runtime();
        cudaStream_t s = rt.stream;
        const int limit = (grid_limit > 0) ? grid_limit : rt.num_sms;
        const int mt = std::min(linear_pick_mt(M), 128);  // the 4-bit kernel's largest token tile
        CPM_REQUIRE(K % 256 == 0 && N % 128 == 0, "linear_w4a16: K must be a multiple of 256 and N of 128");
        DeviceBuf wq(linear_w4_weight_bytes(N, K));
        marlin_retile_for_w4(qweight, scales, K, N, wq.p, s);
        DeviceBuf work(linear_w4_workspace_bytes(mt, limit));
        const size_t tiles = static_cast<size_t>(N / 128) * ceil_div(M, mt);
        DeviceBuf tickets(2 * tiles * sizeof(int));
        CUDA_CHECK(cudaMemsetAsync(tickets.p, 0, 2 * tiles * sizeof(int), s));
        LinearPlan p = make_linear_plan_w4(static_cast<const bf16*>(x), M, wq.p, M, N, K, static_cast<bf16*>(y), N,
                                           static_cast<float*>(work.p), static_cast<int*>(tickets.p), limit);
        launch_linear(p, s);
        sync_and_check("linear_w4a16");
        return 0;
    });
}

static int bench_linear_impl(int M, int N, int K, int copies, int iters, int grid_limit, float* avg_us, bool w4,
                             bool swiglu = false) {
    return guarded([&] {
        Runtime& rt = runtime();
        cudaStream_t s = rt.stream;
        CPM_REQUIRE(copies >= 1 && copies <= 64 && iters >= 1, "bench_linear: bad repetition counts");
        const int limit = (grid_limit > 0) ? grid_limit : rt.num_sms;
        const int mt = linear_pick_mt(M);
        const size_t wbytes = linear_weight_elems(N, K) * 2;   // any contents: the buffer is read as tile-major weights
        DeviceBuf w(wbytes * copies), x(static_cast<size_t>(M) * K * 2), y(static_cast<size_t>(M) * N * 2);
        DeviceBuf ws(linear_workspace_bytes(mt, limit));
        const size_t tiles = static_cast<size_t>(ceil_div(N, 128)) * ceil_div(M, mt);
        DeviceBuf tickets(2 * tiles * sizeof(int));
        CUDA_CHECK(cudaMemsetAsync(tickets.p, 0, 2 * tiles * sizeof(int), s));
        CUDA_CHECK(cudaMemsetAsync(w.p, 0x3c, wbytes * copies, s));
        CUDA_CHECK(cudaMemsetAsync(x.p, 0x3c, static_cast<size_t>(M) * K * 2, s));
        std::vector<LinearPlan> plans;
        for (int c = 0; c < copies; ++c) {
            if (w4) {  // the same buffer read as 4-bit blocks: about a quarter of the bytes per launch
                plans.push_back(make_linear_plan_w4(static_cast<const bf16*>(x.p), M,
                                                    static_cast<uint8_t*>(w.p) + linear_w4_weight_bytes(N, K) * c,
                                                    M, N, K, static_cast<bf16*>(y.p), N,
                                                    static_cast<float*>(ws.p), static_cast<int*>(tickets.p), limit));
                continue;
            }
            if (swiglu) {  // N / 2 gate rows + N / 2 up rows, activation in the epilogue
                plans.push_back(make_linear_swiglu_plan(static_cast<const bf16*>(x.p), M,
                                                        reinterpret_cast<const bf16*>(static_cast<uint8_t*>(w.p) + wbytes * c), M,
                                                        N / 2, K, static_cast<bf16*>(y.p), N / 2, limit));
                continue;
            }
            plans.push_back(make_linear_plan(static_cast<const bf16*>(x.p), M,
                                             reinterpret_cast<const bf16*>(static_cast<uint8_t*>(w.p) + wbytes * c), M, N, K,
                                             static_cast<bf16*>(y.p), N, nullptr, static_cast<float*>(ws.p),
                                             static_cast<int*>(tickets.p), limit));
            const char* dbg = tuning_env("CPMCU_LINEAR_DEBUG");
            if (dbg) plans.back().debug = atoi(dbg);
        }
        for (int c = 0; c < copies && c < 3; ++c) launch_linear(plans[c], s);
        cudaEvent_t e0, e1;
        CUDA_CHECK(cudaEventCreate(&e0));
        CUDA_CHECK(cudaEventCreate(&e1));
        CUDA_CHECK(cudaEventRecord(e0, s));
        for (int i = 0; i < iters; ++i) launch_linear(plans[i % copies], s);
        CUDA_CHECK(cudaEventRecord(e1, s));
        CUDA_CHECK(cudaStreamSynchronize(s));
        float ms = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *avg_us = ms * 1000.f / iters;
        if (w4) linear_w4_print_prof();
        sync_and_check("bench_linear");
        return 0;
    });
}

int cpmcu_bench_linear(int M, int N, int K, int copies, int iters, int grid_limit, float* avg_us) {
    return bench_linear_impl(M, N, K, copies, iters, grid_limit, avg_us, false);
}

int cpmcu_bench_linear_w4(int M, int N, int K, int copies, int iters, int grid_limit, float* avg_us) {
    return bench_linear_impl(M, N, K, copies, iters, grid_limit, avg_us, true);
}

int cpmcu_bench_linear_swiglu(int M, int inter, int K, int copies, int iters, int grid_limit, float* avg_us) {
    return bench_linear_impl(M, 2 * inter, K, copies, iters, grid_limit, avg_us, false, true);
}

int cpmcu_tree_attention(const void* q, int q_ld, const void* k_cache, const void* v_cache, int budget, int tq,
                         int hq, int hkv, const int32_t* kv_len, int kv_len_add, const int32_t* n_valid,
                         const uint64_t* mask, int mask_k, int window, int splits, void* out, int out_ld) {
    return guarded([&] {
        Runtime& rt = runtime();
        CPM_REQUIRE(splits >= 1 && splits <= 32, "attention: splits must be in [1,32]");
        const size_t rows = static_cast<size_t>(tq) * hq;
        DeviceBuf ws_o(splits > 1 ? rows * splits * 128 * sizeof(float) : 0);
        DeviceBuf ws_ml(splits > 1 ? rows * splits * 2 * sizeof(float) : 0);
        AttnPlan p = make_attn_plan(static_cast<const bf16*>(q), q_ld, static_cast<const bf16*>(k_cache),
                                    static_cast<const bf16*>(v_cache), budget, tq, hq, hkv, 128, splits,
                                    static_cast<bf16*>(out), out_ld, static_cast<float*>(ws_o.p),
                                    static_cast<float*>(ws_ml.p));
        p.kv_len = kv_len;
        p.kv_len_add = kv_len_add;
        p.n_valid = n_valid;
        p.mask = mask;
        p.mask_k = mask ? mask_k : 0;
        p.window = window;
        launch_tree_attention(p, rt.stream);
        sync_and_check("tree_attention");
        return 0;
    });
}

int cpmcu_sparse_attention(const void* q, int q_ld, const void* k_cache, const void* v_cache, int budget, int tq,
                           int hq, int hkv, const int32_t* kv_len, int kv_len_add, const uint64_t* mask, int mask_k,
                           const uint64_t* blockmask, int bm_words, int block_window, int splits, void* out,
                           int out_ld) {
    return guarded([&] {
        Runtime& rt = runtime();
        CPM_REQUIRE(splits >= 1 && splits <= 32, "attention: splits must be in [1,32]");
        CPM_REQUIRE(budget <= 262144, "block-sparse attention: at most 262144 keys");
        const size_t rows = static_cast<size_t>(tq) * hq;
        DeviceBuf ws_o(splits > 1 ? rows * splits * 128 * sizeof(float) : 0);
        DeviceBuf ws_ml(splits > 1 ? rows * splits * 2 * sizeof(float) : 0);
        AttnPlan p = make_attn_plan(static_cast<const bf16*>(q), q_ld, static_cast<const bf16*>(k_cache),
                                    static_cast<const bf16*>(v_cache), budget, tq, hq, hkv, 128, splits,
                                    static_cast<bf16*>(out), out_ld, static_cast<float*>(ws_o.p),
                                    static_cast<float*>(ws_ml.p));
        p.kv_len = kv_len;
        p.kv_len_add = kv_len_add;
        p.mask = mask;
        p.mask_k = mask ? mask_k : 0;
        p.blockmask = blockmask;
        p.bm_words = bm_words;
        p.block_window = block_window;
        launch_tree_attention(p, rt.stream);
        sync_and_check("sparse_attention");
        return 0;
    });
}

int cpmcu_sparse_select(const void* q, int q_ld, int tq, int hq, int hkv, const void* k_cache, int budget,
                        const int32_t* kv_len, int kv_len_add, int sink_window_size, int block_window_size,
                        int sparse_topk_k, int sparse_switch, int apply_compress_lse, void* c1_out, void* c2_out,
                        void* scores_out, int score_ld, uint64_t* blockmask_out, int bm_words) {
    return guarded([&] {
        Runtime& rt = runtime();
        cudaStream_t s = rt.stream;
        const int kv_dim = hkv * 128;
        CPM_REQUIRE(budget % 64 == 0 && score_ld >= (budget / 16 + 127) / 128 * 128 && score_ld % 8 == 0,
                    "sparse_select: score rows must hold budget / 16 entries rounded up to 128");
        SparseBuffers b;
        // + 16 rows: the scoring kernels read whole 16-key fragments
        DeviceBuf c1(static_cast<size_t>(budget / 16 + 16) * kv_dim * 2), c2(static_cast<size_t>(budget / 64 + 16) * kv_dim * 2);
        CUDA_CHECK(cudaMemsetAsync(c1.p, 0, static_cast<size_t>(budget / 16 + 16) * kv_dim * 2, s));
        CUDA_CHECK(cudaMemsetAsync(c2.p, 0, static_cast<size_t>(budget / 64 + 16) * kv_dim * 2, s));
        DeviceBuf done(8), scores(static_cast<size_t>(hkv) * tq * score_ld * 2);
        DeviceBuf bm(static_cast<size_t>(hkv) * tq * bm_words * 8), ptrs(2 * sizeof(void*));
        DeviceBuf lse(static_cast<size_t>(hkv) * tq * 16 * (score_ld / 128) * 8);
        CUDA_CHECK(cudaMemsetAsync(done.p, 0, 8, s));
        CUDA_CHECK(cudaMemsetAsync(scores.p, 0, static_cast<size_t>(hkv) * tq * score_ld * 2, s));
        const void* host_ptrs[2] = {k_cache, nullptr};
        CUDA_CHECK(cudaMemcpyAsync(ptrs.p, host_ptrs, sizeof(host_ptrs), cudaMemcpyHostToDevice, s));
        b.c1 = static_cast<bf16*>(c1.p);
        b.c2 = apply_compress_lse ? static_cast<bf16*>(c2.p) : nullptr;
        b.done = static_cast<int32_t*>(done.p);
        b.scores = static_cast<bf16*>(scores.p);
        b.lse = static_cast<float2*>(lse.p);
        b.score_ld = score_ld;
        b.blockmask = static_cast<uint64_t*>(bm.p);
        b.bm_words = bm_words;
        b.max_tokens = tq;
        SparseConfig cfg;
        cfg.enabled = true;
        cfg.sink_blocks = sink_window_size;
        cfg.window_blocks = block_window_size;
        cfg.topk = sparse_topk_k;
        cfg.sparse_switch = sparse_switch;
        cfg.compress_lse = apply_compress_lse != 0;
        launch_sparse_compress(b, static_cast<bf16* const*>(ptrs.p), 1, kv_dim, kv_len, kv_len_add, budget / 16, s);
        launch_sparse_select(b, cfg, 0, static_cast<const bf16*>(q), q_ld, tq, hq, hkv, kv_len, kv_len_add, nullptr, s);
        if (c1_out) CUDA_CHECK(cudaMemcpyAsync(c1_out, c1.p, static_cast<size_t>(budget / 16) * kv_dim * 2, cudaMemcpyDeviceToDevice, s));
        if (c2_out && apply_compress_lse) {
            CUDA_CHECK(cudaMemcpyAsync(c2_out, c2.p, static_cast<size_t>(budget / 64) * kv_dim * 2, cudaMemcpyDeviceToDevice, s));
        }
        if (scores_out) {
            CUDA_CHECK(cudaMemcpyAsync(scores_out, scores.p, static_cast<size_t>(hkv) * tq * score_ld * 2, cudaMemcpyDeviceToDevice, s));
        }
        CUDA_CHECK(cudaMemcpyAsync(blockmask_out, bm.p, static_cast<size_t>(hkv) * tq * bm_words * 8, cudaMemcpyDeviceToDevice, s));
        sync_and_check("sparse_select");
        return 0;
    });
}

int cpmcu_bench_attention(int tq, int hq, int hkv, int kv_total, int splits, int with_mask, int iters, float* avg_us) {
    return guarded([&] {
        Runtime& rt = runtime();
        cudaStream_t s = rt.stream;
        const int budget = (kv_total + 255) / 128 * 128;
        const int q_ld = (hq + 2 * hkv) * 128;
        const size_t kv_bytes = static_cast<size_t>(budget) * hkv * 128 * 2;
        const int layers = 8;  // rotate over several caches like consecutive layers do
        DeviceBuf q(static_cast<size_t>(tq) * q_ld * 2), k(kv_bytes * layers), v(kv_bytes * layers);
        DeviceBuf out(static_cast<size_t>(tq) * hq * 128 * 2), len(4), mask(64 * 8);
        const size_t rows = static_cast<size_t>(tq) * hq;
        DeviceBuf ws_o(rows * splits * 128 * 4), ws_ml(rows * splits * 2 * 4);
        CUDA_CHECK(cudaMemsetAsync(q.p, 0x3c, static_cast<size_t>(tq) * q_ld * 2, s));
        CUDA_CHECK(cudaMemsetAsync(k.p, 0x3c, kv_bytes * layers, s));
        CUDA_CHECK(cudaMemsetAsync(v.p, 0x3c, kv_bytes * layers, s));
        CUDA_CHECK(cudaMemcpyAsync(len.p, &kv_total, 4, cudaMemcpyHostToDevice, s));
        uint64_t hm[64];
        for (int i = 0; i < 64; ++i) hm[i] = (1ull << i) | 1ull;
        CUDA_CHECK(cudaMemcpyAsync(mask.p, hm, sizeof(hm), cudaMemcpyHostToDevice, s));
        std::vector<AttnPlan> plans;
        for (int l = 0; l < layers; ++l) {
            AttnPlan p = make_attn_plan(static_cast<const bf16*>(q.p), q_ld,
                                        reinterpret_cast<const bf16*>(static_cast<uint8_t*>(k.p) + kv_bytes * l),
                                        reinterpret_cast<const bf16*>(static_cast<uint8_t*>(v.p) + kv_bytes * l), budget, tq,
                                        hq, hkv, 128, splits, static_cast<bf16*>(out.p), hq * 128,
                                        static_cast<float*>(ws_o.p), static_cast<float*>(ws_ml.p));
            p.kv_len = static_cast<const int32_t*>(len.p);
            if (with_mask) {
                p.mask = static_cast<const uint64_t*>(mask.p);
                p.mask_k = tq;
            }
            plans.push_back(p);
        }
        for (int l = 0; l < 3; ++l) launch_tree_attention(plans[l], s);
        cudaEvent_t e0, e1;
        CUDA_CHECK(cudaEventCreate(&e0));
        CUDA_CHECK(cudaEventCreate(&e1));
        CUDA_CHECK(cudaEventRecord(e0, s));
        for (int i = 0; i < iters; ++i) launch_tree_attention(plans[i % layers], s);
        CUDA_CHECK(cudaEventRecord(e1, s));
        CUDA_CHECK(cudaStreamSynchronize(s));
        float ms = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        *avg_us = ms * 1000.f / iters;
        sync_and_check("bench_attention");
        return 0;
    });
}

int cpmcu_rms_norm(void* x, const void* delta, float delta_scale, const void* weight, void* y, int rows, int dim,
                   float eps) {
    return guarded([&] {
        cudaStream_t s = runtime().stream;
        if (delta) launch_add_rms_norm(static_cast<bf16*>(x), static_cast<const bf16*>(delta), delta_scale,
                                       static_cast<const bf16*>(weight), static_cast<bf16*>(y), rows, dim, eps, s);
        else launch_rms_norm(static_cast<const bf16*>(x), dim, static_cast<const bf16*>(weight), static_cast<bf16*>(y), dim,
                             rows, dim, eps, s);
        sync_and_check("rms_norm");
        return 0;
    });
}

int cpmcu_rope_append(void* qkv, int rows, int hq, int hkv, const float* inv_freq, const int32_t* pos, void* k_cache,
                      void* v_cache, const int32_t* kv_len, int kv_off) {
    return guarded([&] {
        launch_rope_append(static_cast<bf16*>(qkv), rows, hq, hkv, 128, inv_freq, pos, nullptr, 0, 0,
                           static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), kv_len, kv_off, nullptr,
                           0x7fffffff, runtime().stream);
        sync_and_check("rope_append");
        return 0;
    });
}

int cpmcu_silu_gate(const void* gate_up, void* out, int rows, int inter) {
    return guarded([&] {
        launch_silu_gate(static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), rows, inter, runtime().stream);
        sync_and_check("silu_gate");
        return 0;
    });
}

int cpmcu_sample(const void* logits, int rows, int vocab, float temperature, unsigned long long seed, int draw,
                 int32_t* out) {
    return guarded([&] {
        CPM_REQUIRE(temperature >= 0.f && draw >= 0, "sample: temperature and draw index must not be negative");
        DeviceBuf ws(argmax_workspace_bytes(rows, vocab));
        launch_sample(static_cast<const bf16*>(logits), rows, vocab, vocab, out, ws.p, temperature, seed, nullptr, draw,
                      runtime().stream);
        sync_and_check("sample");
        return 0;
    });
}

int cpmcu_argmax(const void* logits, int rows, int vocab, int32_t* out) {
    return guarded([&] {
        DeviceBuf ws(argmax_workspace_bytes(rows, vocab));
        launch_argmax(static_cast<const bf16*>(logits), rows, vocab, vocab, out, ws.p, runtime().stream);
        sync_and_check("argmax");
        return 0;
    });
}

int cpmcu_draft_tree_from_logits(const void* logits, int vocab, int k, int num_iter, int tree_size,
                                 const int32_t* token_id_remap, const int32_t* cache_length, int32_t* tree_ids,
                                 int32_t* tree_pos, uint64_t* tree_mask, int32_t* tree_parent, void* tried_val,
                                 int32_t* tried_pos, int32_t* tried_parent) {
    return guarded([&] {
        Runtime& rt = runtime();
        cudaStream_t s = rt.stream;
        CPM_REQUIRE(k >= 1 && k <= 32 && num_iter >= 1 && k * num_iter <= 64, "draft tree: k / num_iter out of range");
        CPM_REQUIRE(tree_size >= 2 && tree_size <= 64, "draft tree: tree_size out of range");
        DraftTreeState st;
        st.k = k;
        st.num_iter = num_iter;
        st.tree_size = tree_size;
        st.total_tried = k + k * k * (num_iter - 1);
        CPM_REQUIRE(tree_size - 1 <= st.total_tried, "draft tree: tree larger than the candidate set");
        const int hidden = 8;  // dummy hidden rows: the hidden-state gather is exercised but unused
        DeviceBuf tv((st.total_tried + 64) * 2), tp((st.total_tried + 64) * 4), tpar((k * num_iter + 64) * 4);
        DeviceBuf fs(64 * 2), fi(64 * 4), fm(64 * 8), sp(64 * 4), fsrc(64 * 4);
        DeviceBuf h(static_cast<size_t>(32) * hidden * 2), hid(static_cast<size_t>(32) * hidden * 2);
        DeviceBuf scan(draft_scan_workspace_bytes(32, vocab, 32));
        CUDA_CHECK(cudaMemsetAsync(scan.p, 0, 256, runtime().stream));  // the level kernel's ticket
        CUDA_CHECK(cudaMemsetAsync(h.p, 0, static_cast<size_t>(32) * hidden * 2, s));
        st.tried_val = static_cast<bf16*>(tv.p);
        st.tried_pos = static_cast<int32_t*>(tp.p);
        st.tried_parent = static_cast<int32_t*>(tpar.p);
        st.fr_score = static_cast<bf16*>(fs.p);
        st.fr_id = static_cast<int32_t*>(fi.p);
        st.fr_mask = static_cast<uint64_t*>(fm.p);
        st.fr_src = static_cast<int32_t*>(fsrc.p);
        st.sel_pos = static_cast<int32_t*>(sp.p);
        st.token_id_remap = token_id_remap;
        const bf16* lg = static_cast<const bf16*>(logits);
        for (int d = 0; d < num_iter; ++d) {
            const bf16* rows = (d == 0) ? lg : lg + static_cast<size_t>(1 + (d - 1) * k) * vocab;
            launch_draft_topk_expand(st, rows, vocab, vocab, d, scan.p, static_cast<bf16*>(h.p), hidden, nullptr,
                                     static_cast<bf16*>(hid.p), hidden, hidden, s);
        }
        launch_tree_finalize(st, cache_length, tree_ids, tree_pos, tree_mask, tree_parent, s);
        if (tried_val) CUDA_CHECK(cudaMemcpyAsync(tried_val, st.tried_val, st.total_tried * 2, cudaMemcpyDeviceToDevice, s));
        if (tried_pos) CUDA_CHECK(cudaMemcpyAsync(tried_pos, st.tried_pos, st.total_tried * 4, cudaMemcpyDeviceToDevice, s));
        if (tried_parent && num_iter > 1) {
            CUDA_CHECK(cudaMemcpyAsync(tried_parent, st.tried_parent, static_cast<size_t>(k) * (num_iter - 1) * 4,
                                       cudaMemcpyDeviceToDevice, s));
        }
        sync_and_check("draft_tree_from_logits");
        return 0;
    });
}

int cpmcu_accept_fixup(int tree_size, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                       const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent,
                       void* const* caches, int num_caches, int kv_dim, int cache_rows, int max_accept, int hidden,
                       const void* norm_out, void* prev_hidden, const void* embed_table, float embed_scale,
                       void* prev_embed, int32_t* eagle_pos, int32_t* result) {
    return guarded([&] {
        cudaStream_t s = runtime().stream;
        AcceptIO io;
        io.tree_size = tree_size;
        io.pred = pred;
        io.gt = gt;
        io.position_ids = position_ids;
        io.cache_length = cache_length;
        io.attn_mask = attn_mask;
        io.tree_parent = tree_parent;
        io.result = result;
        FixupArgs f;
        f.caches = reinterpret_cast<bf16* const*>(caches);
        f.num_caches = num_caches;
        f.kv_dim = num_caches > 0 ? kv_dim : 8;
        f.max_accept = max_accept;
        f.hidden = hidden;
        if (hidden > 0) {
            CPM_REQUIRE(norm_out && prev_hidden && embed_table && prev_embed && eagle_pos,
                        "accept_fixup: hidden > 0 needs the hidden-state and embedding buffers");
            f.norm_out = static_cast<const bf16*>(norm_out);
            f.prev_hidden = static_cast<bf16*>(prev_hidden);
            f.embed_table = static_cast<const bf16*>(embed_table);
            f.embed_scale = embed_scale;
            f.prev_embed = static_cast<bf16*>(prev_embed);
            f.eagle_pos = eagle_pos;
        }
        launch_accept_fixup(io, f, cache_rows, s);
        sync_and_check("accept_fixup");
        return 0;
    });
}

int cpmcu_verify_and_compact(int tree_size, int32_t* pred, const int32_t* gt, const int32_t* position_ids,
                             const int32_t* cache_length, const uint64_t* attn_mask, const int32_t* tree_parent,
                             void* const* caches, int num_caches, int kv_dim, int max_accept, int32_t* result) {
    return cpmcu_accept_fixup(tree_size, pred, gt, position_ids, cache_length, attn_mask, tree_parent, caches, num_caches,
                              kv_dim, 0x7fffffff, max_accept, 0, nullptr, nullptr, nullptr, 1.f, nullptr, nullptr, result);
}

}  // extern "C"
