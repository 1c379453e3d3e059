// Engine: storage layout, weight loading, prefill, tree-verify forward, EAGLE
// draft loop, acceptance and the captured speculative step.  See engine.cuh for
// the reference interfaces this mirrors.
#include "engine.cuh"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <regex>

namespace {

__global__ void state_sync_kernel(int32_t* st, const int32_t* cache_length, int32_t* tree_ids, int fused) {
    grid_dependency_sync();
    // S_L=0, S_NPREV=1, S_BASE=2, S_LASTROW=3, S_ACCEPT=4
    const int n = st[4];
    int L;
    if (fused) {
        L = st[0] + n;
        if (n > 0) tree_ids[0] = tree_ids[n - 1];  // new root = bonus token of the previous step
    } else {
        L = cache_length[0];
    }
    st[0] = L;
    st[1] = n;
    st[2] = L - n;
    st[3] = (n > 0) ? n - 1 : 0;
    if (fused) st[8] += 1;  // S_DRAW: index of this step's sampling draw
}

__global__ void publish_kernel(const int32_t* result, const int32_t* tokens, const int* error, int32_t* st,
                               int32_t* out) {
    grid_dependency_sync();
    const int n = result[0];
    if (threadIdx.x == 0) {
        st[4] = n;
        out[0] = n;
        out[31] = *error;
    }
    if (threadIdx.x < 16) out[1 + threadIdx.x] = (threadIdx.x < n) ? tokens[threadIdx.x] : -1;
}

// The engine's split-K counters (two per output tile) live in one buffer of kTicketInts ints.
constexpr int kTicketInts = 1 << 16;
LinearPlan checked(const LinearPlan& p) {
    CPM_REQUIRE(2LL * ceil_div(p.N, 128) * ceil_div(p.M, p.mt) <= kTicketInts,
                "linear: more output tiles than the engine's split-K counters cover");
    return p;
}

void copy_rows(bf16* dst, int ld_dst, const bf16* src, int ld_src, int rows, int dim, cudaStream_t s) {
    if (rows <= 0) return;
    CUDA_CHECK(cudaMemcpy2DAsync(dst, static_cast<size_t>(ld_dst) * 2, src, static_cast<size_t>(ld_src) * 2,
                                 static_cast<size_t>(dim) * 2, rows, cudaMemcpyDeviceToDevice, s));
}

}  // namespace

// ------------------------------------------------------------------ memory
void* Engine::Pool::take(size_t bytes) {
    const size_t off = (used + 255) & ~size_t(255);
    used = off + bytes;
    if (counting) return nullptr;
    if (used > cap) throw std::runtime_error("cpmcu_b200: device pool overflow");
    return base + off;
}

Engine::Engine(const ModelConfig& mc) : mc_(mc) {
    CPM_REQUIRE(mc.head_dim == 128, "only head_dim 128 is supported");
    CPM_REQUIRE(mc.hidden % 64 == 0 && mc.inter % 64 == 0, "hidden and intermediate sizes must be multiples of 64");
    CPM_REQUIRE(mc.hq % mc.hkv == 0, "num_attention_heads must be a multiple of num_key_value_heads");
    CPM_REQUIRE((mc.hq * mc.head_dim) % 64 == 0, "attention width must be a multiple of 64");
    if (mc.w4a16) {
        CPM_REQUIRE(mc.group_size == 128, "W4A16: only group_size 128 is supported");
        CPM_REQUIRE(mc.hidden % 256 == 0 && mc.inter % 256 == 0 && (mc.hq * mc.head_dim) % 256 == 0,
                    "W4A16: hidden, intermediate and attention widths must be multiples of 256");
    }
    qkv_dim_ = (mc.hq + 2 * mc.hkv) * mc.head_dim;
    layers_.resize(mc.layers);
    kv_.resize(mc.layers);
    runtime();
}

Engine::~Engine() {
    if (step_graph_) cudaGraphExecDestroy(step_graph_);
    if (ev0_) cudaEventDestroy(ev0_);
    if (ev1_) cudaEventDestroy(ev1_);
    if (ev_mid_) cudaEventDestroy(ev_mid_);
    if (pool_.base) cudaFree(pool_.base);
    if (h_result_) cudaFreeHost(h_result_);
}

void Engine::attach_eagle(const EagleConfig& ec) {
    CPM_REQUIRE(!storage_ready_, "attach the drafter before init_storage");
    CPM_REQUIRE(ec.num_layers == 1, "only a 1-layer EAGLE drafter is supported");
    CPM_REQUIRE(ec.tree_size >= 2 && ec.tree_size <= 64, "tree_size must be in [2,64]");
    CPM_REQUIRE(ec.topk >= 1 && ec.topk <= 32 && ec.topk <= ec.tree_size - 1, "topk_per_iter out of range");
    CPM_REQUIRE(ec.num_iter >= 1 && ec.num_iter <= 15, "num_iter out of range");
    CPM_REQUIRE(ec.topk * ec.num_iter <= 64, "draft keys (topk * num_iter) exceed the 64-bit mask");
    if (ec.quant) {
        CPM_REQUIRE(ec.group_size == 128, "W4A16 drafter: only group_size 128 is supported");
        CPM_REQUIRE(mc_.hidden % 256 == 0 && mc_.inter % 256 == 0 && (mc_.hq * mc_.head_dim) % 256 == 0 && mc_.hidden % 128 == 0,
                    "W4A16 drafter: hidden, intermediate and attention widths must be multiples of 256");
    }
    ec_ = ec;
    has_eagle_ = true;
    draft_vocab_ = (ec.frspec_vocab > 0 && ec.frspec_vocab != mc_.vocab) ? ec.frspec_vocab : mc_.vocab;
    tree_.k = ec.topk;
    tree_.num_iter = ec.num_iter;
    tree_.tree_size = ec.tree_size;
    tree_.total_tried = ec.topk + ec.topk * ec.topk * (ec.num_iter - 1);
    CPM_REQUIRE(tree_.total_tried <= 2048, "too many draft candidates");
    catchup_rows_ = ec.num_iter + 1;
}

int Engine::attn_splits_for(int rows) const {
    const int grp = mc_.hq / mc_.hkv;
    const int mtiles = ceil_div(rows, 128 / grp) * mc_.hkv;
    int s = runtime().num_sms / mtiles;
    // bench only: sweep the number of key splits of the verify-sized (more than 16 rows) and the draft-sized passes
    static const char* forced = tuning_env("CPMCU_ATTN_SPLITS");
    static const char* forced_draft = tuning_env("CPMCU_ATTN_SPLITS_DRAFT");
    if (rows > 16 && forced && atoi(forced) >= 1) s = atoi(forced);
    if (rows <= 16 && forced_draft && atoi(forced_draft) >= 1) s = atoi(forced_draft);
    // the draft-sized passes (4 token tiles) measured best with 24 splits: 1.460 ms for the draft half of the 8B step
    // against 1.472 with 32 and 1.468 with 16
    return std::max(1, std::min(s, (forced_draft && rows <= 16) ? 32 : 24));
}

void Engine::lay_out(Pool& p) {
    const int H = mc_.hidden, I = mc_.inter, V = mc_.vocab, d = mc_.head_dim;
    const int kvd = mc_.hkv * d;
    const size_t R = max_rows_;
    // weights
    embed_ = take<bf16>(p, static_cast<size_t>(V) * H);
    lm_head_ = take<bf16>(p, linear_weight_elems(V, H));   // GEMM weights are tile-major, rows padded to 128
    final_norm_ = take<bf16>(p, H);
    inv_freq_ = take<float>(p, d / 2);
    for (auto& w : layers_) {
        if (mc_.w4a16) {
            w.qkv_q = take<uint8_t>(p, linear_w4_weight_bytes(qkv_dim_, H));
            w.o_q = take<uint8_t>(p, linear_w4_weight_bytes(H, mc_.hq * d));
            w.gate_up_q = take<uint8_t>(p, linear_w4_weight_bytes(2 * I, H));
            w.down_q = take<uint8_t>(p, linear_w4_weight_bytes(H, I));
        } else {
            w.qkv = take<bf16>(p, linear_weight_elems(qkv_dim_, H));
            w.o = take<bf16>(p, linear_weight_elems(H, mc_.hq * d));
            w.gate_up = take<bf16>(p, gate_up_elems());
            w.down = take<bf16>(p, linear_weight_elems(H, I));
        }
        w.ln_attn = take<bf16>(p, H);
        w.ln_ffn = take<bf16>(p, H);
    }
    if (has_eagle_) {
        fc_bias_ = take<bf16>(p, H);
        in_norm1_ = take<bf16>(p, H);
        in_norm2_ = take<bf16>(p, H);
        if (ec_.quant) {
            fc1_q_ = take<uint8_t>(p, linear_w4_weight_bytes(H, H));
            fc2_q_ = take<uint8_t>(p, linear_w4_weight_bytes(H, H));
            elayer_.qkv_q = take<uint8_t>(p, linear_w4_weight_bytes(qkv_dim_, H));
            elayer_.o_q = take<uint8_t>(p, linear_w4_weight_bytes(H, mc_.hq * d));
            elayer_.gate_up_q = take<uint8_t>(p, linear_w4_weight_bytes(2 * I, H));
            elayer_.down_q = take<uint8_t>(p, linear_w4_weight_bytes(H, I));
        } else {
            fc_ = take<bf16>(p, linear_weight_elems(H, 2 * H));
            elayer_.qkv = take<bf16>(p, linear_weight_elems(qkv_dim_, H));
            elayer_.o = take<bf16>(p, linear_weight_elems(H, mc_.hq * d));
            elayer_.gate_up = take<bf16>(p, gate_up_elems());
            elayer_.down = take<bf16>(p, linear_weight_elems(H, I));
        }
        elayer_.ln_attn = take<bf16>(p, H);
        elayer_.ln_ffn = take<bf16>(p, H);
        token_id_remap_ = take<int32_t>(p, draft_vocab_);
        bf16* dl = (draft_vocab_ != V) ? take<bf16>(p, linear_weight_elems(draft_vocab_, H)) : lm_head_;
        draft_lm_head_ = dl;
    }
    // activations
    x_ = take<bf16>(p, R * H);
    normed_ = take<bf16>(p, R * H);
    qkv_ = take<bf16>(p, R * qkv_dim_);
    attn_out_ = take<bf16>(p, R * mc_.hq * d);
    delta_ = take<bf16>(p, R * H);
    gate_up_ = take<bf16>(p, R * 2 * I);
    act_ = take<bf16>(p, R * I);
    norm_out_ = take<bf16>(p, R * H);
    lm_in_ = take<bf16>(p, static_cast<size_t>(64) * H);
    logits_ = take<bf16>(p, static_cast<size_t>(64) * V);
    gemm_ws_ = reinterpret_cast<float*>(p.take(linear_workspace_bytes(256, runtime().num_sms)));
    tickets_ = take<int>(p, kTicketInts);
    {
        size_t a = 0;
        for (int rows = 1; rows <= 64; ++rows) {
            a = std::max(a, attn_workspace_bytes(rows, mc_.hq, d, attn_splits_for(rows)));
        }
        attn_ws_o_ = reinterpret_cast<float*>(p.take(a));
        attn_ws_ml_ = reinterpret_cast<float*>(p.take(a / 32 + 1024));
    }
    st_ = take<int32_t>(p, S_COUNT);
    d_cache_ptrs_ = reinterpret_cast<bf16**>(p.take(sizeof(bf16*) * 2 * mc_.layers));
    t_ids_ = take<int32_t>(p, 64);
    t_pos_ = take<int32_t>(p, 64);
    t_parent_ = take<int32_t>(p, 64);
    t_gt_ = take<int32_t>(p, 64);
    t_mask_ = take<uint64_t>(p, 64);
    accept_result_ = take<int32_t>(p, 32);
    argmax_ws_ = p.take(argmax_workspace_bytes(64, V));
    d_publish_ = take<int32_t>(p, 32);
    if (has_eagle_) {
        e_in_ = take<bf16>(p, R * 2 * H);
        e_x_ = take<bf16>(p, R * H);
        e_h_ = take<bf16>(p, R * H);
        e_hid_ = take<bf16>(p, static_cast<size_t>(32) * H);
        e_emb_ = take<bf16>(p, static_cast<size_t>(32) * H);
        prev_embed_ = take<bf16>(p, R * H);
        prev_hidden_ = take<bf16>(p, R * H);
        e_logits_ = take<bf16>(p, static_cast<size_t>(32) * draft_vocab_);
        eagle_pos_ = take<int32_t>(p, R);
        scan_ws_ = p.take(draft_scan_workspace_bytes(32, draft_vocab_, 32));
        tree_.tried_val = take<bf16>(p, tree_.total_tried + 64);
        tree_.tried_pos = take<int32_t>(p, tree_.total_tried + 64);
        tree_.tried_parent = take<int32_t>(p, ec_.topk * ec_.num_iter + 64);
        tree_.fr_score = take<bf16>(p, 64);
        tree_.fr_id = take<int32_t>(p, 64);
        tree_.fr_mask = take<uint64_t>(p, 64);
        tree_.fr_src = take<int32_t>(p, 64);
        tree_.sel_pos = take<int32_t>(p, 64);
    }
    // KV caches last: everything that is left up to the budget
    for (auto& c : kv_) {
        c.k = take<bf16>(p, static_cast<size_t>(budget_) * kvd);
        c.v = take<bf16>(p, static_cast<size_t>(budget_) * kvd);
    }
    if (has_eagle_) {
        ekv_.k = take<bf16>(p, static_cast<size_t>(budget_) * kvd);
        ekv_.v = take<bf16>(p, static_cast<size_t>(budget_) * kvd);
    }
    if (mc_.sparse.enabled) {
        // compressed key caches per layer, and the scores / block masks of the layer being run
        sp_.c1_layer_stride = static_cast<size_t>(budget_ / 16) * kvd;
        sp_.c2_layer_stride = static_cast<size_t>(budget_ / 64) * kvd;
        // + 16 rows: the scoring kernels read whole 16-key fragments
        sp_.c1 = take<bf16>(p, sp_.c1_layer_stride * mc_.layers + static_cast<size_t>(16) * kvd);
        sp_.c2 = mc_.sparse.compress_lse ? take<bf16>(p, sp_.c2_layer_stride * mc_.layers + static_cast<size_t>(16) * kvd) : nullptr;
        sp_.done = take<int32_t>(p, 2);
        sp_.score_ld = (budget_ / 16 + 127) / 128 * 128;
        sp_.max_tokens = static_cast<int>(R);
        sp_.scores = take<bf16>(p, static_cast<size_t>(mc_.hkv) * R * sp_.score_ld + 8);
        sp_.lse = reinterpret_cast<float2*>(p.take(static_cast<size_t>(mc_.hkv) * R * 16 * (sp_.score_ld / 128) * sizeof(float2)));
        sp_.bm_words = std::max(1, (budget_ / 64 + 63) / 64);
        sp_.blockmask = take<uint64_t>(p, static_cast<size_t>(mc_.hkv) * R * sp_.bm_words);
    }
}

int Engine::init_storage() {
    CPM_REQUIRE(!storage_ready_, "init_storage called twice");
    Runtime& rt = runtime();
    max_rows_ = std::max(mc_.chunk_length, 64);
    size_t free_b = 0, total_b = 0;
    CUDA_CHECK(cudaMemGetInfo(&free_b, &total_b));
    const size_t limit = std::min(static_cast<size_t>(static_cast<double>(total_b) * mc_.memory_limit), free_b);
    // size of everything except the KV caches
    budget_ = 0;
    Pool count;
    lay_out(count);
    const size_t fixed = count.used + (1 << 20);
    size_t per_token = static_cast<size_t>(mc_.layers + (has_eagle_ ? 1 : 0)) * 2 * mc_.hkv * mc_.head_dim * 2;
    if (mc_.sparse.enabled) {
        // c1 + c2 rows per layer (1/16 + 1/64 of a key row), one score per 16 tokens and one mask bit per 64
        // tokens for each of the hkv * max_rows_ (kv head, query) pairs
        per_token += static_cast<size_t>(mc_.layers) * mc_.hkv * mc_.head_dim * 2 * 5 / 64 + 1;
        per_token += static_cast<size_t>(mc_.hkv) * max_rows_ * 2 / 16 + static_cast<size_t>(mc_.hkv) * max_rows_ / 512 + 2;
    }
    if (fixed + per_token * 256 > limit) {
        throw std::runtime_error("cpmcu_b200: memory_limit too small for the model (" + std::to_string(fixed >> 20) +
                                 " MiB needed before any KV cache)");
    }
    size_t tokens = (limit - fixed) / per_token;
    const char* cap_env = getenv("CPMCU_MAX_TOKENS");
    const size_t cap = cap_env ? static_cast<size_t>(atoll(cap_env)) : (size_t(1) << 20);
    tokens = std::min(tokens, cap);
    if (mc_.sparse.enabled) tokens = std::min<size_t>(tokens, 262144);  // 4096 selectable blocks, 2048 key tiles
    tokens = tokens / 128 * 128;
    budget_ = static_cast<int>(tokens);
    Pool measure;
    lay_out(measure);
    pool_.cap = measure.used + 4096;
    CUDA_CHECK(cudaMalloc(&pool_.base, pool_.cap));
    pool_.counting = false;
    pool_.used = 0;
    lay_out(pool_);
    // KV rows past the valid length are multiplied by zero probabilities, so they
    // must hold finite values: clear the caches (and everything else) once.
    CUDA_CHECK(cudaMemsetAsync(pool_.base, 0, pool_.cap, rt.stream));
    std::vector<bf16*> ptrs;
    for (auto& c : kv_) { ptrs.push_back(c.k); ptrs.push_back(c.v); }
    CUDA_CHECK(cudaMemcpyAsync(d_cache_ptrs_, ptrs.data(), ptrs.size() * sizeof(bf16*), cudaMemcpyHostToDevice,
                               rt.stream));
    CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    CUDA_CHECK(cudaMallocHost(&h_result_, 32 * sizeof(int32_t)));
    memset(h_result_, 0, 32 * sizeof(int32_t));
    CUDA_CHECK(cudaEventCreate(&ev0_));
    CUDA_CHECK(cudaEventCreate(&ev1_));
    CUDA_CHECK(cudaEventCreate(&ev_mid_));
    storage_ready_ = true;

    if (has_eagle_) {
        tree_.token_id_remap = (draft_vocab_ != mc_.vocab) ? token_id_remap_ : nullptr;
        const int H = mc_.hidden, k = ec_.topk, rc = catchup_rows_;
        build_draft_plans(eplan_level_, k, attn_splits_for(k));
        build_draft_plans(eplan_catchup_, rc, attn_splits_for(rc));
        eplan_level_.attn.window = ec_.window;
        eplan_catchup_.attn.window = ec_.window;
        if (ec_.quant) {
            fc_plan_level_ = checked(make_linear_plan_w4(e_in_, k, fc1_q_, k, H, H, e_x_, H, gemm_ws_, tickets_, rt.num_sms));
            fc2_plan_level_ = checked(make_linear_plan_w4(ein_hidden(), k, fc2_q_, k, H, H, delta_, H, gemm_ws_, tickets_, rt.num_sms));
            fc_plan_catchup_ = checked(make_linear_plan_w4(e_in_, rc, fc1_q_, rc, H, H, e_x_, H, gemm_ws_, tickets_, rt.num_sms));
            fc2_plan_catchup_ = checked(make_linear_plan_w4(ein_hidden(), rc, fc2_q_, rc, H, H, delta_, H, gemm_ws_, tickets_, rt.num_sms));
        } else {
            fc_plan_level_ = checked(make_linear_plan(e_in_, k, fc_, k, H, 2 * H, e_x_, H, fc_bias_, gemm_ws_, tickets_, rt.num_sms));
            fc_plan_catchup_ = checked(make_linear_plan(e_in_, rc, fc_, rc, H, 2 * H, e_x_, H, fc_bias_, gemm_ws_, tickets_, rt.num_sms));
        }
        const bool scale_in = (!ec_.minicpm4_variant && mc_.scale_lmhead != 1.0f);
        const bf16* lm_x = scale_in ? lm_in_ : e_h_;
        dlm_plan_level_ = checked(make_linear_plan(lm_x, k, draft_lm_head_, k, draft_vocab_, H, e_logits_, draft_vocab_, nullptr,
                                           gemm_ws_, tickets_, rt.num_sms));
        dlm_plan_catchup_ = checked(make_linear_plan(lm_x, rc, draft_lm_head_, rc, draft_vocab_, H, e_logits_, draft_vocab_,
                                             nullptr, gemm_ws_, tickets_, rt.num_sms));
    }
    return budget_;
}

// ------------------------------------------------------------------ loading
void Engine::load(const std::string& name, const void* src) {
    CPM_REQUIRE(storage_ready_, "load_model before init_storage");
    Runtime& rt = runtime();
    const int H = mc_.hidden, I = mc_.inter, d = mc_.head_dim;
    auto copy = [&](void* dst, size_t bytes) {
        CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, rt.stream));
        CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    };
    auto load_quant_layer = [&](LayerWeights& w, const std::string& key, const std::string& sub) -> bool {
        // fused W4A16 tensors of the reference converter: qkv_proj, o_proj, gate_up_proj, down_proj
        const bool is_scales = sub.find("scales") != std::string::npos;
        if (!is_scales && sub.find("qweight") == std::string::npos) return false;
        if (sub.find("qkv_proj") != std::string::npos) load_quantized(key + ".qkv", is_scales, src, H, qkv_dim_, w.qkv_q);
        else if (sub.find("o_proj") != std::string::npos) load_quantized(key + ".o", is_scales, src, mc_.hq * d, H, w.o_q);
        else if (sub.find("gate_up_proj") != std::string::npos) load_quantized(key + ".gu", is_scales, src, H, 2 * I, w.gate_up_q);
        else if (sub.find("down_proj") != std::string::npos) load_quantized(key + ".down", is_scales, src, I, H, w.down_q);
        else throw std::invalid_argument("Unsupported quantized tensor " + sub);
        return true;
    };
    // a GEMM weight (or the rows / columns one checkpoint tensor contributes to a fused one) into the tile-major layout
    auto retile = [&](bf16* dst, int rows, int src_cols, int K, int mode, int row_offset, int k_offset) {
        retile_weight_rows(src, rows, src_cols, dst, K, mode, row_offset, k_offset, rt.stream);
        CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    };
    auto load_layer = [&](LayerWeights& w, const std::string& sub) {
        const int qr = mc_.hq * d, kr = mc_.hkv * d;
        // gate and up rows share the tiles of their 64-feature groups (SwiGLU epilogue) when the width allows
        const bool il = gate_up_interleaved();
        if (sub.find("q_proj") != std::string::npos) retile(w.qkv, qr, H, H, 0, 0, 0);
        else if (sub.find("k_proj") != std::string::npos) retile(w.qkv, kr, H, H, 0, qr, 0);
        else if (sub.find("v_proj") != std::string::npos) retile(w.qkv, kr, H, H, 0, qr + kr, 0);
        else if (sub.find("o_proj") != std::string::npos) retile(w.o, H, mc_.hq * d, mc_.hq * d, 0, 0, 0);
        else if (sub.find("gate_proj") != std::string::npos) retile(w.gate_up, I, H, H, il ? 1 : 0, 0, 0);
        else if (sub.find("up_proj") != std::string::npos) retile(w.gate_up, I, H, H, il ? 2 : 0, il ? 0 : I, 0);
        else if (sub.find("down_proj") != std::string::npos) retile(w.down, H, I, I, 0, 0, 0);
        else if (sub.find("input_layernorm") != std::string::npos) copy(w.ln_attn, static_cast<size_t>(H) * 2);
        else if (sub.find("post_attention_layernorm") != std::string::npos) copy(w.ln_ffn, static_cast<size_t>(H) * 2);
        else throw std::invalid_argument("Unsupported name " + sub);
    };
    static const std::regex layer_re("layers\\.(\\d+)\\.(.*)");
    std::smatch m;
    if (name.rfind("eagle", 0) == 0) {
        CPM_REQUIRE(has_eagle_, "eagle weight given but no drafter was initialised");
        if (ec_.quant && (name.rfind("eagle.fc1", 0) == 0 || name.rfind("eagle.fc2", 0) == 0) &&
            name.find("bias") == std::string::npos) {
            const bool second = name.rfind("eagle.fc2", 0) == 0;
            const bool is_scales = name.find("scales") != std::string::npos;
            CPM_REQUIRE(is_scales || name.find("qweight") != std::string::npos, "Unsupported name " + name);
            load_quantized(second ? "E.fc2" : "E.fc1", is_scales, src, H, H, second ? fc2_q_ : fc1_q_);
        } else if (name.rfind("eagle.fc1", 0) == 0) {
            if (name.find("weight") != std::string::npos) {
                retile(fc_, H, H, 2 * H, 0, 0, 0);   // columns [0, H) of the fused [H, 2H] matrix
            } else if (name.find("bias") != std::string::npos) {
                copy(fc_bias_, static_cast<size_t>(H) * 2);
            } else throw std::invalid_argument("Unsupported name " + name);
        } else if (name.rfind("eagle.fc2", 0) == 0) {
            CPM_REQUIRE(name.find("weight") != std::string::npos, "Unsupported name " + name);
            retile(fc_, H, H, 2 * H, 0, 0, H);       // columns [H, 2H)
        } else if (name.rfind("eagle.token_id_remap", 0) == 0) {
            copy(token_id_remap_, static_cast<size_t>(draft_vocab_) * 4);
            remap_loaded_ = true;
        } else if (name.find("eagle.input_norm1") != std::string::npos) {
            CPM_REQUIRE(ec_.use_input_norm, "norm is not used, but input_norm1 is found");
            copy(in_norm1_, static_cast<size_t>(H) * 2);
        } else if (name.find("eagle.input_norm2") != std::string::npos) {
            CPM_REQUIRE(ec_.use_input_norm, "norm is not used, but input_norm2 is found");
            copy(in_norm2_, static_cast<size_t>(H) * 2);
        } else if (name.find("eagle.rotary_emb") != std::string::npos) {
            copy(inv_freq_, static_cast<size_t>(d / 2) * 4);
        } else if (std::regex_search(name, m, layer_re)) {
            CPM_REQUIRE(std::stoi(m[1]) == 0, "drafter has a single layer");
            if (ec_.quant && load_quant_layer(elayer_, "E", m[2])) return;
            load_layer(elayer_, m[2]);
        } else {
            throw std::invalid_argument("Unsupported name (layer_idx not found): " + name);
        }
        return;
    }
    if (name.rfind("model.embed_tokens", 0) == 0) {
        copy(embed_, static_cast<size_t>(mc_.vocab) * H * 2);
    } else if (name.rfind("model.norm", 0) == 0) {
        copy(final_norm_, static_cast<size_t>(H) * 2);
    } else if (name.rfind("lm_head", 0) == 0) {
        retile(lm_head_, mc_.vocab, H, H, 0, 0, 0);
        if (has_eagle_ && draft_vocab_ != mc_.vocab) {
            // FR-Spec: the draft head is the rows of the full head picked by token_id_remap,
            // which therefore has to be loaded first (reference minicpm4_eagle.cuh:215-218)
            CPM_REQUIRE(remap_loaded_, "eagle.token_id_remap must be loaded before lm_head");
            gather_retiled_rows(lm_head_, token_id_remap_, draft_vocab_, draft_lm_head_, H, rt.stream);
            CUDA_CHECK(cudaStreamSynchronize(rt.stream));
        }
    } else if (name.find("rotary_emb") != std::string::npos) {
        copy(inv_freq_, static_cast<size_t>(d / 2) * 4);
    } else if (name.rfind("model.layers", 0) == 0 && std::regex_search(name, m, layer_re)) {
        const int li = std::stoi(m[1]);
        CPM_REQUIRE(li >= 0 && li < mc_.layers, "layer index out of range: " + name);
        if (mc_.w4a16 && load_quant_layer(layers_[li], "L" + std::to_string(li), m[2])) return;
        load_layer(layers_[li], m[2]);
    } else {
        throw std::invalid_argument("Unsupported name " + name);
    }
}

void Engine::load_quantized(const std::string& key, bool is_scales, const void* src, int K, int N, uint8_t* wq) {
    Runtime& rt = runtime();
    PendingQuant& p = pending_quant_[key];
    const size_t bytes = is_scales ? static_cast<size_t>(K / mc_.group_size) * N * 2 : static_cast<size_t>(K) * N / 2;
    void*& slot = is_scales ? p.scales : p.qweight;
    CPM_REQUIRE(slot == nullptr, "quantized tensor loaded twice: " + key);
    CUDA_CHECK(cudaMalloc(&slot, bytes));
    CUDA_CHECK(cudaMemcpyAsync(slot, src, bytes, cudaMemcpyDefault, rt.stream));
    CUDA_CHECK(cudaStreamSynchronize(rt.stream));
    if (p.qweight != nullptr && p.scales != nullptr) {
        // Marlin tile order -> row-major k-contiguous nibbles + group-major scales for the streaming kernel
        marlin_retile_for_w4(p.qweight, p.scales, K, N, wq, rt.stream);
        CUDA_CHECK(cudaStreamSynchronize(rt.stream));
        cudaFree(p.qweight);
        cudaFree(p.scales);
        pending_quant_.erase(key);
    }
}

// ------------------------------------------------------------------ plans
void Engine::build_layer_plans(LayerPlans& lp, const LayerWeights& w, const KVLayer& kv, int rows, int attn_splits) {
    const int H = mc_.hidden, I = mc_.inter, d = mc_.head_dim;
    const int sms = runtime().num_sms;
    if (w.qkv_q != nullptr) {  // W4A16 layer
        lp.qkv = checked(make_linear_plan_w4(normed_, rows, w.qkv_q, rows, qkv_dim_, H, qkv_, qkv_dim_, gemm_ws_, tickets_, sms));
        lp.o = checked(make_linear_plan_w4(attn_out_, rows, w.o_q, rows, H, mc_.hq * d, delta_, H, gemm_ws_, tickets_, sms));
        lp.gate_up = checked(make_linear_plan_w4(normed_, rows, w.gate_up_q, rows, 2 * I, H, gate_up_, 2 * I, gemm_ws_, tickets_, sms));
        lp.down = checked(make_linear_plan_w4(act_, rows, w.down_q, rows, H, I, delta_, H, gemm_ws_, tickets_, sms));
    } else {
        lp.qkv = checked(make_linear_plan(normed_, rows, w.qkv, rows, qkv_dim_, H, qkv_, qkv_dim_, nullptr, gemm_ws_, tickets_, sms));
        lp.o = checked(make_linear_plan(attn_out_, rows, w.o, rows, H, mc_.hq * d, delta_, H, nullptr, gemm_ws_, tickets_, sms));
        // the activation is applied in the gate/up GEMM's epilogue and the two projections are never stored, whenever
        // the whole-tile schedule that needs fills the GPU
        static const bool unfused = tuning_env("CPMCU_NO_SWIGLU_FUSE") != nullptr;   // bench only
        lp.gate_up = (!unfused && gate_up_interleaved() && linear_swiglu_fits(rows, I, sms))
                         ? make_linear_swiglu_plan(normed_, rows, w.gate_up, rows, I, H, act_, I, sms)
                         : checked(make_linear_plan(normed_, rows, w.gate_up, rows, 2 * I, H, gate_up_, 2 * I, nullptr, gemm_ws_, tickets_, sms));
        lp.down = checked(make_linear_plan(act_, rows, w.down, rows, H, I, delta_, H, nullptr, gemm_ws_, tickets_, sms));
    }
    lp.attn = make_attn_plan(qkv_, qkv_dim_, kv.k, kv.v, budget_, rows, mc_.hq, mc_.hkv, d, attn_splits, attn_out_,
                             mc_.hq * d, attn_ws_o_, attn_ws_ml_);
}

void Engine::build_draft_plans(LayerPlans& lp, int rows, int attn_splits) {
    build_layer_plans(lp, elayer_, ekv_, rows, attn_splits);
    if (!ec_.use_attn_norm) {
        const int H = mc_.hidden, sms = runtime().num_sms;
        lp.qkv = elayer_.qkv_q != nullptr
                     ? checked(make_linear_plan_w4(e_x_, rows, elayer_.qkv_q, rows, qkv_dim_, H, qkv_, qkv_dim_, gemm_ws_, tickets_, sms))
                     : checked(make_linear_plan(e_x_, rows, elayer_.qkv, rows, qkv_dim_, H, qkv_, qkv_dim_, nullptr, gemm_ws_, tickets_, sms));
    }
}

ForwardPlans& Engine::target_plans(int rows) {
    auto it = plans_.find(rows);
    if (it != plans_.end()) return *it->second;
    auto fp = std::make_unique<ForwardPlans>();
    fp->rows = rows;
    fp->layers.resize(mc_.layers);
    const int splits = (rows <= 64) ? attn_splits_for(rows) : 1;
    for (int l = 0; l < mc_.layers; ++l) build_layer_plans(fp->layers[l], layers_[l], kv_[l], rows, splits);
    ForwardPlans& ref = *fp;
    plans_[rows] = std::move(fp);
    return ref;
}

// ------------------------------------------------------------------ forward pieces
void Engine::layer_forward(LayerPlans& lp, const LayerWeights& w, const KVLayer& kv, const RowCtx& c, bf16* x,
                           const bf16* pending, float pending_scale, bool first_norm, float res_scale,
                           cudaStream_t s, int sparse_layer) {
    const int H = mc_.hidden, rows = c.rows;
    if (first_norm) {
        if (pending) launch_add_rms_norm(x, pending, pending_scale, w.ln_attn, normed_, rows, H, mc_.eps, s);
        else launch_rms_norm(x, H, w.ln_attn, normed_, H, rows, H, mc_.eps, s);
    } else {
        if (pending) launch_add_scaled(x, x, pending, pending_scale, rows, H, s);
        // (only the draft layer runs without a first norm; its q/k/v plan reads x directly: build_draft_plans)
    }
    launch_linear(lp.qkv, s);
    launch_rope_append(qkv_, rows, mc_.hq, mc_.hkv, mc_.head_dim, inv_freq_, c.pos, c.pos_base, c.pos_off, c.pos_step,
                       kv.k, kv.v, c.kv_len, c.kv_append_off, c.n_valid, budget_, s);
    lp.attn.kv_len = c.kv_len;
    lp.attn.kv_len_add = c.attn_kv_add;
    lp.attn.n_valid = c.n_valid;
    lp.attn.mask = c.mask;
    lp.attn.mask_k = c.mask_k;
    lp.attn.window = c.window;
    lp.attn.blockmask = nullptr;
    if (sparse_layer >= 0) {
        // InfLLM-v2: score the compressed keys of the accepted rows, pick blocks per (kv head, token)
        launch_sparse_select(sp_, mc_.sparse, sparse_layer, qkv_, qkv_dim_, rows, mc_.hq, mc_.hkv, c.kv_len,
                             c.kv_append_off, c.n_valid, s);
        if (bm_capture_ != nullptr) {
            const size_t per_layer = static_cast<size_t>(mc_.hkv) * max_rows_ * sp_.bm_words;
            CUDA_CHECK(cudaMemcpyAsync(bm_capture_ + per_layer * sparse_layer, sp_.blockmask,
                                       static_cast<size_t>(mc_.hkv) * rows * sp_.bm_words * sizeof(uint64_t),
                                       cudaMemcpyDeviceToDevice, s));
        }
        lp.attn.blockmask = sp_.blockmask;
        lp.attn.bm_words = sp_.bm_words;
        lp.attn.block_window = mc_.sparse.window_blocks;
    }
    launch_tree_attention(lp.attn, s);
    launch_linear(lp.o, s);
    launch_add_rms_norm(x, delta_, res_scale, w.ln_ffn, normed_, rows, H, mc_.eps, s);
    launch_linear(lp.gate_up, s);
    if (!lp.gate_up.swiglu) launch_silu_gate(gate_up_, act_, rows, mc_.inter, s, w.gate_up != nullptr && gate_up_interleaved());
    launch_linear(lp.down, s);
}

// Bring every layer's compressed key caches up to the accepted rows (all rows below
// *kv_len + kv_append_off are final: written by earlier passes, compacted by the last fix-up).
void Engine::sparse_prepare(const RowCtx& c, cudaStream_t s) {
    if (!mc_.sparse.enabled) return;
    launch_sparse_compress(sp_, d_cache_ptrs_, mc_.layers, mc_.hkv * mc_.head_dim, c.kv_len, c.kv_append_off,
                           max_rows_ / 16 + 2, s);
}

void Engine::lm_head_rows(const bf16* x, int x_rows, int rows, bf16* logits_out, int ld, cudaStream_t s) {
    const bf16* in = x;
    if (mc_.scale_lmhead != 1.0f) {
        CPM_REQUIRE(rows <= 64, "lm head: at most 64 rows");
        launch_scale(lm_in_, x, mc_.scale_lmhead, static_cast<size_t>(rows) * mc_.hidden, s);
        in = lm_in_;
        x_rows = rows;
    }
    LinearPlan p = checked(make_linear_plan(in, x_rows, lm_head_, rows, mc_.vocab, mc_.hidden, logits_out, ld, nullptr,
                                    gemm_ws_, tickets_, runtime().num_sms));
    launch_linear(p, s);
}

void Engine::target_forward(ForwardPlans& fp, const RowCtx& c, const int32_t* ids, bool all_logits,
                            bf16* logits_out, int logits_ld, cudaStream_t s) {
    const int H = mc_.hidden, rows = c.rows;
    launch_embedding(ids, embed_, x_, H, rows, H, mc_.scale_embed, s);
    sparse_prepare(c, s);
    const bf16* pending = nullptr;
    for (int l = 0; l < mc_.layers; ++l) {
        // chunk-sized plans are built per call, each layer's while the GPU works on the layers before it
        if (fp.lazy) build_layer_plans(fp.layers[l], layers_[l], kv_[l], rows, 1);
        layer_forward(fp.layers[l], layers_[l], kv_[l], c, x_, pending, mc_.scale_residual, true, mc_.scale_residual, s,
                      mc_.sparse.enabled ? l : -1);
        pending = delta_;
    }
    launch_add_rms_norm(x_, pending, mc_.scale_residual, final_norm_, norm_out_, rows, H, mc_.eps, s);
    if (all_logits) lm_head_rows(norm_out_, rows, rows, logits_out, logits_ld, s);
    else lm_head_rows(norm_out_ + static_cast<size_t>(rows - 1) * H, 1, 1, logits_out, logits_ld, s);
}

// ------------------------------------------------------------------ prefill / decode (reference API)
void Engine::prefill(int n, int history, const int32_t* ids, const int32_t* pos, bf16* logits_out) {
    CPM_REQUIRE(storage_ready_, "prefill before init_storage");
    CPM_REQUIRE(n >= 1 && n <= max_rows_, "prefill chunk larger than chunk_length");
    CPM_REQUIRE(history >= 0 && history + n <= budget_, "prefill exceeds the KV budget");
    Runtime& rt = runtime();
    cudaStream_t s = rt.stream;
    const int H = mc_.hidden;
    if (has_eagle_ && history > 0) {
        // deferred draft prefill of the previous chunk; its last "next token" is this chunk's first token
        launch_embedding(ids, embed_, prev_embed_ + static_cast<size_t>(num_prev_ - 1) * H, H, 1, H, mc_.scale_embed, s);
        draft_first(num_history_, s);
    }
    CUDA_CHECK(cudaMemcpyAsync(st_ + 6, &history, sizeof(int), cudaMemcpyHostToDevice, s));
    RowCtx c;
    c.rows = n;
    c.pos = pos;
    c.kv_len = st_ + 6;
    c.kv_append_off = 0;
    c.attn_kv_add = n;
    ForwardPlans fp;
    fp.rows = n;
    fp.lazy = true;
    fp.layers.resize(mc_.layers);
    static const bool prof_prefill = tuning_env("CPMCU_PROFILE_PREFILL") != nullptr;   // bench only
    if (prof_prefill) {
        for (int k = 0; k < KC_COUNT; ++k) rt.prof[k].clear();
        rt.profile = true;
    }
    target_forward(fp, c, ids, false, logits_out, mc_.vocab, s);
    if (prof_prefill) {
        // CUDA events around every launch of the pass: time per kernel class, and the GEMMs of the last layer
        rt.profile = false;
        CUDA_CHECK(cudaStreamSynchronize(s));
        const char* names[KC_COUNT] = {"linear", "attention", "other"};
        for (int k = 0; k < KC_COUNT; ++k) {
            double sum = 0.0;
            std::vector<float> each;
            for (auto& pr : rt.prof[k]) {
                float x = 0.f;
                cudaEventElapsedTime(&x, pr.first, pr.second);
                sum += x;
                each.push_back(x);
                cudaEventDestroy(pr.first);
                cudaEventDestroy(pr.second);
            }
            fprintf(stderr, "prefill profile: %s %.2f ms over %zu launches", names[k], sum, each.size());
            if (k == KC_LINEAR && each.size() >= 9) {
                const size_t b = each.size() - 5;
                fprintf(stderr, " (last layer qkv %.0f o %.0f gate_up %.0f down %.0f us)", each[b] * 1e3, each[b + 1] * 1e3,
                        each[b + 2] * 1e3, each[b + 3] * 1e3);
            }
            fprintf(stderr, "\n");
            rt.prof[k].clear();
        }
    }
    if (has_eagle_) {
        if (n > 1) launch_embedding(ids + 1, embed_, prev_embed_, H, n - 1, H, mc_.scale_embed, s);
        copy_rows(prev_hidden_, H, norm_out_, H, n, H, s);
        CUDA_CHECK(cudaMemcpyAsync(eagle_pos_, pos, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToDevice, s));
        num_prev_ = n;
        num_history_ = history;
        first_draft_ = true;
    }
    host_len_ = static_cast<long>(history) + n;
    CUDA_CHECK(cudaStreamSynchronize(s));
    check_errors("prefill");
}

void Engine::decode(int n, int padded_len, const int32_t* ids, const int32_t* pos, const int32_t* cache_length,
                    const uint64_t* mask, bf16* logits_out, bool cuda_graph) {
    (void)cuda_graph;
    CPM_REQUIRE(storage_ready_, "decode before init_storage");
    CPM_REQUIRE(n >= 1 && n <= 64, "decode supports 1..64 tokens");
    // padded_len is the caller's ceil((cache length + n) / 128) * 128 and the budget is a multiple of 128
    CPM_REQUIRE(padded_len <= 0 || padded_len <= budget_, "decode: cache length + tokens exceeds the KV budget");
    require_room(n, "decode");
    cudaStream_t s = runtime().stream;
    RowCtx c;
    c.rows = n;
    c.pos = pos;
    c.kv_len = cache_length;  // the caller has already added n (reference cpmcu/llm.py:263-283)
    c.kv_append_off = -n;
    c.attn_kv_add = 0;
    c.mask = mask;
    c.mask_k = mask ? n : 0;
    target_forward(target_plans(n), c, ids, true, logits_out, mc_.vocab, s);
    CUDA_CHECK(cudaStreamSynchronize(s));
    check_errors("decode");
}

// ------------------------------------------------------------------ draft
// x = fc([n1(embed) | n2(hidden)]) + b ; h = x + s * DecoderLayer(x).  e_in_ must hold the concatenated input rows.
void Engine::draft_forward(const RowCtx& c, int rows, LayerPlans& lp, cudaStream_t s) {
    (void)rows;
    layer_forward(lp, elayer_, ekv_, c, e_x_, nullptr, 1.f, ec_.use_attn_norm, ec_.residual_scale, s);
    launch_add_scaled(e_h_, e_x_, delta_, ec_.residual_scale, c.rows, mc_.hidden, s);
}

// x = fc1(embedding half) + b + fc2(hidden half) into e_x_.  bf16 drafter: one GEMM over K = 2H with the bias in
// its epilogue.  W4A16 drafter: two int4 GEMMs and one add, each rounded as the reference rounds them
// (src/model/minicpm4/minicpm4_eagle.cuh:228-243).
void Engine::draft_fc(int rows, const LinearPlan& fc, const LinearPlan& fc2, cudaStream_t s) {
    launch_linear(fc, s);
    if (!ec_.quant) return;
    launch_linear(fc2, s);
    launch_add_bias_add(e_x_, e_x_, fc_bias_, delta_, rows, mc_.hidden, s);
}

// Draft pass over the num_prev_ rows left by prefill (reference eagle_prefill).
void Engine::draft_first(int history, cudaStream_t s) {
    const int H = mc_.hidden, P = num_prev_;
    Runtime& rt = runtime();
    if (ec_.use_input_norm) {
        launch_rms_norm(prev_embed_, H, in_norm1_, e_in_, ein_ld(), P, H, mc_.eps, s);
        launch_rms_norm(prev_hidden_, H, in_norm2_, ein_hidden(), ein_ld(), P, H, mc_.eps, s);
    } else {
        copy_rows(e_in_, ein_ld(), prev_embed_, H, P, H, s);
        copy_rows(ein_hidden(), ein_ld(), prev_hidden_, H, P, H, s);
    }
    if (ec_.quant) {
        LinearPlan f1 = checked(make_linear_plan_w4(e_in_, P, fc1_q_, P, H, H, e_x_, H, gemm_ws_, tickets_, rt.num_sms));
        LinearPlan f2 = checked(make_linear_plan_w4(ein_hidden(), P, fc2_q_, P, H, H, delta_, H, gemm_ws_, tickets_, rt.num_sms));
        draft_fc(P, f1, f2, s);
    } else {
        LinearPlan fc = checked(make_linear_plan(e_in_, P, fc_, P, H, 2 * H, e_x_, H, fc_bias_, gemm_ws_, tickets_, rt.num_sms));
        draft_fc(P, fc, fc, s);
    }
    CUDA_CHECK(cudaMemcpyAsync(st_ + 7, &history, sizeof(int), cudaMemcpyHostToDevice, s));
    LayerPlans lp;
    build_draft_plans(lp, P, 1);
    RowCtx c;
    c.rows = P;
    c.pos = eagle_pos_;
    c.kv_len = st_ + 7;
    c.kv_append_off = 0;
    c.attn_kv_add = P;
    c.window = ec_.window;
    draft_forward(c, P, lp, s);
}

// Draft pass over the tokens accepted by the previous step (reference eagle_decode);
// fixed launch shape, the valid row count lives on the device.
void Engine::draft_catchup(cudaStream_t s) {
    const int H = mc_.hidden, rc = catchup_rows_;
    if (ec_.use_input_norm) {
        launch_rms_norm(prev_embed_, H, in_norm1_, e_in_, ein_ld(), rc, H, mc_.eps, s);
        launch_rms_norm(prev_hidden_, H, in_norm2_, ein_hidden(), ein_ld(), rc, H, mc_.eps, s);
    }  // without input norms the fix-up of the previous step wrote the rows straight into the fc input
    draft_fc(rc, fc_plan_catchup_, fc2_plan_catchup_, s);
    // layer_forward takes kv_len for both append and attention; the catch-up needs
    // different bases (append at L-n, attend over L), so split it here.
    {
        LayerPlans& lp = eplan_catchup_;
        const LayerWeights& w = elayer_;
        if (ec_.use_attn_norm) launch_rms_norm(e_x_, H, w.ln_attn, normed_, H, rc, H, mc_.eps, s);
        launch_linear(lp.qkv, s);
        launch_rope_append(qkv_, rc, mc_.hq, mc_.hkv, mc_.head_dim, inv_freq_, eagle_pos_, nullptr, 0, 0, ekv_.k, ekv_.v,
                           st_ + S_BASE, 0, st_ + S_NPREV, budget_, s);
        lp.attn.kv_len = st_ + S_L;
        lp.attn.kv_len_add = 0;
        lp.attn.n_valid = st_ + S_NPREV;
        lp.attn.mask = nullptr;
        lp.attn.mask_k = 0;
        lp.attn.window = ec_.window;
        launch_tree_attention(lp.attn, s);
        launch_linear(lp.o, s);
        launch_add_rms_norm(e_x_, delta_, ec_.residual_scale, w.ln_ffn, normed_, rc, H, mc_.eps, s);
        launch_linear(lp.gate_up, s);
        if (!lp.gate_up.swiglu) launch_silu_gate(gate_up_, act_, rc, mc_.inter, s, w.gate_up != nullptr && gate_up_interleaved());
        launch_linear(lp.down, s);
        launch_add_scaled(e_h_, e_x_, delta_, ec_.residual_scale, rc, H, s);
    }
}

void Engine::draft_levels(int32_t* tree_ids, int32_t* tree_pos, const int32_t* cache_length, uint64_t* tree_mask,
                          int32_t* tree_parent, bool first, cudaStream_t s) {
    const int H = mc_.hidden, k = ec_.topk;
    Runtime& rt = runtime();
    const bool scale_in = (!ec_.minicpm4_variant && mc_.scale_lmhead != 1.0f);
    bf16* hid_dst = ec_.use_input_norm ? e_hid_ : ein_hidden();
    const int hid_ld = ec_.use_input_norm ? H : ein_ld();
    // level 0: logits of the last pending row.  The frontier's hidden rows are gathered by the next level's
    // embedding kernel from `h_src` (the expansion kernel only records which row each node continues from).
    const bf16* h_src = e_h_;
    if (first) {
        const bf16* last = e_h_ + static_cast<size_t>(num_prev_ - 1) * H;
        h_src = last;
        const bf16* in = last;
        if (scale_in) {
            launch_scale(lm_in_, last, mc_.scale_lmhead, H, s);
            in = lm_in_;
        }
        LinearPlan p = checked(make_linear_plan(in, 1, draft_lm_head_, 1, draft_vocab_, H, e_logits_, draft_vocab_, nullptr,
                                        gemm_ws_, tickets_, rt.num_sms));
        launch_linear(p, s);
        launch_draft_topk_expand(tree_, e_logits_, draft_vocab_, draft_vocab_, 0, scan_ws_, last, H, nullptr, nullptr,
                                 hid_ld, H, s);
    } else {
        if (scale_in) launch_scale(lm_in_, e_h_, mc_.scale_lmhead, static_cast<size_t>(catchup_rows_) * H, s);
        launch_linear(dlm_plan_catchup_, s);
        launch_draft_topk_expand(tree_, e_logits_, draft_vocab_, draft_vocab_, 0, scan_ws_, e_h_, H, st_ + S_LASTROW,
                                 nullptr, hid_ld, H, s);
    }
    for (int d = 1; d < ec_.num_iter; ++d) {
        if (ec_.use_input_norm) {
            launch_embedding_gather(tree_.fr_id, embed_, e_emb_, H, k, H, mc_.scale_embed, h_src, H, tree_.fr_src, hid_dst,
                                    hid_ld, s);
            launch_rms_norm(e_emb_, H, in_norm1_, e_in_, ein_ld(), k, H, mc_.eps, s);
            launch_rms_norm(e_hid_, H, in_norm2_, ein_hidden(), ein_ld(), k, H, mc_.eps, s);
        } else {
            launch_embedding_gather(tree_.fr_id, embed_, e_in_, ein_ld(), k, H, mc_.scale_embed, h_src, H, tree_.fr_src, hid_dst,
                                    hid_ld, s);
        }
        h_src = e_h_;
        draft_fc(k, fc_plan_level_, fc2_plan_level_, s);
        RowCtx c;
        c.rows = k;
        c.pos_base = cache_length;
        c.pos_off = d - 1;
        c.pos_step = 0;
        c.kv_len = cache_length;
        c.kv_append_off = k * (d - 1);
        c.attn_kv_add = k * d;
        c.mask = tree_.fr_mask;
        c.mask_k = k * d;
        c.window = ec_.window;
        draft_forward(c, k, eplan_level_, s);
        if (scale_in) launch_scale(lm_in_, e_h_, mc_.scale_lmhead, static_cast<size_t>(k) * H, s);
        launch_linear(dlm_plan_level_, s);
        launch_draft_topk_expand(tree_, e_logits_, draft_vocab_, draft_vocab_, d, scan_ws_, e_h_, H, nullptr, nullptr,
                                 hid_ld, H, s);
    }
    launch_tree_finalize(tree_, cache_length, tree_ids, tree_pos, tree_mask, tree_parent, s);
}

void Engine::draft(int32_t* tree_ids, int32_t* tree_pos, const int32_t* cache_length, uint64_t* tree_mask,
                   int32_t* tree_parent) {
    CPM_REQUIRE(has_eagle_ && storage_ready_, "draft needs an initialised drafter");
    require_room(static_cast<long>(ec_.topk) * (ec_.num_iter - 1), "draft");
    cudaStream_t s = runtime().stream;
    const int H = mc_.hidden;
    if (first_draft_) {
        // the root token's embedding is the last "next token" input of the prompt rows
        launch_embedding(tree_ids, embed_, prev_embed_ + static_cast<size_t>(num_prev_ - 1) * H, H, 1, H,
                         mc_.scale_embed, s);
        draft_first(num_history_, s);
    } else {
        launch_kernel(state_sync_kernel, dim3(1), dim3(1), 0, s, st_, cache_length, tree_ids, 0);
        draft_catchup(s);
    }
    draft_levels(tree_ids, tree_pos, cache_length, tree_mask, tree_parent, first_draft_, s);
    first_draft_ = false;
    CUDA_CHECK(cudaStreamSynchronize(s));
    check_errors("draft");
}

// ------------------------------------------------------------------ accept
void Engine::accept_and_fix(int T, int32_t* pred, const int32_t* gt, const int32_t* pos, const int32_t* cache_length,
                            const uint64_t* mask, const int32_t* parent, cudaStream_t s) {
    AcceptIO io;
    io.tree_size = T;
    io.pred = pred;
    io.gt = gt;
    io.position_ids = pos;
    io.cache_length = cache_length;
    io.attn_mask = mask;
    io.tree_parent = parent;
    io.result = accept_result_;
    FixupArgs f;
    f.caches = d_cache_ptrs_;
    f.num_caches = 2 * mc_.layers;
    f.kv_dim = mc_.hkv * mc_.head_dim;
    f.max_accept = has_eagle_ ? catchup_rows_ : 1;
    f.norm_out = norm_out_;
    // without input norms the next catch-up pass takes these rows as its fc input as they are: write them there
    const bool direct = has_eagle_ && !ec_.use_input_norm;
    f.prev_ld = direct ? ein_ld() : mc_.hidden;
    f.prev_hidden = direct ? ein_hidden() : prev_hidden_;
    f.embed_table = embed_;
    f.embed_scale = mc_.scale_embed;
    f.prev_embed = direct ? e_in_ : prev_embed_;
    f.eagle_pos = eagle_pos_;
    f.hidden = mc_.hidden;
    launch_accept_fixup(io, f, budget_, s);
    launch_kernel(publish_kernel, dim3(1), dim3(32), 0, s, accept_result_, pred, runtime().d_error, st_, d_publish_);
}

int Engine::verify_and_fix(int T, int32_t* pred, const int32_t* gt, const int32_t* pos, const int32_t* cache_length,
                           const uint64_t* mask, const int32_t* parent) {
    CPM_REQUIRE(has_eagle_ && storage_ready_, "verify needs an initialised drafter");
    CPM_REQUIRE(T == ec_.tree_size, "verify: tree size differs from the drafter's");
    cudaStream_t s = runtime().stream;
    accept_and_fix(T, pred, gt, pos, cache_length, mask, parent, s);
    CUDA_CHECK(cudaMemcpyAsync(h_result_, d_publish_, 32 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CUDA_CHECK(cudaStreamSynchronize(s));
    if (h_result_[31] != 0) check_errors("verify_and_fix");
    num_prev_ = h_result_[0];
    if (host_len_ >= 0) host_len_ += h_result_[0];
    return h_result_[0];
}

void Engine::check_errors(const char* where) {
    const int e = read_and_clear_error();
    if (e != 0) {
        if (e & ERR_GEMM_TIMEOUT) {
            // a split-K tile that gave up leaves its piece counters non-zero; later GEMMs would miscount
            cudaMemsetAsync(tickets_, 0, sizeof(int) * kTicketInts, runtime().stream);
            cudaMemsetAsync(runtime().d_accept_ticket, 0, sizeof(unsigned), runtime().stream);
            cudaStreamSynchronize(runtime().stream);
        }
        throw std::runtime_error(std::string("cpmcu_b200: kernel error flags ") + std::to_string(e) + " raised in " +
                                 where + " (1 = GEMM pipeline timeout, 2 = attention pipeline timeout, 4 = malformed draft tree, "
                                 "8 = K/V row beyond the cache budget)");
    }
}

// A pass that appends `rows_after_len` K/V rows behind the host-known length must fit the budget.
void Engine::require_room(long rows_after_len, const char* where) const {
    if (host_len_ >= 0 && host_len_ + rows_after_len > budget_) {
        throw std::runtime_error(std::string("cpmcu_b200: ") + where + " would write K/V row " +
                                 std::to_string(host_len_ + rows_after_len - 1) + " but the cache holds " +
                                 std::to_string(budget_) + " rows (raise memory_limit or shorten the generation)");
    }
}

// ------------------------------------------------------------------ fused step
void Engine::set_sampling(float temperature, unsigned long long seed) {
    CPM_REQUIRE(temperature >= 0.f, "temperature must not be negative");
    if ((temperature > 0.f) != (temperature_ > 0.f) || temperature != temperature_ || seed != sample_seed_) {
        // temperature and seed are baked into the captured step
        if (step_graph_) {
            cudaGraphExecDestroy(step_graph_);
            step_graph_ = nullptr;
        }
    }
    temperature_ = temperature;
    sample_seed_ = seed;
}

void Engine::begin_generation(int prefix_length, int32_t root_token) {
    CPM_REQUIRE(has_eagle_ && storage_ready_, "begin_generation needs an initialised drafter");
    CPM_REQUIRE(first_draft_, "begin_generation must follow prefill");
    cudaStream_t s = runtime().stream;
    int32_t init[S_COUNT] = {0};
    init[S_L] = prefix_length;
    CPM_REQUIRE(prefix_length >= 1 && prefix_length <= budget_, "begin_generation: prefix length out of range");
    host_len_ = prefix_length;
    CUDA_CHECK(cudaMemcpyAsync(st_, init, S_COUNT * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    CUDA_CHECK(cudaMemcpyAsync(t_ids_, &root_token, sizeof(int32_t), cudaMemcpyHostToDevice, s));
    CUDA_CHECK(cudaStreamSynchronize(s));
}

// One speculative step on engine-owned buffers: state advance, draft, tree,
// target verify forward, argmax, acceptance, fix-up, publish.
void Engine::enqueue_step(bool first, cudaStream_t s) {
    const int T = ec_.tree_size, H = mc_.hidden;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    CUDA_CHECK(cudaStreamIsCapturing(s, &cap));
    const bool capturing = (cap == cudaStreamCaptureStatusActive);
    launch_kernel(state_sync_kernel, dim3(1), dim3(1), 0, s, st_, static_cast<const int32_t*>(nullptr), t_ids_, 1);
    if (first) {
        launch_embedding(t_ids_, embed_, prev_embed_ + static_cast<size_t>(num_prev_ - 1) * H, H, 1, H, mc_.scale_embed, s);
        draft_first(num_history_, s);
    } else {
        draft_catchup(s);
    }
    draft_levels(t_ids_, t_pos_, st_ + S_L, t_mask_, t_parent_, first, s);
    // boundary between the draft half and the verify half of the step (an event node when captured)
    CUDA_CHECK(cudaEventRecordWithFlags(ev_mid_, s, capturing ? cudaEventRecordExternal : cudaEventRecordDefault));
    RowCtx c;
    c.rows = T;
    c.pos = t_pos_;
    c.kv_len = st_ + S_L;
    c.kv_append_off = 0;
    c.attn_kv_add = T;
    c.mask = t_mask_;
    c.mask_k = T;
    ForwardPlans& fp = target_plans(T);
    const int V = mc_.vocab;
    // target forward; the LM-head plan is cached because its output buffer is engine-owned
    launch_embedding(t_ids_, embed_, x_, H, T, H, mc_.scale_embed, s);
    sparse_prepare(c, s);
    const bf16* pending = nullptr;
    for (int l = 0; l < mc_.layers; ++l) {
        layer_forward(fp.layers[l], layers_[l], kv_[l], c, x_, pending, mc_.scale_residual, true, mc_.scale_residual, s,
                      mc_.sparse.enabled ? l : -1);
        pending = delta_;
    }
    launch_add_rms_norm(x_, pending, mc_.scale_residual, final_norm_, norm_out_, T, H, mc_.eps, s);
    if (mc_.scale_lmhead != 1.0f) launch_scale(lm_in_, norm_out_, mc_.scale_lmhead, static_cast<size_t>(T) * H, s);
    if (lm_plan_tree_.grid == 0) {
        lm_plan_tree_ = checked(make_linear_plan(mc_.scale_lmhead != 1.0f ? lm_in_ : norm_out_, T, lm_head_, T, V, H, logits_, V,
                                         nullptr, gemm_ws_, tickets_, runtime().num_sms));
    }
    launch_linear(lm_plan_tree_, s);
    launch_sample(logits_, T, V, V, t_gt_, argmax_ws_, temperature_, sample_seed_, st_ + S_DRAW, 0, s);
    accept_and_fix(T, t_ids_, t_gt_, t_pos_, st_ + S_L, t_mask_, t_parent_, s);
    CUDA_CHECK(cudaMemcpyAsync(h_result_, d_publish_, 32 * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
}

int Engine::spec_step(int32_t* out_tokens, int max_tokens) {
    CPM_REQUIRE(has_eagle_ && storage_ready_, "spec_step needs an initialised drafter");
    require_room(std::max<long>(ec_.tree_size, static_cast<long>(ec_.topk) * (ec_.num_iter - 1)), "spec_step");
    Runtime& rt = runtime();
    cudaStream_t s = rt.stream;
    if (first_draft_) {
        CUDA_CHECK(cudaEventRecord(ev0_, s));
        enqueue_step(true, s);
        CUDA_CHECK(cudaEventRecord(ev1_, s));
        first_draft_ = false;
    } else {
        if (step_graph_ == nullptr) {
            const long before = rt.launches;
            cudaGraph_t graph = nullptr;
            CUDA_CHECK(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
            try {
                enqueue_step(false, s);
            } catch (...) {
                cudaStreamEndCapture(s, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            CUDA_CHECK(cudaStreamEndCapture(s, &graph));
            CUDA_CHECK(cudaGraphInstantiate(&step_graph_, graph, 0));
            CUDA_CHECK(cudaGraphDestroy(graph));
            launches_per_step_ = rt.launches - before;
        }
        CUDA_CHECK(cudaEventRecord(ev0_, s));
        CUDA_CHECK(cudaGraphLaunch(step_graph_, s));
        CUDA_CHECK(cudaEventRecord(ev1_, s));
        rt.launches += launches_per_step_;
    }
    CUDA_CHECK(cudaStreamSynchronize(s));
    float ms = 0.f;
    CUDA_CHECK(cudaEventElapsedTime(&ms, ev0_, ev1_));
    last_step_ms_ = ms;
    float ms_d = 0.f, ms_v = 0.f;
    CUDA_CHECK(cudaEventElapsedTime(&ms_d, ev0_, ev_mid_));
    CUDA_CHECK(cudaEventElapsedTime(&ms_v, ev_mid_, ev1_));
    last_draft_ms_ = ms_d;
    last_verify_ms_ = ms_v;
    if (h_result_[31] != 0) check_errors("spec_step");
    const int n = h_result_[0];
    num_prev_ = n;
    if (host_len_ >= 0) host_len_ += n;
    for (int i = 0; i < n && i < max_tokens; ++i) out_tokens[i] = h_result_[1 + i];
    return n;
}

const int32_t* Engine::tree_buffers(int which) const {
    switch (which) {
        case 0: return t_ids_;
        case 1: return t_pos_;
        case 2: return t_parent_;
        case 3: return t_gt_;
        case 4: return reinterpret_cast<const int32_t*>(t_mask_);
        case 5: return st_;
        default: return nullptr;
    }
}

// One eager (uncaptured) step with every linear / attention launch bracketed by
// CUDA events; returns summed device milliseconds and launch counts per class.
void Engine::profile_step(float* ms, int* counts, float* total_ms) {
    CPM_REQUIRE(has_eagle_ && storage_ready_ && !first_draft_, "profile_step needs a generation in progress");
    require_room(std::max<long>(ec_.tree_size, static_cast<long>(ec_.topk) * (ec_.num_iter - 1)), "profile_step");
    Runtime& rt = runtime();
    cudaStream_t s = rt.stream;
    for (int c = 0; c < KC_COUNT; ++c) rt.prof[c].clear();
    rt.profile = true;
    CUDA_CHECK(cudaEventRecord(ev0_, s));
    try {
        enqueue_step(false, s);
    } catch (...) {
        rt.profile = false;
        throw;
    }
    rt.profile = false;
    CUDA_CHECK(cudaEventRecord(ev1_, s));
    CUDA_CHECK(cudaStreamSynchronize(s));
    float t = 0.f;
    CUDA_CHECK(cudaEventElapsedTime(&t, ev0_, ev1_));
    *total_ms = t;
    for (int c = 0; c < KC_COUNT; ++c) {
        double sum = 0.0;
        for (auto& pr : rt.prof[c]) {
            float x = 0.f;
            cudaEventElapsedTime(&x, pr.first, pr.second);
            sum += x;
            cudaEventDestroy(pr.first);
            cudaEventDestroy(pr.second);
        }
        ms[c] = static_cast<float>(sum);
        counts[c] = static_cast<int>(rt.prof[c].size());
        rt.prof[c].clear();
    }
    if (h_result_[31] != 0) check_errors("profile_step");
    num_prev_ = h_result_[0];
    if (host_len_ >= 0) host_len_ += h_result_[0];
}
