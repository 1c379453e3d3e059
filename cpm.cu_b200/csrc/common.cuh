// Shared declarations for the speculative-decoding kernels: error handling,
// the per-process runtime (stream, device error word, TMA encoder), and the
// launch prototypes each .cu file exports to the engine and to the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

typedef __nv_bfloat16 bf16;

#define CUDA_CHECK(expr)                                                                            \
    do {                                                                                            \
        cudaError_t err__ = (expr);                                                                 \
        if (err__ != cudaSuccess) {                                                                 \
            throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(err__) + " at " + \
                                     __FILE__ + ":" + std::to_string(__LINE__) + " (" #expr ")");   \
        }                                                                                           \
    } while (0)

#define CPM_REQUIRE(cond, msg)                                                        \
    do {                                                                              \
        if (!(cond)) throw std::invalid_argument(std::string("cpmcu_b200: ") + (msg)); \
    } while (0)

// Tuning switches (grid and split sweeps, A/B of the cluster split-K, plan printing, timing experiments that skip
// loads or stores and therefore give wrong results) exist only in builds made with
// CPMCU_BUILD_DEFINES=-DCPMCU_TUNING: a normal build reads none of these variables and its kernels carry none of
// these branches.
#ifdef CPMCU_TUNING
#include <cstdlib>
inline const char* tuning_env(const char* name) { return getenv(name); }
#define CPM_EXPERIMENT(args, bits) ((args).debug & (bits))
#else
inline const char* tuning_env(const char*) { return nullptr; }
#define CPM_EXPERIMENT(args, bits) 0
#endif

// Records the message cpmcu_last_error() returns on this thread (capi.cu).
void cpm_set_error(const char* msg);

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------- runtime
// Error word bits written by kernels (device memory, read by the host).
enum KernelError : int {
    ERR_NONE = 0,
    ERR_GEMM_TIMEOUT = 1,
    ERR_ATTN_TIMEOUT = 2,
    ERR_BAD_TREE = 4,
    ERR_KV_OVERFLOW = 8,  // a K/V row beyond the cache budget was about to be written (the store is skipped)
};

enum KernelClass : int { KC_LINEAR = 0, KC_ATTENTION = 1, KC_OTHER = 2, KC_COUNT = 3 };

struct Runtime {
    cudaStream_t stream = nullptr;
    int* d_error = nullptr;  // device error word, or-ed into by kernels
    unsigned* d_accept_ticket = nullptr;  // CTAs of the acceptance kernel that have read the tree (zero between launches)
    int num_sms = 148;
    int device = 0;
    long launches = 0;  // kernels launched (or captured) so far by this library
    bool pdl = true;  // launch kernels with programmatic stream serialization (prologue overlap)
    // Optional per-launch timing (eager runs only): event pairs per kernel class.
    bool profile = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof[KC_COUNT];
};

// Brackets one launch with CUDA events on its stream while Runtime::profile is set.
struct ProfileScope {
    cudaStream_t s;
    int kind;
    bool on;
    cudaEvent_t e1 = nullptr;
    ProfileScope(int kind_, cudaStream_t s_);
    ~ProfileScope();
};
Runtime& runtime();          // lazily initialised, one per process
int read_and_clear_error();  // synchronises the stream

// Kernel launch with programmatic dependent launch enabled: the grid may start
// while its predecessor in the stream drains; every kernel here executes
// griddepcontrol.wait before touching global memory, which restores the order.
template <typename... KArgs, typename... Args>
void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = runtime().pdl ? 1 : 0;
    CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    runtime().launches++;
}

// The same for a kernel that runs as thread-block clusters of `cluster` CTAs (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
void launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, int cluster,
                           Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = runtime().pdl ? 2 : 1;
    CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    runtime().launches++;
}

// Clusters of `cluster` CTAs of this kernel that the device runs at once (0 when the query fails).  The SMs
// come in groups that need not be multiples of the cluster size, so this can be fewer than SMs / cluster.
template <typename... KArgs>
int max_active_clusters(void (*kernel)(KArgs...), dim3 block, size_t smem, int cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster * 32);
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    return n;
}

// Device side of the above.  Every kernel lets its successor start launching at once
// (the successor can only set up and read constant data until its own wait returns) and
// waits for its predecessor before it touches anything a previous kernel may have written.
__device__ __forceinline__ void grid_dep_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_sync() {
    grid_dep_trigger();
    grid_dep_wait();
}

// 2-D / 3-D bf16 tensor maps with 128-byte swizzle; inner box extent is 64
// elements (128 B).  Strides are in bytes and must be multiples of 16.
CUtensorMap make_tmap_2d(const void* base, uint64_t inner, uint64_t outer, uint64_t outer_stride_bytes,
                         uint32_t box_inner, uint32_t box_outer);
// Untyped byte matrix without swizzle (packed int4 weights).
CUtensorMap make_tmap_2d_u8(const void* base, uint64_t inner_bytes, uint64_t outer, uint64_t outer_stride_bytes,
                            uint32_t box_inner_bytes, uint32_t box_outer);
CUtensorMap make_tmap_3d(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                         uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// ---------------------------------------------------------------- GEMM
// Y[M,N] = X[M,K] * W[N,K]^T (+ bias[N]); bf16 in, fp32 accumulate in TMEM.
// silu(g) * u as the reference's kernel computes it (src/model/activation.cuh:12-16: g * (1 / (1 + expf(-g))) * u in
// fp32, built with --use_fast_math, i.e. the ex2.approx form of expf and an approximate reciprocal).
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float s = __fdividef(1.0f, 1.0f + __expf(-g));
    return g * s * u;
}

struct LinearPlan {
    CUtensorMap tm_w;   // W  [N,K], box 64 x 128
    CUtensorMap tm_x;   // X  [Mrows,K], box 64 x MT
    int M = 0, N = 0, K = 0;
    int mt = 0;         // token tile: 16, 32, 64, 128 or 256
    int grid = 0;
    bf16* y = nullptr;
    int ldy = 0;
    const bf16* bias = nullptr;
    float* workspace = nullptr;  // split-K partials: grid * 2 * mt * 128 floats
    int* tickets = nullptr;      // two counters per output tile (pieces counted, readers gone), zero between launches
    int debug = 0;               // timing experiments of -DCPMCU_TUNING builds (CPM_EXPERIMENT); unused otherwise
    int cluster = 0;             // > 0: CTAs per tile, pieces summed inside a thread-block cluster (bf16 path)
    int wave_tiles = 0;          // several token tiles: tiles computed whole, in waves of `grid` (the rest is cut along K)
    int tail_grid = 0;           // CTAs that share the tiles after wave_tiles (0 = all)
    int swiglu = 0;              // SwiGLU epilogue: w = [gate ; up], N = output features, y = silu(gate) * up
    // W4A16: when wq is set the weights are 4-bit blocks in the streaming layout (see gemm_w4_umma.cu)
    const void* wq = nullptr;
};

// Weight layout of the bf16 GEMMs ("tile-major"): W [N, K] is stored as ceil(N / 128) x (K / 64) blocks of 128 rows x
// 64 elements, each block 16 KB of consecutive memory, blocks of a 128-row tile consecutive along K.  The kernels
// fetch one block per TMA copy; from a row-major W the same copy gathers 128 segments of 128 B that lie K * 2 bytes
// apart, one DRAM page each, and the GEMMs of the step ran at 5.4-6.3 TB/s instead of 6.5-8 TB/s.  Rows beyond N are
// zero.  With `mode` 1 / 2 the source rows are the gate / up projection of a SwiGLU pair and go to rows 0-63 / 64-127 of
// the tile of their 64-feature group, so one tile holds both projections of the same features.
size_t linear_weight_elems(int N, int K);
// src: `rows` x `src_cols` row-major bf16, device OR host memory; they become rows [row_offset, row_offset + rows) (or
// the gate / up slots) and columns [k_offset, k_offset + src_cols) of the tile-major matrix `dst` with K columns.
void retile_weight_rows(const void* src, int rows, int src_cols, bf16* dst, int K, int mode, int row_offset, int k_offset,
                        cudaStream_t s);
// dst row i = src row idx[i], both tile-major with K columns (FR-Spec draft head).
void gather_retiled_rows(const bf16* src, const int32_t* idx, int rows, bf16* dst, int K, cudaStream_t s);
size_t linear_workspace_bytes(int mt, int grid);
int linear_pick_mt(int M);
LinearPlan make_linear_plan(const bf16* x, int x_rows, const bf16* w, int M, int N, int K, bf16* y, int ldy,
                            const bf16* bias, float* workspace, int* tickets, int grid_limit);
int linear_schedule_dump(int M, int N, int K, int grid_limit, int32_t* out, int cap);
bool linear_swiglu_fits(int M, int inter, int grid_limit);
LinearPlan make_linear_swiglu_plan(const bf16* x, int x_rows, const bf16* w, int M, int inter, int K, bf16* act, int ld,
                                   int grid_limit);
void launch_linear(const LinearPlan& plan, cudaStream_t stream);
// Same contract with 4-bit weights, w = (q - 8) * scale, K % 256 == 0 and N % 128 == 0.  `wq` holds one
// contiguous 16896-byte block per (128-feature tile, 256-k unit), tile-major: [4 k-blocks][2 halves]
// [128 rows][16 B] of nibbles (a 32-bit word holds k0 k2 k4 k6 k1 k3 k5 k7 from bit 0) then
// [2 groups][128 rows] bf16 scales.
LinearPlan make_linear_plan_w4(const bf16* x, int x_rows, const void* wq, int M, int N, int K, bf16* y, int ldy,
                               float* workspace, int* tickets, int grid_limit);
void launch_linear_w4(const LinearPlan& plan, cudaStream_t stream);
size_t linear_w4_workspace_bytes(int mt, int grid);
void linear_w4_print_prof();  // bench only (CPMCU_W4_PROF)
size_t linear_w4_weight_bytes(int N, int K);
// Marlin tensors (packed int32 [K/16, 2N], permuted scales [K/128, N]) -> the layout above.
void marlin_retile_for_w4(const void* packed, const void* scales, int K, int N, void* wq, cudaStream_t s);

// W4A16 GPTQ-Marlin tensor (packed int32 [K/16, 2N] + permuted bf16 scales [K/128, N]) -> bf16 [N, K].
void marlin_dequant_to_bf16(const void* packed, const void* scales, int K, int N, int group_size, bf16* dst,
                            cudaStream_t s);

// ---------------------------------------------------------------- small ops
void launch_rms_norm(const bf16* x, int ldx, const bf16* w, bf16* y, int ldy, int rows, int dim, float eps,
                     cudaStream_t s);
// x += delta * scale (in bf16, in place), then y = rmsnorm(x) * w
void launch_add_rms_norm(bf16* x, const bf16* delta, float delta_scale, const bf16* w, bf16* y, int rows, int dim,
                         float eps, cudaStream_t s);
void launch_embedding(const int32_t* ids, const bf16* table, bf16* out, int ld_out, int rows, int dim, float scale,
                      cudaStream_t s);
// The same plus, in the same launch, hid_out[r] = h_rows[src[r]] for r < rows (rows of `dim` elements).
void launch_embedding_gather(const int32_t* ids, const bf16* table, bf16* out, int ld_out, int rows, int dim, float scale,
                             const bf16* h_rows, int h_ld, const int32_t* src, bf16* hid_out, int hid_ld,
                             cudaStream_t s);
// qkv: [rows, (hq + 2 hkv) * d].  Applies NeoX RoPE to q (in place) and k, then
// writes k,v into the cache at row (*kv_len + kv_off + r) for r < *n_valid
// (n_valid may be null = rows).  Position of row r: pos[r], or when pos is
// null *pos_base + pos_off + r * pos_step.  cache_rows: rows the caches hold; a row at or beyond it is not
// stored and raises ERR_KV_OVERFLOW in the device error word.
void launch_rope_append(bf16* qkv, int rows, int hq, int hkv, int d, const float* inv_freq, const int32_t* pos,
                        const int32_t* pos_base, int pos_off, int pos_step, bf16* k_cache, bf16* v_cache,
                        const int32_t* kv_len, int kv_off, const int32_t* n_valid, int cache_rows, cudaStream_t s);
// interleaved: gate_up is [rows, 2 * inter] with gate / up of features 64 t .. 64 t + 63 in columns 128 t .. 128 t + 63 /
// 128 t + 64 .. 128 t + 127 (the output of a GEMM over SwiGLU-interleaved weight tiles) instead of [gate | up] halves
void launch_silu_gate(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t s, bool interleaved = false);
void launch_add_scaled(bf16* x, const bf16* a, const bf16* b, float scale_b, int rows, int dim,
                       cudaStream_t s);  // x = a + b*scale
void launch_scale(bf16* out, const bf16* in, float scale, size_t n, cudaStream_t s);
// x = (a + bias[col]) + b, each sum rounded to bf16 (bias may be null): the two halves of a quantised fc
void launch_add_bias_add(bf16* x, const bf16* a, const bf16* bias, const bf16* b, int rows, int dim, cudaStream_t s);
size_t argmax_workspace_bytes(int rows, int vocab);
void launch_argmax(const bf16* logits, int rows, int vocab, int ld, int32_t* out, void* workspace, cudaStream_t s);
// Row pick with a temperature: out[r] ~ softmax(logits[r] / temperature), drawn by Gumbel-max with Philox noise
// keyed by (seed, r, *draw + draw_add, column); temperature <= 0 is launch_argmax.  `draw` (device, may be null)
// lets a captured step advance its draw index without re-capturing.
void launch_sample(const bf16* logits, int rows, int vocab, int ld, int32_t* out, void* workspace, float temperature,
                   unsigned long long seed, const int32_t* draw, int draw_add, cudaStream_t s);

// ---------------------------------------------------------------- attention
struct AttnPlan {
    CUtensorMap tm_q;  // [tq, hq, d] viewed as 3-D (d, heads, tokens)
    CUtensorMap tm_k;  // [budget, hkv*d]
    CUtensorMap tm_v;
    int tq = 0, hq = 0, hkv = 0, d = 128;
    int splits = 1;
    const int32_t* kv_len = nullptr;  // device scalar
    int kv_len_add = 0;               // keys visible = *kv_len + kv_len_add
    const int32_t* n_valid = nullptr; // device scalar: valid query rows (null = tq)
    const uint64_t* mask = nullptr;   // per-token tree mask over the last mask_k keys
    int mask_k = 0;
    int window = 0;                   // >0: block-granular sliding window (tokens)
    const uint64_t* blockmask = nullptr;  // block-sparse mode: [hkv][tq][bm_words] bits over 64-key blocks
    int bm_words = 0;
    int block_window = 0;             // trailing 64-key blocks every token sees in block-sparse mode
    float scale = 0.f;
    bf16* out = nullptr;              // token t, head h at out + t*out_ld + h*d
    int out_ld = 0;
    float* ws_o = nullptr;            // [splits, tq*hq, d]
    float* ws_ml = nullptr;           // [splits, tq*hq, 2]
};
size_t attn_workspace_bytes(int tq, int hq, int d, int splits);
AttnPlan make_attn_plan(const bf16* q, int q_ld_tokens, const bf16* k_cache, const bf16* v_cache, int budget,
                        int tq, int hq, int hkv, int d, int splits, bf16* out, int out_ld, float* ws_o,
                        float* ws_ml);
void launch_tree_attention(const AttnPlan& plan, cudaStream_t s);
