// Tree-verification attention over the contiguous bf16 KV cache, sm_100a.
//
// Replaces the reference's FlashAttention fork entry `mha_fwd_kvcache`
// (src/flash_attn/flash_api.hpp:292-392: split-KV kernel + combine) for the
// verify pass (tree rows), the draft levels, the draft's catch-up pass and the
// causal prefill.  Visibility of key c for query token t follows the reference
// (src/flash_attn/src/mask.h:182-222): c < kv_total - tq + t + 1 (causal), and
// for the last `mask_k` keys additionally bit (c - (kv_total - mask_k)) of the
// token's 64-bit tree mask.
//
// Mapping.  All `grp = hq / hkv` query heads that share a KV head are packed
// with 128 / grp consecutive tokens into one 128-row tile, so a K/V tile is
// read once per KV head and tile instead of once per query head.  Per CTA:
//   S = Q K^T   tcgen05.mma, A = Q (K-major), B = K tile (K-major), S in TMEM
//   softmax     one thread per row reads S with tcgen05.ld, online max/sum,
//               writes bf16 P into 128-byte-swizzled shared memory
//   O += P V    tcgen05.mma, A = P (K-major), B = V tile (N-major), O in TMEM
// K/V tiles of 128 keys arrive by TMA (each CTA loads its own) into a two-stage ring.
//
// Block-sparse mode (InfLLM-v2 target layers; replaces compute_attn_1rowblock_splitkv_headlevel,
// src/flash_attn/src/flash_fwd_kernel.h:580-1171 with the iterator of flash_blockmask.h): every
// (kv head, token) carries a bitmask over 64-key blocks; a token sees block b iff its bit is set or
// b >= ceil((t + kv_total - tq) / 64) - block_window.  A tile holds 128 / grp tokens, so the CTA
// visits the union of their blocks (kept as a bitmask over 128-key tiles in shared memory) and each
// row masks the 64-key halves its own token may not see.
// gridDim.y key splits each write an unnormalised partial (O, max, sum); a
// small second kernel merges them.  With one split the kernel normalises and
// stores bf16 directly.
#include <algorithm>
#include <cstdio>
#include <vector>

#include "common.cuh"
#include "ptx.cuh"

namespace {

constexpr int D = 128;          // head dim
constexpr int ROWS = 128;       // query rows per tile (UMMA M)
constexpr int KEYS = 128;       // keys per tile
constexpr int HALF_BYTES = ROWS * 128;        // one 64-column half: 128 rows x 128 B
constexpr int TILE_BYTES = 2 * HALF_BYTES;    // 32 KB
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + TILE_BYTES;          // 2 stages
constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;      // 2 stages
constexpr int SMEM_P = SMEM_V + 2 * TILE_BYTES;      // 2 stages
constexpr int SMEM_CTRL = SMEM_P + 2 * TILE_BYTES;
constexpr int SMEM_UNION = SMEM_CTRL + 128;  // 256 B: bitmask over up to 2048 key tiles (block-sparse mode)
constexpr int SMEM_XCH = SMEM_CTRL + 512;   // 2 x 128 floats
constexpr int SMEM_TOTAL = SMEM_XCH + 1024 + 1024;
constexpr int TMEM_COLS = 512;  // S stage 0: [0,128), S stage 1: [128,256), O: [256,384)
constexpr int TMEM_O = 256;
constexpr int SOFTMAX_THREADS = 256;  // two threads per query row: warps 0-3 keys 0-63 of a tile, warps 4-7 keys 64-127
constexpr int NTHREADS = SOFTMAX_THREADS + 32;  // + one control warp (TMA and MMA issue)

struct AttnArgs {
    int tq, hq, hkv, grp, tok_per_tile, num_mtiles;
    int heavy_first;  // causal prefill: token tiles are handed out last-to-first, longest key range first
    const int32_t* kv_len;
    int kv_len_add;
    const int32_t* n_valid;
    const uint64_t* mask;
    int mask_k;
    int window;
    const uint64_t* blockmask;  // [hkv][tq][bm_words] bits over 64-key blocks, or null
    int bm_words, block_window;
    float scale_log2;
    bf16* out;
    int out_ld;
    float* ws_o;
    float* ws_ml;
    int* error;
    long long* prof;  // bench only (-DCPMCU_ATTN_PROFILE): clock counters of CTA 0, or null
};

#ifdef CPMCU_ATTN_PROFILE
constexpr bool kAttnProf = true;
#else
constexpr bool kAttnProf = false;
#endif
__device__ __forceinline__ long long prof_clock() { return kAttnProf ? clock64() : 0; }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Software pipeline over 128-key tiles.  The control warp keeps the tensor pipe one tile
// ahead: S(i+1) = Q K(i+1)^T is already in TMEM (two S stages) while the softmax warps work
// on tile i, and O += P(i) V(i) is issued as soon as P(i) is in shared memory (two P stages),
// so in steady state an iteration costs one softmax pass.
__global__ void __launch_bounds__(NTHREADS, 1)
tree_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_CTRL);
    uint64_t* q_bar = bars;
    uint64_t* k_full = bars + 1;   // [2]
    uint64_t* v_full = bars + 3;   // [2]
    uint64_t* s_bar = bars + 5;    // [2]  S(i) is in TMEM
    uint64_t* o_bar = bars + 7;    // [2]  PV(i) has finished (P stage, V stage and O are free / stable)
    uint64_t* p_ready = bars + 9;  // [2]  P(i) is in shared memory (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(smem + SMEM_XCH);  // [2][128] row maxima / sums of the two column halves

    const long long pt_kernel = prof_clock();
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool is_control = (warp == SOFTMAX_THREADS / 32);
    const int ch = (warp >> 2) & 1;              // column half of the key tile
    const int row = (warp & 3) * 32 + lane;      // query row of the tile == TMEM lane
    grid_dep_trigger();
    const int mt_in = blockIdx.x % a.num_mtiles;
    const int mt = a.heavy_first ? a.num_mtiles - 1 - mt_in : mt_in;
    const int h = blockIdx.x / a.num_mtiles;  // kv head
    const int split = blockIdx.y;
    const int nsplit = gridDim.y;

    if (tid == 0) {
        ptx::mbar_init(q_bar, 1);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&k_full[i], 1);
            ptx::mbar_init(&v_full[i], 1);
            ptx::mbar_init(&s_bar[i], 1);
            ptx::mbar_init(&o_bar[i], 1);
            ptx::mbar_init(&p_ready[i], SOFTMAX_THREADS / 32);  // one arrival per softmax warp
        }
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
    }
    if (warp == 0) {
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_o = tmem_base + lane_sel + TMEM_O + ch * 64;  // this thread's 64 output columns
    grid_dep_wait();  // everything above overlaps the previous kernel's tail
    const long long pt_dep = prof_clock();

    // ---- geometry of this tile
    const int kv_total = *a.kv_len + a.kv_len_add;
    const int tq_eff = (a.n_valid != nullptr) ? min(*a.n_valid, a.tq) : a.tq;
    const int t0 = mt * a.tok_per_tile;
    const int t = t0 + row / a.grp;          // query token of this thread's row
    const int qh = h * a.grp + row % a.grp;  // query head of this thread's row
    const bool row_valid = (t < tq_eff);
    const int causal_base = kv_total - tq_eff;  // token t sees keys < causal_base + t + 1
    int limit = row_valid ? min(kv_total, causal_base + t + 1) : 0;
    if (limit < 0) limit = 0;
    const int mbeg = (a.mask != nullptr) ? (kv_total - a.mask_k) : 0x7fffffff;
    const uint64_t mword = (a.mask != nullptr && row_valid) ? a.mask[t] : ~0ull;
    // keys any row of this tile may see: [key_lo, key_hi)
    const int t_last = min(t0 + a.tok_per_tile, tq_eff) - 1;
    int key_hi = (t_last >= t0) ? min(kv_total, causal_base + t_last + 1) : 0;
    if (key_hi < 0) key_hi = 0;
    int key_lo = 0;
    if (a.window > 0) {
        // block-granular sliding window of the draft layer: the reference derives the bound per
        // 64-row query block (src/flash_attn/src/flash_fwd_kernel.h:1517 passes m_block * 64 to
        // src/flash_attn/src/flash_blockmask.h:29-33, 128-key blocks)
        const int q0 = causal_base + (t0 / 64) * 64;
        const int lo_blk = (q0 + KEYS - 1) / KEYS - a.window / KEYS;
        if (lo_blk > 0) key_lo = lo_blk * KEYS;
    }
    const int kt_lo = key_lo / KEYS;
    const int kt_hi = (key_hi + KEYS - 1) / KEYS;
    const int n_kt = max(kt_hi - kt_lo, 0);
    int kt_begin = kt_lo + static_cast<int>((static_cast<long long>(n_kt) * split) / nsplit);
    const int kt_end = kt_lo + static_cast<int>((static_cast<long long>(n_kt) * (split + 1)) / nsplit);
    int n_it = kt_end - kt_begin;

    // ---- block-sparse mode: union of the tile's tokens' blocks, then this split's share of the set tiles
    const bool sparse = (a.blockmask != nullptr);
    uint32_t* uni = reinterpret_cast<uint32_t*>(smem + SMEM_UNION);       // 64 words = 2048 key tiles
    volatile int* sp_info = reinterpret_cast<volatile int*>(abort_flag + 1);  // [0] first tile, [1] count
    // this row's token: first 64-key block always visible, and its mask row
    const int win_left = sparse ? (t + causal_base + 63) / 64 - a.block_window : 0;
    const uint64_t* bm_row = (sparse && row_valid) ? a.blockmask + (static_cast<size_t>(h) * a.tq + t) * a.bm_words : nullptr;
    if (sparse) {
        if (tid < 64) uni[tid] = 0u;
        __syncthreads();
        const int tok_n = max(min(t0 + a.tok_per_tile, tq_eff) - t0, 0);
        for (int kt = kt_lo + tid; kt < kt_hi; kt += NTHREADS) {
            bool any = false;
            for (int tt = 0; tt < tok_n && !any; ++tt) {
                const int left = (t0 + tt + causal_base + 63) / 64 - a.block_window;
                const uint64_t* r = a.blockmask + (static_cast<size_t>(h) * a.tq + t0 + tt) * a.bm_words;
#pragma unroll
                for (int hb = 0; hb < 2; ++hb) {
                    const int b = kt * 2 + hb;
                    any = any || b >= left || (((b >> 6) < a.bm_words) && ((r[b >> 6] >> (b & 63)) & 1ull));
                }
            }
            if (any) atomicOr(&uni[kt >> 5], 1u << (kt & 31));
        }
        __syncthreads();
        if (tid == 0) {
            int total = 0;
            for (int w = 0; w < 64; ++w) total += __popc(uni[w]);
            const int r0 = static_cast<int>((static_cast<long long>(total) * split) / nsplit);
            const int r1 = static_cast<int>((static_cast<long long>(total) * (split + 1)) / nsplit);
            int first = 0, seen = 0;
            for (int w = 0; w < 64 && r0 < r1; ++w) {  // tile index of the set bit with rank r0
                const int c = __popc(uni[w]);
                if (seen + c > r0) {
                    uint32_t v = uni[w];
                    for (int k = seen; k < r0; ++k) v &= v - 1;
                    first = w * 32 + __ffs(v) - 1;
                    break;
                }
                seen += c;
            }
            sp_info[0] = first;
            sp_info[1] = r1 - r0;
        }
        __syncthreads();
        kt_begin = sp_info[0];
        n_it = sp_info[1];
    }
    // key tile of iteration i + 1 given the tile of iteration i (dense: the next one)
    auto next_tile = [&](int kt) -> int {
        if (!sparse) return kt + 1;
        int w = (kt + 1) >> 5;
        uint32_t v = (w < 64) ? (uni[w] & (0xffffffffu << ((kt + 1) & 31))) : 0u;
        while (v == 0u && ++w < 64) v = uni[w];
        return v ? w * 32 + __ffs(v) - 1 : kt + 1;
    };

    float m_run = -INFINITY;  // running max of raw scores (same in both threads of a row)
    float l_run = 0.f;        // this thread's share of the running sum
    bool ok = true;

    if (is_control) {
        // ================================================= control warp: TMA + MMA issue
        if (lane == 0 && n_it > 0) {
            const uint32_t q_addr = ptx::smem_u32(smem + SMEM_Q);
            const uint32_t p_addr = ptx::smem_u32(smem + SMEM_P);
            constexpr uint32_t idesc_s = ptx::umma_idesc_bf16(ROWS, KEYS, 0, 0);
            constexpr uint32_t idesc_o = ptx::umma_idesc_bf16(ROWS, D, 0, 1);
            int k_tile = kt_begin, v_tile = kt_begin;  // tiles of the next K / V load (issued in iteration order)
            auto load_k = [&](int i) {
                const int st = i & 1, key0 = k_tile * KEYS;
                k_tile = next_tile(k_tile);
                ptx::mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
                ptx::tma_load_2d(smem + SMEM_K + st * TILE_BYTES, &tm_k, &k_full[st], h * D, key0);
                ptx::tma_load_2d(smem + SMEM_K + st * TILE_BYTES + HALF_BYTES, &tm_k, &k_full[st], h * D + 64, key0);
            };
            auto load_v = [&](int i) {
                const int st = i & 1, key0 = v_tile * KEYS;
                v_tile = next_tile(v_tile);
                ptx::mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
                ptx::tma_load_2d(smem + SMEM_V + st * TILE_BYTES, &tm_v, &v_full[st], h * D, key0);
                ptx::tma_load_2d(smem + SMEM_V + st * TILE_BYTES + HALF_BYTES, &tm_v, &v_full[st], h * D + 64, key0);
            };
            auto issue_s = [&](int i) -> bool {  // S(i) = Q K(i)^T into S stage i & 1
                const int st = i & 1;
                if (!ptx::mbar_wait(&k_full[st], (i >> 1) & 1, abort_flag)) return false;
                ptx::tc_fence_after();
                const uint32_t k_addr = ptx::smem_u32(smem + SMEM_K + st * TILE_BYTES);
#pragma unroll
                for (int dh = 0; dh < 2; ++dh) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t da = ptx::umma_desc_sw128(q_addr + dh * HALF_BYTES + j * 32, 16, 1024);
                        const uint64_t db = ptx::umma_desc_sw128(k_addr + dh * HALF_BYTES + j * 32, 16, 1024);
                        ptx::umma_ss(tmem_base + st * KEYS, da, db, idesc_s, (dh | j) ? 1u : 0u);
                    }
                }
                ptx::umma_commit(&s_bar[st]);
                return true;
            };
            ptx::mbar_arrive_expect_tx(q_bar, TILE_BYTES);
            ptx::tma_load_3d(smem + SMEM_Q, &tm_q, q_bar, 0, h * a.grp, t0);
            ptx::tma_load_3d(smem + SMEM_Q + HALF_BYTES, &tm_q, q_bar, 64, h * a.grp, t0);
            for (int i = 0; i < 2 && i < n_it; ++i) {
                load_k(i);
                load_v(i);
            }
            bool w = ptx::mbar_wait(q_bar, 0, abort_flag);
            for (int i = 0; w && i < 2 && i < n_it; ++i) w = issue_s(i);
            for (int i = 0; w && i < n_it; ++i) {
                const int st = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                // K stage st is free once S(i) has been computed: fetch K(i+2)
                if (i + 2 < n_it) {
                    if (!ptx::mbar_wait(&s_bar[st], ph, abort_flag)) { w = false; break; }
                    load_k(i + 2);
                }
                // O += P(i) V(i)
                if (!ptx::mbar_wait(&p_ready[st], ph, abort_flag)) { w = false; break; }
                if (!ptx::mbar_wait(&v_full[st], ph, abort_flag)) { w = false; break; }
                ptx::tc_fence_after();
                const uint32_t v_addr = ptx::smem_u32(smem + SMEM_V + st * TILE_BYTES);
                const uint32_t pa = p_addr + st * TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk) {
                    // A: P, K-major: 64-key half (kk / 4), 32 B per 16-key step inside it
                    const uint64_t da = ptx::umma_desc_sw128(pa + (kk >> 2) * HALF_BYTES + (kk & 3) * 32, 16, 1024);
                    // B: V, N-major: 16 key rows of 128 B per step; 64-wide d halves HALF_BYTES apart
                    const uint64_t db = ptx::umma_desc_sw128(v_addr + kk * 16 * 128, HALF_BYTES, 1024);
                    ptx::umma_ss(tmem_base + TMEM_O, da, db, idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
                }
                ptx::umma_commit(&o_bar[st]);
                // S(i+2) reuses S stage st: softmax(i) has read it (p_ready) and K(i+2) is on its way
                if (i + 2 < n_it) {
                    if (!issue_s(i + 2)) { w = false; break; }
                    // V stage st is free once PV(i) has finished
                    if (!ptx::mbar_wait(&o_bar[st], ph, abort_flag)) { w = false; break; }
                    load_v(i + 2);
                }
            }
        }
    } else {
        // ================================================= softmax warps
        int s_tile = kt_begin;
        long long pt_s = 0, pt_ld = 0, pt_bar = 0, pt_o = 0, pt_exp = 0;
        const long long pt_begin = prof_clock();
        for (int i = 0; i < n_it && ok; ++i) {
            const int st = i & 1;
            const uint32_t ph = (i >> 1) & 1;
            const int key0 = s_tile * KEYS + ch * 64;  // first key of this thread's 64 columns
            const long long pc0 = prof_clock();
            s_tile = next_tile(s_tile);
            // block-sparse mode: this row's token may not see this 64-key block at all
            bool blk_ok = true;
            if (sparse) {
                const int b = key0 >> 6;
                blk_ok = b >= win_left ||
                         (bm_row != nullptr && (b >> 6) < a.bm_words && ((bm_row[b >> 6] >> (b & 63)) & 1ull));
            }
            // one polling lane per warp (the shuffle also converges it for the collective TMEM loads)
            if (!ptx::mbar_wait_warp(&s_bar[st], ph, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const long long pc1 = prof_clock();

            // ---- scores of this thread: 64 columns, kept in registers for both passes
            uint32_t sc[64];
            const uint32_t tmem_s = tmem_base + lane_sel + st * KEYS + ch * 64;
            ptx::tmem_ld32(tmem_s, sc);
            ptx::tmem_ld32(tmem_s + 32, sc + 32);
            ptx::tmem_wait_ld();
            // visibility of this thread's 64 keys as one 64-bit word: causal bound, window bound, tree-mask bits,
            // block selection.  (A per-key chain of comparisons here made the half-empty last token tile of a
            // verify pass, whose rows see nothing, 2.2 times slower than the full tiles.)
            uint64_t vb = ~0ull;
            if (!blk_ok || limit <= key0 || key_lo >= key0 + 64) {
                vb = 0ull;
            } else {
                if (limit < key0 + 64) vb &= (1ull << (limit - key0)) - 1ull;
                if (key_lo > key0) vb &= ~((1ull << (key_lo - key0)) - 1ull);
                const int mo = mbeg - key0;  // first column the tree mask applies to (mbeg is huge when there is none)
                if (mo < 64) {
                    const uint64_t tm = (mo >= 0) ? ((mo > 0 ? (mword << mo) : mword) | ((1ull << mo) - 1ull))
                                                  : ((-mo < 64) ? (mword >> (-mo)) : 0ull);
                    vb &= tm;
                }
            }
            if (vb != ~0ull) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    if (!((vb >> c) & 1ull)) sc[c] = 0xff800000u;  // -inf
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; c += 4) {
                mx[0] = fmaxf(mx[0], __uint_as_float(sc[c]));
                mx[1] = fmaxf(mx[1], __uint_as_float(sc[c + 1]));
                mx[2] = fmaxf(mx[2], __uint_as_float(sc[c + 2]));
                mx[3] = fmaxf(mx[3], __uint_as_float(sc[c + 3]));
            }
            const float m_half = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const long long pc2 = prof_clock();
            xch[ch * ROWS + row] = m_half;
            ptx::named_bar_sync(1, SOFTMAX_THREADS);
            const float m_tile = fmaxf(m_half, xch[(ch ^ 1) * ROWS + row]);
            ptx::named_bar_sync(2, SOFTMAX_THREADS);  // xch is rewritten by the next iteration
            const long long pc3 = prof_clock();
            // Lazy running maximum: the reference maximum of a row moves only when the new one is more than
            // 2^8 above it (or the row had none yet).  Exponentials then stay below 256 (exact enough in bf16 P
            // and fp32 sums), and O has to be rescaled - which needs the previous PV to have finished and
            // serialises the pipeline - only on such jumps instead of whenever any row of a warp sees a new maximum.
            float m_new = m_run;
            if (m_tile != -INFINITY && (m_run == -INFINITY || (m_tile - m_run) * a.scale_log2 > 8.f)) m_new = m_tile;
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = (m_run == -INFINITY) ? 1.f : fast_exp2((m_run - m_use) * a.scale_log2);
            const bool rescale = (i > 0) && __any_sync(0xffffffffu, alpha != 1.f);
            if (rescale) {  // O must hold every product issued so far: wait for PV(i-1)
                if (!ptx::mbar_wait_warp(&o_bar[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 32) {
                    uint32_t r[32];
                    ptx::tmem_ld32(tmem_o + c0, r);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                    ptx::tmem_st32(tmem_o + c0, r);
                }
                ptx::tmem_wait_st();
            }
            m_run = m_new;
            if (i >= 2) {  // P stage st was last read by PV(i-2)
                if (!ptx::mbar_wait_warp(&o_bar[st], ((i - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
            }
            const long long pc4 = prof_clock();

            // ---- P = 2^((s - m) * scale) in bf16 into the swizzled A-operand tile; row sums in fp32
            const float m_off = m_use * a.scale_log2;
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
            uint8_t* p_half = smem + SMEM_P + st * TILE_BYTES + ch * HALF_BYTES + row * 128;
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = fast_exp2(fmaf(__uint_as_float(sc[c8 * 8 + e]), a.scale_log2, -m_off));
                    ls[e & 3] += p[e];
                }
                uint4 pk;
                uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(p[e * 2], p[e * 2 + 1]);
                    w[e] = *reinterpret_cast<uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(p_half + ((c8 ^ (row & 7)) << 4)) = pk;
            }
            l_run = l_run * alpha + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
            ptx::fence_proxy_async_smem();  // P stores -> visible to the tensor core's async proxy
            ptx::tc_fence_before();         // TMEM reads / rescale ordered before the control warp's next MMA
            __syncwarp();
            if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(&p_ready[st]);
            if (kAttnProf) {
                const long long pc5 = prof_clock();
                pt_s += pc1 - pc0; pt_ld += pc2 - pc1; pt_bar += pc3 - pc2; pt_o += pc4 - pc3; pt_exp += pc5 - pc4;
            }
        }
        if (kAttnProf && a.prof != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) {
            a.prof[0] = prof_clock() - pt_begin; a.prof[1] = pt_s; a.prof[2] = pt_ld; a.prof[3] = pt_bar;
            a.prof[4] = pt_o; a.prof[5] = pt_exp; a.prof[6] = n_it; a.prof[7] = pt_begin - pt_kernel;
        }
        if (ok && n_it > 0) {
            if (!ptx::mbar_wait_warp(&o_bar[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, abort_flag)) ok = false;
            ptx::tc_fence_after();
        }
        ok = __all_sync(0xffffffffu, ok);  // keep each warp together for the collective TMEM reads

        // ---- write-out.  TMEM reads are warp-collective, so every thread runs them
        // and only the global stores depend on whether the row exists.
        xch[ch * ROWS + row] = l_run;
        ptx::named_bar_sync(1, SOFTMAX_THREADS);
        const float l_row = l_run + xch[(ch ^ 1) * ROWS + row];
        if (ok) {
            const bool store = (t < a.tq);
            const size_t grow = static_cast<size_t>(store ? t : 0) * a.hq + qh;
            const float inv = (nsplit == 1) ? ((l_row > 0.f) ? 1.f / l_row : 0.f) : 1.f;
            bf16* dst_b = a.out + static_cast<size_t>(store ? t : 0) * a.out_ld + qh * D + ch * 64;
            float* dst_f =
                (nsplit > 1) ? a.ws_o + (static_cast<size_t>(split) * a.tq * a.hq + grow) * D + ch * 64 : nullptr;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t r[32];
                if (n_it > 0) {  // uniform across the CTA
                    ptx::tmem_ld32(tmem_o + c0, r);
                    ptx::tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) r[c] = 0;
                }
                if (store) {
                    if (nsplit == 1) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint4 pk;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[c + e * 2]) * inv,
                                                                          __uint_as_float(r[c + e * 2 + 1]) * inv);
                                w[e] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(dst_b + c0 + c) = pk;
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; c += 4) {
                            *reinterpret_cast<uint4*>(dst_f + c0 + c) = make_uint4(r[c], r[c + 1], r[c + 2], r[c + 3]);
                        }
                    }
                }
            }
            if (store && nsplit > 1 && ch == 0) {
                float* ml = a.ws_ml + (static_cast<size_t>(split) * a.tq * a.hq + grow) * 2;
                ml[0] = m_run;
                ml[1] = l_row;
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (tid == 0 && *abort_flag) atomicOr(a.error, ERR_ATTN_TIMEOUT);
    if (kAttnProf && a.prof != nullptr && tid == 0) {
        if (blockIdx.x == 0 && blockIdx.y == 0) a.prof[8] = prof_clock() - pt_kernel;
        a.prof[16 + blockIdx.y * gridDim.x + blockIdx.x] = prof_clock() - pt_dep;  // active time of every CTA
    }
}

// Merge split partials: out = sum_s 2^((m_s - M) c) O_s / sum_s 2^((m_s - M) c) l_s.
// One warp per (token, head) row; lane s first owns split s's (max, sum) pair, then
// every lane accumulates four output columns with independent loads in flight.
__global__ void attn_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, int nsplit,
                                    int rows, int hq, float scale_log2, bf16* __restrict__ out, int out_ld) {
    grid_dependency_sync();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    // the first twelve splits' partial outputs are requested before the (max, sum) pairs they are weighted
    // with: both loads are in flight together instead of one L2 round trip after the other
    constexpr int B = 12;
    const float* base = ws_o + static_cast<size_t>(row) * D + lane * 4;
    const size_t stride = static_cast<size_t>(rows) * D;
    float4 o[B];
#pragma unroll
    for (int j = 0; j < B; ++j) {
        o[j] = (j < nsplit) ? __ldcg(reinterpret_cast<const float4*>(base + j * stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m_s = -INFINITY, l_s = 0.f;
    if (lane < nsplit) {
        const float2 ml = *reinterpret_cast<const float2*>(ws_ml + (static_cast<size_t>(lane) * rows + row) * 2);
        m_s = ml.x;
        l_s = ml.y;
    }
    float M = m_s;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
    const float w_s = (m_s == -INFINITY) ? 0.f : exp2f((m_s - M) * scale_log2);
    float l = w_s * l_s;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o2);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsplit; s0 += B) {
        if (s0 > 0) {
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int s = s0 + j;
                o[j] = (s < nsplit) ? __ldcg(reinterpret_cast<const float4*>(base + s * stride)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int s = s0 + j;
            const float w = (s < nsplit) ? __shfl_sync(0xffffffffu, w_s, s & 31) : 0.f;
            acc.x += w * o[j].x;
            acc.y += w * o[j].y;
            acc.z += w * o[j].z;
            acc.w += w * o[j].w;
        }
    }
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    const int t = row / hq, qh = row - t * hq;
    __nv_bfloat162 a0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    __nv_bfloat162 a1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&a0);
    pk.y = *reinterpret_cast<uint32_t*>(&a1);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(t) * out_ld + qh * D + lane * 4) = pk;
}

}  // namespace

size_t attn_workspace_bytes(int tq, int hq, int d, int splits) {
    return static_cast<size_t>(splits) * tq * hq * (d + 2) * sizeof(float);
}

AttnPlan make_attn_plan(const bf16* q, int q_ld_tokens, const bf16* k_cache, const bf16* v_cache, int budget, int tq,
                        int hq, int hkv, int d, int splits, bf16* out, int out_ld, float* ws_o, float* ws_ml) {
    CPM_REQUIRE(d == D, "attention: head_dim must be 128");
    CPM_REQUIRE(hq % hkv == 0, "attention: query heads must be a multiple of kv heads");
    const int grp = hq / hkv;
    CPM_REQUIRE(grp <= ROWS && ROWS % grp == 0, "attention: unsupported GQA ratio");
    CPM_REQUIRE(tq >= 1 && splits >= 1 && splits <= 32, "attention: splits must be in [1,32]");
    AttnPlan p;
    p.tq = tq; p.hq = hq; p.hkv = hkv; p.d = d; p.splits = splits;
    p.out = out; p.out_ld = out_ld; p.ws_o = ws_o; p.ws_ml = ws_ml;
    p.scale = 1.0f / sqrtf(static_cast<float>(d));
    p.tm_q = make_tmap_3d(q, d, hq, tq, static_cast<uint64_t>(d) * 2, static_cast<uint64_t>(q_ld_tokens) * 2, 64, grp,
                          ROWS / grp);
    p.tm_k = make_tmap_2d(k_cache, static_cast<uint64_t>(hkv) * d, budget, static_cast<uint64_t>(hkv) * d * 2, 64, KEYS);
    p.tm_v = make_tmap_2d(v_cache, static_cast<uint64_t>(hkv) * d, budget, static_cast<uint64_t>(hkv) * d * 2, 64, KEYS);
    return p;
}

void launch_tree_attention(const AttnPlan& p, cudaStream_t s) {
    ProfileScope prof(KC_ATTENTION, s);
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(tree_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        configured = true;
    }
    AttnArgs a;
    a.tq = p.tq; a.hq = p.hq; a.hkv = p.hkv;
    a.grp = p.hq / p.hkv;
    a.tok_per_tile = ROWS / a.grp;
    a.num_mtiles = ceil_div(p.tq, a.tok_per_tile);
    // One split over many token tiles is a causal prefill: a tile's work grows with its position, and CTAs are
    // dispatched in blockIdx order, so the longest tiles go first and the short ones fill the tail.
    a.heavy_first = (p.splits == 1 && a.num_mtiles > 1) ? 1 : 0;
    a.kv_len = p.kv_len; a.kv_len_add = p.kv_len_add;
    a.n_valid = p.n_valid;
    a.mask = p.mask; a.mask_k = p.mask_k;
    a.window = p.window;
    a.blockmask = p.blockmask; a.bm_words = p.bm_words; a.block_window = p.block_window;
    CPM_REQUIRE(p.blockmask == nullptr || (p.bm_words >= 1 && p.bm_words <= 64 && p.block_window >= 1),
                "attention: block mask needs 1..64 words per row and a local window of at least one block");
    a.scale_log2 = p.scale * 1.4426950408889634f;
    a.out = p.out; a.out_ld = p.out_ld;
    a.ws_o = p.ws_o; a.ws_ml = p.ws_ml;
    a.error = runtime().d_error;
    a.prof = nullptr;
    if (kAttnProf) {
        static long long* buf = nullptr;
        if (buf == nullptr) {
            CUDA_CHECK(cudaMalloc(&buf, 4096 * sizeof(long long)));
            CUDA_CHECK(cudaMemset(buf, 0, 4096 * sizeof(long long)));
        }
        a.prof = buf;
        static int calls = 0;
        if (++calls % 32 == 0) {
            long long hst[9];
            CUDA_CHECK(cudaMemcpy(hst, buf, sizeof(hst), cudaMemcpyDeviceToHost));
            fprintf(stderr, "attn prof (CTA 0, softmax thread 0): loop %lld cycles, %lld tiles: wait S %lld, load+max %lld, "
                            "row-max exchange %lld, rescale + wait PV(i-2) %lld, exp + P store %lld; before the loop %lld, "
                            "whole kernel %lld\n",
                    hst[0], hst[6], hst[1], hst[2], hst[3], hst[4], hst[5], hst[7], hst[8]);
            std::vector<long long> act(a.num_mtiles * p.hkv * p.splits);
            CUDA_CHECK(cudaMemcpy(act.data(), buf + 16, act.size() * sizeof(long long), cudaMemcpyDeviceToHost));
            long long lo = act[0], hi = act[0], sum = 0;
            for (long long v : act) { lo = std::min(lo, v); hi = std::max(hi, v); sum += v; }
            fprintf(stderr, "attn prof: active cycles per CTA after the dependency wait: min %lld mean %lld max %lld over %zu CTAs\n",
                    lo, sum / static_cast<long long>(act.size()), hi, act.size());
            const int gx = a.num_mtiles * p.hkv;
            for (int sp = 0; sp < p.splits; ++sp) {
                fprintf(stderr, "  split %d:", sp);
                for (int x = 0; x < gx; ++x) fprintf(stderr, " %lld", act[sp * gx + x] / 1000);
                fprintf(stderr, "\n");
            }
        }
    }
    CPM_REQUIRE(p.splits == 1 || (p.ws_o != nullptr && p.ws_ml != nullptr), "attention: split-KV needs a workspace");
    dim3 grid(a.num_mtiles * p.hkv, p.splits);
    launch_kernel(tree_attn_kernel, grid, dim3(NTHREADS), SMEM_TOTAL, s, p.tm_q, p.tm_k, p.tm_v, a);
    if (p.splits > 1) {
        const int rows = p.tq * p.hq;
        launch_kernel(attn_combine_kernel, dim3(ceil_div(rows, 4)), dim3(128), 0, s, p.ws_o, p.ws_ml, p.splits, rows, p.hq,
                      a.scale_log2, p.out, p.out_ld);
    }
}
