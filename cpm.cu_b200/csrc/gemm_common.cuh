// Pieces shared by the bf16 and the W4A16 weight-streaming GEMM kernels: the stream-K work
// split and the epilogue (TMEM read-out, split-K partials, ticketed deterministic fix-up).
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace gemm {

constexpr int BLOCK_N = 128;  // weight rows per tile (UMMA M)

struct LinearArgs {
    int M, N, K;
    int n_tiles, m_tiles, kblocks;
    long long total_units;
    bf16* y;
    int ldy;
    const bf16* bias;
    float* workspace;
    int* tickets;
    int* error;
    int debug;  // bench-only switches: 1 = skip the X loads, 2 = skip epilogue stores and the split-K fix-up
    long long* prof;  // bench only (-DCPMCU_GEMM_PROFILE): [grid][4] clock counters, or null
    // Tiles [0, wave_tiles) are computed whole, tile g + i * gridDim.x by CTA g; total_units counts the k-blocks of
    // the tiles from wave_tiles on, which the first tail_grid CTAs (0 = all) share in equal contiguous pieces.
    int wave_tiles = 0;
    int tail_grid = 0;
    // SwiGLU epilogue (whole tiles only): a weight tile is 64 gate rows followed by the 64 up rows of the same
    // features, N counts output features (the gate half), y[token][feature] = silu(gate) * up.
    int swiglu = 0;
    int band = 16;   // token tiles per raster band (tile_to_mn)
};

// Shared memory the SwiGLU epilogue exchanges up-projection values through: two buffers of
// [2 warps][16 tokens][32 lanes] floats.
constexpr int SWIGLU_XCH_BYTES = 2 * 2 * 16 * 32 * 4;

#ifdef CPMCU_GEMM_PROFILE
constexpr bool kGemmProf = true;
#else
constexpr bool kGemmProf = false;
#endif

// The work of one CTA: the k-blocks [u, u_end) of the line of (tile, k-block) units that starts at tile wave_tiles,
// then the whole tiles wave_tile, wave_tile + stride, ... below wave_tiles.
struct SegIter {
    long long u, u_end;
    int kblocks;
    int wave_tile = 0, wave_tiles = 0, stride = 1;
    // The cut tiles come first: the piece counted last sums the tile in the epilogue warps while the MMA warp is
    // already on the CTA's whole tiles, so the fix-up through the workspace hides behind them instead of ending
    // the kernel.
    __host__ __device__ bool next(int& tile, int& kb0, int& kb1) {
        if (u < u_end) {
            const int t = static_cast<int>(u / kblocks);
            tile = wave_tiles + t;
            kb0 = static_cast<int>(u - static_cast<long long>(t) * kblocks);
            long long rem = u_end - u;
            kb1 = (kb0 + rem < kblocks) ? static_cast<int>(kb0 + rem) : kblocks;
            u += kb1 - kb0;
            return true;
        }
        if (wave_tile < wave_tiles) {
            tile = wave_tile;
            kb0 = 0;
            kb1 = kblocks;
            wave_tile += stride;
            return true;
        }
        return false;
    }
};

// Work of CTA g of G.  With wave_tiles = 0 (every launch of a single token tile) this is plain stream-K: the
// line of all (tile, k-block) units cut into G equal pieces.  Launches with several token tiles run whole tiles
// in waves: the CTAs of a wave walk K in step, so tiles that share a weight or an activation slab find it
// in L2 instead of each fetching it from HBM at a different time; only the tiles of the partial wave are cut along K.
__host__ __device__ __forceinline__ SegIter make_seg_iter(const LinearArgs& a, int g, int G) {
    SegIter it;
    it.kblocks = a.kblocks;
    it.wave_tiles = a.wave_tiles;
    it.wave_tile = g;
    it.stride = G;
    const int gt = a.tail_grid > 0 ? a.tail_grid : G;
    if (g < gt) {
        it.u = (a.total_units * g) / gt;
        it.u_end = (a.total_units * (g + 1)) / gt;
    } else {
        it.u = it.u_end = 0;
    }
    return it;
}

// Tile number -> (token tile, feature tile).  Token tiles are taken in bands of a.band; inside a band the
// token tile runs fastest, so the tiles a wave of CTAs works on at one time cover few feature tiles x all token
// tiles of the band: every weight slab is fetched from HBM once per band and the band's activations stay in L2.
__host__ __device__ __forceinline__ void tile_to_mn(const LinearArgs& a, int tile, int& m_tile, int& n_tile) {
    if (a.m_tiles == 1) {
        m_tile = 0;
        n_tile = tile;
        return;
    }
    const int band_tiles = a.band * a.n_tiles;
    const int band = tile / band_tiles;
    const int r = tile - band * band_tiles;
    int bm = a.m_tiles - band * a.band;
    if (bm > a.band) bm = a.band;
    n_tile = r / bm;
    m_tile = band * a.band + (r - n_tile * bm);
}

// Token tiles per band: as many as keep the band's activations (band * mt rows of K bf16) within half of the
// 126 MB L2, at most 16.  With K = 16384 and 256-token tiles that is 8: a band of 16 (134 MB) was re-read from HBM by
// every wave (1.1 GB of DRAM reads for 268 MB of operands in one ncu capture of the 4096-token down projection).
inline int raster_band(int mt, int K) {
    const long long rows = (64LL << 20) / (static_cast<long long>(K) * 2);
    int band = static_cast<int>(rows / mt);
    if (band < 1) band = 1;
    if (band > 16) band = 16;
    return band;
}

// Host side of make_seg_iter for a launch with several token tiles: whole waves of `grid` tiles, and the CTAs
// that share the rest (pieces of at least eight k-blocks, or whole tiles when a tile has fewer).
inline void plan_waves(long long tiles, int kblocks, int grid, int& wave_tiles, int& tail_grid) {
    wave_tiles = static_cast<int>((tiles / grid) * grid);
    const long long tail_units = (tiles - wave_tiles) * kblocks;
    long long gt = tail_units / 8;
    if (gt < tiles - wave_tiles) gt = tiles - wave_tiles;
    if (gt < 1) gt = 1;
    if (gt > grid) gt = grid;
    tail_grid = static_cast<int>(gt);
}

// CTA that owns work unit u when [0,U) is cut into G pieces starting at floor(g*U/G).
__host__ __device__ __forceinline__ int unit_owner(long long u, long long U, int G) {
    return static_cast<int>(((u + 1) * G - 1) / U);
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// A split tile this CTA holds a piece of: summed after the CTA's last segment.
struct PendingTile {
    int tile, g_first, nseg, m_base, m_cnt, n;
    float bias;
};

// Sum tokens [t_begin, t_end) of a split tile over its pieces in CTA order (deterministic) and store them:
// CH tokens per pass, the coalesced loads of up to four pieces (4 * CH per thread) in flight before the adds.
template <int MT, int CH>
__device__ __forceinline__ void sum_pieces(const LinearArgs& a, const PendingTile& p, int t_begin, int t_end, int row) {
    const int g_last = p.g_first + p.nseg - 1;
#pragma unroll 1
    for (int c0 = t_begin; c0 < t_end; c0 += CH) {
        float sum[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) sum[c] = 0.f;
#pragma unroll 1
        for (int g0 = p.g_first; g0 <= g_last; g0 += 4) {
            float v[4][CH];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const int gg = g0 + s;
                const float* ws = a.workspace + (static_cast<size_t>(gg) * 2 + (gg == p.g_first ? 1 : 0)) * (MT * BLOCK_N) +
                                  static_cast<size_t>(c0) * BLOCK_N + row;
#pragma unroll
                for (int c = 0; c < CH; ++c) v[s][c] = (gg <= g_last && c0 + c < t_end) ? __ldcg(ws + c * BLOCK_N) : 0.f;
            }
#pragma unroll
            for (int s = 0; s < 4; ++s) {
#pragma unroll
                for (int c = 0; c < CH; ++c) sum[c] += v[s][c];
            }
        }
        if (p.n < a.N) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                if (c0 + c < t_end) {
                    a.y[static_cast<size_t>(p.m_base + c0 + c) * a.ldy + p.n] = __float2bfloat16(sum[c] + p.bias);
                }
            }
        }
    }
}

// Longest a CTA waits for the other pieces of a tile (about 50 ms); they are computed by CTAs of the same
// launch that finish at about the same time, so only a grid that is not co-resident gets near it.
constexpr long long kFixupBudgetClocks = 100000000LL;

// Epilogue of the four warps whose (warp & 3) selects the TMEM lane quarter.  `it` walks the same
// segments as the producer and MMA roles; a.kblocks is the number of work units per tile.
//
// Whole tiles are written to y directly.  A piece of a split tile goes to this CTA's workspace slot as
// fp32 [token][feature] and is counted in tickets[2 * tile].  Tiles cut in two, or with few tokens, are
// summed on the spot by whichever piece is counted last.  A tile cut into three or more pieces is summed
// after the CTA's last segment instead: the CTA waits until every piece of that tile has been counted and
// sums ITS share of the tokens over all pieces, so the fix-up is spread over the CTAs that produced the
// tile instead of falling to one (tickets[2 * tile + 1] counts departures; the last one clears both
// counters for the next launch).  That path needs the whole grid resident (grid <= SMs, one CTA per
// SM).  Pieces are always added in CTA order, so the result does not depend on timing.  CH = tokens
// summed per pass.  chain2_off != 0: the MMA role accumulated alternate k-blocks into a second
// accumulator that many columns further on; the two are added here.
template <int MT, int CH>
__device__ __forceinline__ void run_epilogue(const LinearArgs& a, SegIter it, uint32_t tmem_base, uint64_t* acc_full,
                                             uint64_t* acc_empty, volatile int* abort_flag, volatile int* s_last, int warp,
                                             int lane, int epi_tid, int g, int G, uint32_t chain2_off = 0,
                                             int acc_stages = 2, float* swiglu_xch = nullptr) {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // output feature within the tile
    int acc = 0;
    uint32_t acc_phase = 0;
    int tile, kb0, kb1;
    PendingTile pend[2];
    int n_pend = 0;
    int xi = 0;  // SwiGLU exchange buffer of the next 16-token batch
    // ---- split tiles: wait for the other pieces, sum this CTA's share of the tokens
    auto flush_pending = [&]() {
        for (int i = 0; i < n_pend; ++i) {
            const PendingTile& p = pend[i];
            if (epi_tid == 0) {
                const long long t0 = clock64();
                int ok = 1;
                while (ld_acquire(&a.tickets[2 * p.tile]) < p.nseg) {
                    if (*abort_flag || clock64() - t0 > kFixupBudgetClocks) { ok = 0; *abort_flag = 1; break; }
                }
                *s_last = ok;
            }
            ptx::named_bar_sync(1, 128);
            const bool ready = (*s_last != 0);
            ptx::named_bar_sync(1, 128);  // everyone has read s_last before it can change
            if (ready && !CPM_EXPERIMENT(a, 16)) {
                const int piece = g - p.g_first;
                sum_pieces<MT, CH>(a, p, (p.m_cnt * piece) / p.nseg, (p.m_cnt * (piece + 1)) / p.nseg, row);
            }
            if (ready) {
                // the partials of this tile may be overwritten once every piece's reader has left
                ptx::named_bar_sync(1, 128);
                if (epi_tid == 0) {
                    const int old = atomicAdd(&a.tickets[2 * p.tile + 1], 1);
                    if (old == p.nseg - 1) {
                        a.tickets[2 * p.tile + 1] = 0;
                        __threadfence();
                        a.tickets[2 * p.tile] = 0;  // ready for the next launch
                    }
                }
            }
        }
        n_pend = 0;
    };
    while (it.next(tile, kb0, kb1)) {
        // the cut tiles of a launch come before its whole tiles: their sums are done here, while the MMA warp
        // works on the whole tiles, not at the end of the kernel
        if (n_pend > 0 && tile < a.wave_tiles) flush_pending();
        int m_tile, n_tile;
        tile_to_mn(a, tile, m_tile, n_tile);
        const int m_base = m_tile * MT;
        if (a.swiglu != 0 && swiglu_xch != nullptr) {
            // Lanes 0-63 of the accumulator hold the gate projection of 64 features, lanes 64-127 the up projection
            // of the same features.  Both are rounded to bf16 as the unfused pair of kernels stores them; the two
            // warps of the gate half pass theirs through shared memory and the two warps of the up half (the ones
            // that share no scheduler with the producer or the MMA warp) store silu(gate) * up.
            int m_cnt = a.M - m_base;
            if (m_cnt > MT) m_cnt = MT;
            const int n_out = n_tile * 64 + (row & 63);
            if (!ptx::mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag)) break;
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * MT;
#pragma unroll 1
            for (int c0 = 0; c0 < MT; c0 += 16) {
                if (c0 >= m_cnt) break;  // uniform across the CTA
                uint32_t r[16];
                ptx::tmem_ld16(t_addr + c0, r);
                ptx::tmem_wait_ld();
                float* xb = swiglu_xch + (xi & 1) * (2 * 16 * 32);
                ++xi;
                if (q < 2) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        xb[(q * 16 + c) * 32 + lane] = __bfloat162float(__float2bfloat16(__uint_as_float(r[c])));
                    }
                }
                // the batch after the next one reuses this buffer: its writers pass the next batch's barrier only
                // after this batch's readers have arrived there
                ptx::named_bar_sync(1, 128);
                if (q >= 2 && n_out < a.N) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        if (c0 + c < m_cnt) {
                            const float uv = __bfloat162float(__float2bfloat16(__uint_as_float(r[c])));
                            const float gv = xb[((q - 2) * 16 + c) * 32 + lane];
                            a.y[static_cast<size_t>(m_base + c0 + c) * a.ldy + n_out] = __float2bfloat16(silu_mul(gv, uv));
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(&acc_empty[acc]);
            if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }
            continue;
        }
        const int n = n_tile * BLOCK_N + row;
        int m_cnt = a.M - m_base;
        if (m_cnt > MT) m_cnt = MT;
        const bool complete = (kb0 == 0 && kb1 == a.kblocks);
        // partial slot: pieces that start mid-tile use slot 0 of this CTA, the
        // piece that starts a tile but does not finish it uses slot 1
        float* my_ws = a.workspace + (static_cast<size_t>(g) * 2 + (kb0 == 0 ? 1 : 0)) * (MT * BLOCK_N);
        const float bias_v = (a.bias != nullptr && n < a.N) ? __bfloat162float(a.bias[n]) : 0.f;

        if (!ptx::mbar_wait_warp(&acc_full[acc], acc_phase, abort_flag)) break;  // also converges the warp
        ptx::tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * MT;
        // partial slot layout: [MT tokens][128 features] fp32: a warp touches one 128-byte line per token
#pragma unroll 1
        for (int c0 = 0; c0 < MT; c0 += 16) {
            if (c0 >= m_cnt || CPM_EXPERIMENT(a, 2)) break;  // uniform across the CTA
            uint32_t r[16];
            ptx::tmem_ld16(t_addr + c0, r);
            if (chain2_off != 0) {
                uint32_t r2[16];
                ptx::tmem_ld16(t_addr + chain2_off + c0, r2);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) + __uint_as_float(r2[c]));
            }
            ptx::tmem_wait_ld();
            if (complete) {
                if (n < a.N) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        if (c0 + c < m_cnt) {
                            a.y[static_cast<size_t>(m_base + c0 + c) * a.ldy + n] =
                                __float2bfloat16(__uint_as_float(r[c]) + bias_v);
                        }
                    }
                }
            } else if (!CPM_EXPERIMENT(a, 4)) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    if (c0 + c < m_cnt) my_ws[(c0 + c) * BLOCK_N + row] = __uint_as_float(r[c]);
                }
            }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(&acc_empty[acc]);
        if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }

        if (!complete && !CPM_EXPERIMENT(a, 2 | 8)) {
            const long long tile_u0 = static_cast<long long>(tile - a.wave_tiles) * a.kblocks;
            const int gt = a.tail_grid > 0 ? a.tail_grid : G;
            PendingTile p;
            p.tile = tile;
            p.g_first = unit_owner(tile_u0, a.total_units, gt);
            p.nseg = unit_owner(tile_u0 + a.kblocks - 1, a.total_units, gt) - p.g_first + 1;
            p.m_base = m_base; p.m_cnt = m_cnt; p.n = n; p.bias = bias_v;
            const bool spread = (p.nseg >= 3 && m_cnt > 16);
            __threadfence();               // this thread's partials are visible before the count
            ptx::named_bar_sync(1, 128);
            if (spread) {
                if (epi_tid == 0) atomicAdd(&a.tickets[2 * tile], 1);
                pend[n_pend++] = p;
            } else {
                if (epi_tid == 0) {
                    const int old = atomicAdd(&a.tickets[2 * tile], 1);
                    const int last = (old == p.nseg - 1) ? 1 : 0;
                    if (last) a.tickets[2 * tile] = 0;  // ready for the next launch
                    *s_last = last;
                }
                ptx::named_bar_sync(1, 128);
                const bool is_last = (*s_last != 0);
                ptx::named_bar_sync(1, 128);  // everyone has read s_last before it can change
                if (is_last && !CPM_EXPERIMENT(a, 16)) {
                    __threadfence();
                    sum_pieces<MT, CH>(a, p, 0, m_cnt, row);
                }
            }
        }
    }

    flush_pending();
}

// Second half of split-K inside a thread-block cluster of CS CTAs that hold the CS k-pieces of one output
// tile (rank = piece).  Called by EVERY thread of the CTA after a cluster barrier that found all operand
// rings idle; `epi` marks the 128 epilogue threads, whose v[] holds this CTA's partial sums of feature `row`
// for all MT tokens.  Every CTA sends each peer that peer's share of the tokens (TPR = ceil(MT / CS)) into the
// peer's `red` buffer (fp32 [source][token][feature], CS * TPR * 128 floats of idle shared memory), one more
// cluster barrier, then sums and stores its own tokens in rank order: the order the workspace path adds its
// pieces in.  No waits other than the two hardware barriers, which every thread reaches.
template <int MT, int CS>
__device__ __forceinline__ void cluster_reduce_store(const LinearArgs& a, const float (&v)[MT], float* red, int rank,
                                                     int n_tile, bool epi, int row) {
    constexpr int TPR = (MT + CS - 1) / CS;
    int m_cnt = a.M;
    if (m_cnt > MT) m_cnt = MT;
    if (epi) {
        const uint32_t mine = ptx::smem_u32(red + (rank * TPR) * BLOCK_N + row);
#pragma unroll
        for (int d = 0; d < CS; ++d) {
            if (d != rank) {
                const uint32_t dst = ptx::cluster_map(mine, static_cast<uint32_t>(d));
#pragma unroll
                for (int tt = 0; tt < TPR; ++tt) {
                    if (d * TPR + tt < MT) {
                        if (d * TPR + tt < m_cnt) ptx::st_cluster_f32(dst + tt * BLOCK_N * 4, v[(d * TPR + tt) % MT]);
                    }
                }
            }
        }
    }
    __syncwarp();
    ptx::cluster_sync();   // the peers' shares of this CTA's tokens have arrived
    if (epi) {
        const int n = n_tile * BLOCK_N + row;
        const float bias_v = (a.bias != nullptr && n < a.N) ? __bfloat162float(a.bias[n]) : 0.f;
#pragma unroll
        for (int tt = 0; tt < TPR; ++tt) {
            float own = 0.f;
#pragma unroll
            for (int d = 0; d < CS; ++d) {
                if (d * TPR + tt < MT) {
                    if (d == rank) own = v[(d * TPR + tt) % MT];
                }
            }
            const int t = rank * TPR + tt;
            if (t < m_cnt && n < a.N) {
                float sum = 0.f;
#pragma unroll
                for (int s = 0; s < CS; ++s) sum += (s == rank) ? own : red[(s * TPR + tt) * BLOCK_N + row];
                a.y[static_cast<size_t>(t) * a.ldy + n] = __float2bfloat16(sum + bias_v);
            }
        }
    }
}

}  // namespace gemm
