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
};

struct SegIter {
    long long u, u_end;
    int kblocks;
    __device__ bool next(int& tile, int& kb0, int& kb1) {
        if (u >= u_end) return false;
        tile = static_cast<int>(u / kblocks);
        kb0 = static_cast<int>(u - static_cast<long long>(tile) * kblocks);
        long long rem = u_end - u;
        kb1 = (kb0 + rem < kblocks) ? static_cast<int>(kb0 + rem) : kblocks;
        u += kb1 - kb0;
        return true;
    }
};

// CTA that owns work unit u when [0,U) is cut into G pieces starting at floor(g*U/G).
__device__ __forceinline__ int unit_owner(long long u, long long U, int G) {
    return static_cast<int>(((u + 1) * G - 1) / U);
}

// Epilogue of the four warps whose (warp & 3) selects the TMEM lane quarter.  `it` walks the same
// segments as the producer and MMA roles; a.kblocks is the number of work units per tile.  CH = tokens
// summed per fix-up pass (4 * CH loads in flight per thread).  chain2_off != 0: the MMA role accumulated
// alternate instructions into a second accumulator that many columns further on; the two are added here.
template <int MT, int CH>
__device__ __forceinline__ void run_epilogue(const LinearArgs& a, SegIter it, uint32_t tmem_base, uint64_t* acc_full,
                                             uint64_t* acc_empty, volatile int* abort_flag, volatile int* s_last, int warp,
                                             int lane, int epi_tid, int g, int G, uint32_t chain2_off = 0,
                                             int acc_stages = 2) {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // output feature within the tile
    int acc = 0;
    uint32_t acc_phase = 0;
    int tile, kb0, kb1;
    while (it.next(tile, kb0, kb1)) {
        const int m_tile = tile / a.n_tiles;
        const int n_tile = tile - m_tile * a.n_tiles;
        const int m_base = m_tile * MT;
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
            if (c0 >= m_cnt || (a.debug & 2)) break;  // uniform across the CTA
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
            } else if (!(a.debug & 4)) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    if (c0 + c < m_cnt) my_ws[(c0 + c) * BLOCK_N + row] = __uint_as_float(r[c]);
                }
            }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(&acc_empty[acc]);
        if (++acc == acc_stages) { acc = 0; acc_phase ^= 1; }

        if (!complete && !(a.debug & (2 | 8))) {
            const long long tile_u0 = static_cast<long long>(tile) * a.kblocks;
            const int g_first = unit_owner(tile_u0, a.total_units, G);
            const int g_last = unit_owner(tile_u0 + a.kblocks - 1, a.total_units, G);
            const int nseg = g_last - g_first + 1;
            __threadfence();
            ptx::named_bar_sync(1, 128);
            if (epi_tid == 0) {
                const int old = atomicAdd(&a.tickets[tile], 1);
                const int last = (old == nseg - 1) ? 1 : 0;
                if (last) a.tickets[tile] = 0;  // ready for the next launch
                *s_last = last;
            }
            ptx::named_bar_sync(1, 128);
            const bool is_last = (*s_last != 0);
            ptx::named_bar_sync(1, 128);  // everyone has read s_last before it can change
            if (is_last && !(a.debug & 16)) {
                __threadfence();
                // sum the pieces in CTA order (deterministic): CH tokens per pass, the coalesced
                // loads of up to four pieces (4 * CH per thread) in flight before the first add
#pragma unroll 1
                for (int c0 = 0; c0 < m_cnt; c0 += CH) {
                    float sum[CH];
#pragma unroll
                    for (int c = 0; c < CH; ++c) sum[c] = 0.f;
#pragma unroll 1
                    for (int g0 = g_first; g0 <= g_last; g0 += 4) {
                        float v[4][CH];
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            const int gg = g0 + s;
                            const float* ws = a.workspace +
                                              (static_cast<size_t>(gg) * 2 + (gg == g_first ? 1 : 0)) * (MT * BLOCK_N) +
                                              static_cast<size_t>(c0) * BLOCK_N + row;
#pragma unroll
                            for (int c = 0; c < CH; ++c) {
                                v[s][c] = (gg <= g_last && c0 + c < m_cnt) ? __ldcg(ws + c * BLOCK_N) : 0.f;
                            }
                        }
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
#pragma unroll
                            for (int c = 0; c < CH; ++c) sum[c] += v[s][c];
                        }
                    }
                    if (n < a.N) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            if (c0 + c < m_cnt) {
                                a.y[static_cast<size_t>(m_base + c0 + c) * a.ldy + n] =
                                    __float2bfloat16(sum[c] + bias_v);
                            }
                        }
                    }
                }
            }
        }
    }
}

}  // namespace gemm
