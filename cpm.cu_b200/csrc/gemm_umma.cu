// Weight-streaming linear layer for the speculative step, sm_100a.
//
//   Y[M,N] = X[M,K] * W[N,K]^T (+ bias)      bf16 in, fp32 accumulate, bf16 out
//
// Replaces the reference's cuBLAS call `linear<T>` (src/model/linear.cuh:8-37)
// for every GEMM of the draft loop (M = 1..16) and of the tree-verify pass
// (M = tree size <= 64), where the op is bound by reading W once from HBM.
//
// Mapping.  The weight tile is the UMMA "A" operand (128 rows of N, full-rate
// M=128 MMA) and the token tile is the "B" operand (UMMA N = MT = 16..256), so
// the accumulator in TMEM is Y^T: lane = output feature, column = token.  Both
// operands are K-major and arrive through TMA with 128-byte swizzle into a
// multi-stage shared-memory ring; one thread issues tcgen05.mma; four epilogue
// warps read TMEM back with tcgen05.ld.  W is held tile-major (one contiguous
// 16 KB block per 128-row tile and 64-column k-block, see linear_weight_elems),
// so a weight fetch is one sequential burst instead of 128 strided segments.
//
// Scheduling.  The (tile, k-block) work units are laid out in one line and cut
// into gridDim.x equal pieces (stream-K), so every SM streams the same number
// of weight bytes whatever N and K are.  A piece that covers only part of a
// tile's K range writes its fp32 partial to a workspace slot and bumps the
// tile's ticket; the last piece to arrive sums the slots in a fixed order
// (deterministic) and writes the bf16 result.  No CTA ever waits on another.
#include <algorithm>

#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

using namespace gemm;

namespace {

constexpr int BLOCK_K = 64;   // bf16 elements per 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BLOCK_N * BLOCK_K * 2;
constexpr int NUM_THREADS = 192;  // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 epilogue

template <int MT>
struct Cfg {
    static constexpr int X_TILE_BYTES = MT * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES;
    static constexpr int STAGES = (MT <= 16) ? 10 : (MT <= 32) ? 9 : (MT <= 64) ? 8 : (MT <= 128) ? 6 : 4;
    static constexpr int TMEM_COLS = (2 * MT < 32) ? 32 : 2 * MT;
    static constexpr int CTRL_BYTES = 256;
    static constexpr int XCH_BYTES = SWIGLU_XCH_BYTES;   // SwiGLU epilogue: gate values on their way to the up warps
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + CTRL_BYTES + XCH_BYTES + 1024;
};

template <int MT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_umma_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const LinearArgs a) {
    using C = Cfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* s_last = abort_flag + 1;
    float* swiglu_xch = (C::XCH_BYTES > 0) ? reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES + C::CTRL_BYTES) : nullptr;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int g = blockIdx.x;
    grid_dep_trigger();

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&acc_full[s], 1);
            ptx::mbar_init(&acc_empty[s], 128);
        }
        *abort_flag = 0;
        *s_last = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&tm_w);
        ptx::prefetch_tensormap(&tm_x);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    SegIter it = make_seg_iter(a, g, G);
    // Weights never depend on the previous kernel: the producer fills the ring with W tiles
    // first, and only then does the CTA wait for the predecessor grid (activations, workspace).
    if (warp != 0) grid_dep_wait();
    const long long pt_dep = kGemmProf ? clock64() : 0;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int tile, kb0, kb1;
            bool ok = true;
            // one k-block of a 128-row weight tile: one contiguous 16 KB block of the tile-major weights (for a SwiGLU
            // launch the tile holds 64 gate rows and the 64 up rows of the same features)
            auto load_w = [&](uint8_t* dst, uint64_t* bar, int kb, int n_tile) {
                ptx::tma_load_2d(dst, &tm_w, bar, 0, (n_tile * a.kblocks + kb) * BLOCK_N);
            };
            // ---- phase 1: W tiles of the first STAGES k-blocks, before the dependency wait
            int pre = 0;
            {
                SegIter pit = it;
                while (pre < C::STAGES && pit.next(tile, kb0, kb1)) {
                    int m_tile, n_tile;
                    tile_to_mn(a, tile, m_tile, n_tile);
                    for (int kb = kb0; kb < kb1 && pre < C::STAGES; ++kb, ++pre) {
                        ptx::mbar_arrive_expect_tx(&full[pre], CPM_EXPERIMENT(a, 1) ? W_TILE_BYTES : C::STAGE_BYTES);
                        load_w(tiles + pre * C::STAGE_BYTES, &full[pre], kb, n_tile);
                    }
                }
            }
            grid_dep_wait();
            // ---- phase 2: the matching X tiles, then the steady-state ring
            int issued = 0;
            while (ok && it.next(tile, kb0, kb1)) {
                int m_tile, n_tile;
                tile_to_mn(a, tile, m_tile, n_tile);
                for (int kb = kb0; kb < kb1; ++kb, ++issued) {
                    uint8_t* dst = tiles + stage * C::STAGE_BYTES;
                    if (issued < pre) {
                        if (!CPM_EXPERIMENT(a, 1)) {
                            ptx::tma_load_2d(dst + W_TILE_BYTES, &tm_x, &full[stage], kb * BLOCK_K, m_tile * MT);
                        }
                    } else {
                        if (!ptx::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                        if (CPM_EXPERIMENT(a, 1)) {
                            ptx::mbar_arrive_expect_tx(&full[stage], W_TILE_BYTES);
                            load_w(dst, &full[stage], kb, n_tile);
                        } else {
                            ptx::mbar_arrive_expect_tx(&full[stage], C::STAGE_BYTES);
                            load_w(dst, &full[stage], kb, n_tile);
                            ptx::tma_load_2d(dst + W_TILE_BYTES, &tm_x, &full[stage], kb * BLOCK_K, m_tile * MT);
                        }
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // give copies already in flight time to land before the CTA retires
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) {}
            }
        }
        else {
            grid_dep_wait();  // the other lanes of the producer warp
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BLOCK_N, MT, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            int tile, kb0, kb1;
            bool ok = true;
            while (ok && it.next(tile, kb0, kb1)) {
                if (!ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * MT;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ptx::mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t wa = ptx::smem_u32(tiles + stage * C::STAGE_BYTES);
                    const uint32_t xa = wa + W_TILE_BYTES;
#pragma unroll
                    for (int j = 0; j < BLOCK_K / UMMA_K; ++j) {
                        const uint64_t da = ptx::umma_desc_sw128(wa + j * UMMA_K * 2, 16, 1024);
                        const uint64_t db = ptx::umma_desc_sw128(xa + j * UMMA_K * 2, 16, 1024);
                        ptx::umma_ss(d_tmem, da, db, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
                    }
                    ptx::umma_commit(&empty[stage]);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                ptx::umma_commit(&acc_full[acc]);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------ epilogue (128 threads)
        run_epilogue<MT, (MT < 32) ? MT : 32>(a, it, tmem_base, acc_full, acc_empty, abort_flag, s_last, warp, lane,
                                              threadIdx.x - 64, g, G, 0, 2, swiglu_xch);
        if (kGemmProf && a.prof != nullptr && threadIdx.x == 64) a.prof[g * 4 + 1] = clock64() - pt_dep;  // epilogue done
    }
    if (kGemmProf && a.prof != nullptr && warp == 1 && lane == 0) a.prof[g * 4 + 0] = clock64() - pt_dep;  // last MMA issued

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error, ERR_GEMM_TIMEOUT);
}

// Split-K inside a thread-block cluster, for launches whose CTAs number CS per output tile: CTA `rank` of
// cluster `n_tile` accumulates k-blocks [rank * kblocks / CS, (rank + 1) * kblocks / CS) of the tile, then the CS partial tiles
// are summed through distributed shared memory instead of the global workspace and its tickets: every CTA
// sends each peer that peer's share of the tokens (ceil(MT / CS), fp32 [source][token][feature] in a buffer next
// to the operand ring), one cluster barrier, and every CTA sums and stores its own tokens in rank order, which
// is the order the workspace path adds its pieces in.  A first barrier only says "every CTA of the cluster has
// started": arrived at on entry, waited for before the first write to a peer.  All other waits are the bounded
// mbarrier waits of the roles; every thread reaches both cluster barriers whatever those waits returned.
// The cluster kernel gives one or two ring stages to a reduction buffer of its own, so that a peer may write its
// partial sums as soon as IT is done, whatever this CTA's ring is doing.
template <int MT, int CS>
struct ClusterCfg {
    static constexpr int STAGE_BYTES = Cfg<MT>::STAGE_BYTES;
    static constexpr int TMEM_COLS = Cfg<MT>::TMEM_COLS;
    static constexpr int TPR = (MT + CS - 1) / CS;                 // tokens summed and stored by each rank
    static constexpr int RED_BYTES = (CS * TPR * BLOCK_N * 4 + 1023) / 1024 * 1024;
    static constexpr int STAGES = Cfg<MT>::STAGES - (RED_BYTES + STAGE_BYTES - 1) / STAGE_BYTES + ((MT >= 64) ? 1 : 0);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RED_BYTES + Cfg<MT>::CTRL_BYTES + 1024;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

template <int MT, int CS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_umma_cluster_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                           const LinearArgs a) {
    using C = ClusterCfg<MT, CS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    float* red = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES);   // peers write here; nothing else does
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + C::RED_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int rank = static_cast<int>(ptx::cluster_ctarank());
    const int n_tile = blockIdx.x / CS;
    const int kb_begin = (a.kblocks * rank) / CS, kb_end = (a.kblocks * (rank + 1)) / CS;
    const int kpc = kb_end - kb_begin;
    grid_dep_trigger();
    ptx::cluster_arrive_relaxed();   // "this CTA runs": waited for just before the first write to a peer

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(acc_full, 1);
        *abort_flag = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&tm_w);
        ptx::prefetch_tensormap(&tm_x);
    }
    if (warp == 1) {
        ptx::tmem_alloc(tmem_slot, C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp != 0) grid_dep_wait();

    float v[MT];   // epilogue threads: this CTA's partial sums of feature `row`, all tokens
#pragma unroll
    for (int c = 0; c < MT; ++c) v[c] = 0.f;
    const int q = warp & 3;
    const int row = q * 32 + lane;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (W tiles first: they need no predecessor)
        if (lane == 0) {
            const int pre = (kpc < C::STAGES) ? kpc : C::STAGES;
            for (int i = 0; i < pre; ++i) {
                ptx::mbar_arrive_expect_tx(&full[i], C::STAGE_BYTES);
                ptx::tma_load_2d(tiles + i * C::STAGE_BYTES, &tm_w, &full[i], 0, (n_tile * a.kblocks + kb_begin + i) * BLOCK_N);
            }
            grid_dep_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int i = 0; i < kpc && ok; ++i) {
                uint8_t* dst = tiles + stage * C::STAGE_BYTES;
                const int kb = kb_begin + i;
                if (i < pre) {
                    ptx::tma_load_2d(dst + W_TILE_BYTES, &tm_x, &full[stage], kb * BLOCK_K, 0);
                } else {
                    if (!ptx::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&full[stage], C::STAGE_BYTES);
                    ptx::tma_load_2d(dst, &tm_w, &full[stage], 0, (n_tile * a.kblocks + kb) * BLOCK_N);
                    ptx::tma_load_2d(dst + W_TILE_BYTES, &tm_x, &full[stage], kb * BLOCK_K, 0);
                }
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                const long long t0 = clock64();   // copies already in flight land before peers reuse the ring
                while (clock64() - t0 < 2000000LL) {}
            }
        } else {
            grid_dep_wait();
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BLOCK_N, MT, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!ptx::mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t wa = ptx::smem_u32(tiles + stage * C::STAGE_BYTES);
                const uint32_t xa = wa + W_TILE_BYTES;
#pragma unroll
                for (int j = 0; j < BLOCK_K / UMMA_K; ++j) {
                    const uint64_t da = ptx::umma_desc_sw128(wa + j * UMMA_K * 2, 16, 1024);
                    const uint64_t db = ptx::umma_desc_sw128(xa + j * UMMA_K * 2, 16, 1024);
                    ptx::umma_ss(tmem_base, da, db, idesc, (kb > kb_begin || j > 0) ? 1u : 0u);
                }
                ptx::umma_commit(&empty[stage]);
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) ptx::umma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------ epilogue, part 1: partial sums out of tensor memory
        if (ptx::mbar_wait_warp(acc_full, 0, abort_flag)) {
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
            for (int c0 = 0; c0 < MT; c0 += 16) {
                uint32_t r[16];
                ptx::tmem_ld16(t_addr + c0, r);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c0 + c] = __uint_as_float(r[c]);
            }
            ptx::tc_fence_before();
        }
    }
    __syncwarp();
    ptx::cluster_wait();   // every CTA of the cluster has started (arrivals at entry): its shared memory may be written

    cluster_reduce_store<MT, CS>(a, v, red, rank, n_tile, warp >= 2, row);

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error, ERR_GEMM_TIMEOUT);
}

template <int MT, int CS>
void configure_cluster_kernel() {
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(linear_umma_cluster_kernel<MT, CS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ClusterCfg<MT, CS>::SMEM_BYTES));
        configured = true;
    }
}

template <int MT, int CS>
int max_active_clusters() {
    static int cached = -1;
    if (cached < 0) {
        configure_cluster_kernel<MT, CS>();
        cached = ::max_active_clusters(linear_umma_cluster_kernel<MT, CS>, dim3(NUM_THREADS), ClusterCfg<MT, CS>::SMEM_BYTES, CS);
    }
    return cached;
}

template <int MT, int CS>
void launch_cluster(const LinearPlan& p, const LinearArgs& args, cudaStream_t stream) {
    configure_cluster_kernel<MT, CS>();
    launch_kernel_cluster(linear_umma_cluster_kernel<MT, CS>, dim3(p.grid), dim3(NUM_THREADS), ClusterCfg<MT, CS>::SMEM_BYTES, stream,
                          CS, p.tm_w, p.tm_x, args);
}

int cluster_capacity(int mt, int cs) {
    if (cs == 2) return mt == 16 ? max_active_clusters<16, 2>() : mt == 32 ? max_active_clusters<32, 2>() : mt == 64 ? max_active_clusters<64, 2>() : 0;
    if (cs == 3) return mt == 16 ? max_active_clusters<16, 3>() : mt == 32 ? max_active_clusters<32, 3>() : mt == 64 ? max_active_clusters<64, 3>() : 0;
    if (cs == 4) return mt == 16 ? max_active_clusters<16, 4>() : mt == 32 ? max_active_clusters<32, 4>() : mt == 64 ? max_active_clusters<64, 4>() : 0;
    return 0;
}

bool launch_cluster_any(const LinearPlan& p, const LinearArgs& a, cudaStream_t s) {
    switch (p.mt * 8 + p.cluster) {
        case 16 * 8 + 2: launch_cluster<16, 2>(p, a, s); return true;
        case 16 * 8 + 3: launch_cluster<16, 3>(p, a, s); return true;
        case 16 * 8 + 4: launch_cluster<16, 4>(p, a, s); return true;
        case 32 * 8 + 3: launch_cluster<32, 3>(p, a, s); return true;
        case 64 * 8 + 3: launch_cluster<64, 3>(p, a, s); return true;
        case 32 * 8 + 2: launch_cluster<32, 2>(p, a, s); return true;
        case 32 * 8 + 4: launch_cluster<32, 4>(p, a, s); return true;
        case 64 * 8 + 2: launch_cluster<64, 2>(p, a, s); return true;
        case 64 * 8 + 4: launch_cluster<64, 4>(p, a, s); return true;
        default: return false;
    }
}

template <int MT>
void launch_mt(const LinearPlan& p, const LinearArgs& args, cudaStream_t stream) {
    using C = Cfg<MT>;
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(linear_umma_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C::SMEM_BYTES));
        configured = true;
    }
    launch_kernel(linear_umma_kernel<MT>, dim3(p.grid), dim3(NUM_THREADS), C::SMEM_BYTES, stream, p.tm_w, p.tm_x, args);
}

}  // namespace

int linear_pick_mt(int M) {
    if (M <= 16) return 16;
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    if (M <= 128) return 128;
    return 256;
}

size_t linear_workspace_bytes(int mt, int grid) {
    return static_cast<size_t>(grid) * 2 * mt * BLOCK_N * sizeof(float);
}

// Number of CTAs for a decode-shaped launch (one token tile).  Every CTA gets the same
// share of the (tile, k-block) line; the model below trades streaming time (per-SM and
// HBM limits as measured on B200) against the cost of split-K fix-ups, which vanish when
// the shares line up with tile boundaries.
static int pick_grid(int n_tiles, int kblocks, int m_valid, int limit) {
    const long long units = static_cast<long long>(n_tiles) * kblocks;
    const double tile_bytes = 16384.0;        // one W k-block
    const double sm_rate = 55e9, hbm_rate = 6.3e12;
    double best_t = 1e30;
    int best_g = 1;
    for (int g = 1; g <= limit && g <= units; ++g) {
        const long long per = (units + g - 1) / g;
        const double rate = std::min(sm_rate, hbm_rate / g);
        double t = per * tile_bytes / rate;
        const bool aligned_whole = (units % g == 0) && ((units / g) % kblocks == 0);
        if (!aligned_whole) {
            const double share = static_cast<double>(units) / g;
            int nseg;
            if (units % g == 0 && kblocks % (units / g) == 0) nseg = static_cast<int>(kblocks / (units / g));
            else nseg = static_cast<int>(kblocks / share) + 2;
            t += 4.5e-6 + 1.0e-6 * ((m_valid + 31) / 32) * ((nseg + 3) / 4);
        }
        if (t < best_t - 1e-9) {
            best_t = t;
            best_g = g;
        }
    }
    return best_g;
}

// Tensor map of tile-major weights (linear_weight_elems): every (128-row tile, 64-column k-block) is one box of 128
// consecutive 128-byte rows.
static CUtensorMap make_weight_tmap(const bf16* w, int N, int K) {
    return make_tmap_2d(w, BLOCK_K, static_cast<uint64_t>(ceil_div(N, BLOCK_N)) * (K / BLOCK_K) * BLOCK_N, BLOCK_K * 2, BLOCK_K,
                        BLOCK_N);
}

// CTAs of a launch before the cluster and wave decisions: at least four k-blocks each.
static long long base_grid(int n_tiles, int m_tiles, int kblocks, int M, int grid_limit) {
    const long long units = static_cast<long long>(n_tiles) * m_tiles * kblocks;
    long long grid = units / 4;
    if (grid < 1) grid = 1;
    if (grid > grid_limit) grid = grid_limit;
    if (m_tiles == 1 && grid_limit >= 64) grid = pick_grid(n_tiles, kblocks, M, static_cast<int>(grid));
    return grid;
}

// Host-side walk of the work distribution make_linear_plan + launch_linear give a launch (without the cluster
// variant, which cuts every tile into equal pieces): for every CTA its segments as six ints
// (cta, tile, token tile, feature tile, first k-block, end k-block), in the order the CTA runs them.  The same
// iterator and raster functions the kernels use, compiled for the host.  Returns the number of segments, or -1 when
// `cap` segments do not hold them.
int linear_schedule_dump(int M, int N, int K, int grid_limit, int32_t* out, int cap) {
    LinearArgs a = {};
    const int mt = linear_pick_mt(M);
    a.M = M; a.N = N; a.K = K;
    a.n_tiles = ceil_div(N, BLOCK_N);
    a.m_tiles = ceil_div(M, mt);
    a.kblocks = K / BLOCK_K;
    const int grid = static_cast<int>(base_grid(a.n_tiles, a.m_tiles, a.kblocks, M, grid_limit));
    a.wave_tiles = 0;
    a.tail_grid = 0;
    if (a.m_tiles > 1) plan_waves(static_cast<long long>(a.n_tiles) * a.m_tiles, a.kblocks, grid, a.wave_tiles, a.tail_grid);
    a.total_units = (static_cast<long long>(a.n_tiles) * a.m_tiles - a.wave_tiles) * a.kblocks;
    a.band = raster_band(mt, K);
    int n = 0;
    for (int g = 0; g < grid; ++g) {
        SegIter it = make_seg_iter(a, g, grid);
        int tile, kb0, kb1;
        while (it.next(tile, kb0, kb1)) {
            if (n >= cap) return -1;
            int m_tile, n_tile;
            tile_to_mn(a, tile, m_tile, n_tile);
            int32_t* o = out + static_cast<size_t>(n) * 6;
            o[0] = g; o[1] = tile; o[2] = m_tile; o[3] = n_tile; o[4] = kb0; o[5] = kb1;
            ++n;
        }
    }
    return n;
}

LinearPlan make_linear_plan(const bf16* x, int x_rows, const bf16* w, int M, int N, int K, bf16* y, int ldy,
                            const bf16* bias, float* workspace, int* tickets, int grid_limit) {
    CPM_REQUIRE(M >= 1 && N >= 1 && K >= BLOCK_K, "linear: empty problem");
    CPM_REQUIRE(K % BLOCK_K == 0, "linear: K must be a multiple of 64");
    CPM_REQUIRE(x_rows >= 1, "linear: x_rows must be positive");
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                "linear: operands must be 16-byte aligned");
    LinearPlan p;
    p.M = M; p.N = N; p.K = K;
    p.mt = linear_pick_mt(M);
    p.y = y; p.ldy = ldy; p.bias = bias;
    p.workspace = workspace; p.tickets = tickets;
    const int n_tiles = ceil_div(N, BLOCK_N), m_tiles = ceil_div(M, p.mt), kblocks = K / BLOCK_K;
    const long long units = static_cast<long long>(n_tiles) * m_tiles * kblocks;
    long long grid = base_grid(n_tiles, m_tiles, kblocks, M, grid_limit);
    {
        static const char* forced = tuning_env("CPMCU_LINEAR_GRID");  // bench only: sweep the grid size
        if (forced && atoi(forced) >= 1 && atoi(forced) <= grid_limit && atoi(forced) <= units) grid = atoi(forced);
        // bench only: per-shape grids, "MxNxK:grid,MxNxK:grid,..."
        static const char* per_shape = tuning_env("CPMCU_LINEAR_GRIDS");
        if (per_shape) {
            char key[64];
            snprintf(key, sizeof(key), "%dx%dx%d:", M, N, K);
            const char* hit = strstr(per_shape, key);
            if (hit) {
                const int gsz = atoi(hit + strlen(key));
                if (gsz >= 1 && gsz <= grid_limit && gsz <= units) grid = gsz;
            }
        }
    }
    p.grid = static_cast<int>(grid);
    if (m_tiles > 1) {
        static const bool flat = tuning_env("CPMCU_LINEAR_NO_WAVES") != nullptr;   // bench only: plain stream-K
        if (!flat) plan_waves(static_cast<long long>(n_tiles) * m_tiles, kblocks, p.grid, p.wave_tiles, p.tail_grid);
    }
    // CS CTAs per tile with equal k ranges: sum the pieces inside a cluster when the device runs all clusters at once
    p.cluster = 0;
    {
        static const bool off = tuning_env("CPMCU_LINEAR_NO_CLUSTER") != nullptr;
        // the grid picker's pieces per tile first; when the device cannot hold that many clusters at once
        // (its SMs come in groups that need not be multiples of the cluster size), fewer and longer pieces
        int cs = (m_tiles == 1 && grid % n_tiles == 0) ? static_cast<int>(grid / n_tiles) : 0;
        if (!off && p.mt <= 64 && cs >= 2 && cs <= 4) {
            for (; cs >= 2; --cs) {
                if (kblocks >= 4 * cs && cluster_capacity(p.mt, cs) >= n_tiles) {
                    p.cluster = cs;
                    p.grid = n_tiles * cs;
                    break;
                }
            }
        }
        static const bool verbose = tuning_env("CPMCU_LINEAR_VERBOSE") != nullptr;   // bench only
        if (verbose) {
            fprintf(stderr, "linear plan M=%d N=%d K=%d: grid %d, %d tiles, cluster %d (device runs %d / %d / %d clusters of 2 / 3 / 4)\n",
                    M, N, K, p.grid, n_tiles, p.cluster, cluster_capacity(p.mt <= 64 ? p.mt : 64, 2),
                    cluster_capacity(p.mt <= 64 ? p.mt : 64, 3), cluster_capacity(p.mt <= 64 ? p.mt : 64, 4));
        }
    }
    p.tm_w = make_weight_tmap(w, N, K);
    p.tm_x = make_tmap_2d(x, K, x_rows, static_cast<uint64_t>(K) * 2, BLOCK_K, p.mt);
    return p;
}

// Grid of a SwiGLU launch: its tiles (64 features x one token tile) are never cut along K.  One token tile: the
// largest grid that gives every CTA the same number of tiles; more: one CTA per SM, tiles in waves.
static int swiglu_grid(int n_tiles, int m_tiles, int grid_limit) {
    const long long tiles = static_cast<long long>(n_tiles) * m_tiles;
    if (tiles <= grid_limit) return static_cast<int>(tiles);
    if (m_tiles > 1) return grid_limit;
    int g = grid_limit;
    while (n_tiles % g != 0) --g;
    return g;
}

// Whether the whole-tile schedule keeps the SMs about as busy as the stream-K schedule of the unfused GEMM would
// (launches smaller than the grid limit always qualify: they are a single wave either way).
bool linear_swiglu_fits(int M, int inter, int grid_limit) {
    if (inter < 64 || inter % 64 != 0) return false;
    const int n_tiles = inter / 64, m_tiles = ceil_div(M, linear_pick_mt(M));
    const long long tiles = static_cast<long long>(n_tiles) * m_tiles;
    if (tiles <= grid_limit) return true;
    const int g = swiglu_grid(n_tiles, m_tiles, grid_limit);
    const long long waves = (tiles + g - 1) / g;
    return static_cast<double>(tiles) >= 0.85 * static_cast<double>(waves) * grid_limit;
}

// act[M, inter] = silu(X Wg^T) * (X Wu^T); w holds the two projections as tile-major tiles of 64 gate rows + the 64 up
// rows of the same features (retile_weight_rows modes 1 and 2); both projections are rounded to bf16 before the product
// like the unfused pair (GEMM, then silu_gate_kernel).  Whole tiles only.
LinearPlan make_linear_swiglu_plan(const bf16* x, int x_rows, const bf16* w, int M, int inter, int K, bf16* act, int ld,
                                   int grid_limit) {
    CPM_REQUIRE(M >= 1 && inter >= 64 && inter % 64 == 0, "linear: SwiGLU width must be a multiple of 64");
    CPM_REQUIRE(K >= BLOCK_K && K % BLOCK_K == 0, "linear: K must be a multiple of 64");
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                "linear: operands must be 16-byte aligned");
    LinearPlan p;
    p.M = M; p.N = inter; p.K = K;
    p.mt = linear_pick_mt(M);
    p.y = act; p.ldy = ld; p.bias = nullptr;
    p.swiglu = 1;
    const long long tiles = static_cast<long long>(inter / 64) * ceil_div(M, p.mt);
    const int m_tiles = ceil_div(M, p.mt);
    p.grid = swiglu_grid(inter / 64, m_tiles, grid_limit);
    // No tile is cut, nothing goes through the workspace.  Several token tiles: whole tiles in waves.  One token tile:
    // the grid divides the tiles, and every CTA takes consecutive ones (one contiguous run of gate rows and one of up
    // rows per CTA instead of two scattered 64-row slabs per tile).
    p.wave_tiles = (m_tiles > 1) ? static_cast<int>(tiles) : 0;
    p.tail_grid = (m_tiles > 1) ? 1 : p.grid;
    p.tm_w = make_weight_tmap(w, 2 * inter, K);
    p.tm_x = make_tmap_2d(x, K, x_rows, static_cast<uint64_t>(K) * 2, BLOCK_K, p.mt);
    return p;
}

void launch_linear(const LinearPlan& p, cudaStream_t stream) {
    if (p.wq != nullptr) {  // 4-bit weights
        launch_linear_w4(p, stream);
        return;
    }
    ProfileScope prof(KC_LINEAR, stream);
    LinearArgs a;
    a.M = p.M; a.N = p.N; a.K = p.K;
    a.n_tiles = ceil_div(p.N, BLOCK_N);
    a.m_tiles = ceil_div(p.M, p.mt);
    a.kblocks = p.K / BLOCK_K;
    a.wave_tiles = p.wave_tiles;
    a.tail_grid = p.tail_grid;
    a.swiglu = p.swiglu;
    a.band = raster_band(p.mt, p.K);
    if (p.swiglu) {   // N = output features; a tile covers 64 of them (gate + up rows)
        a.n_tiles = ceil_div(p.N, 64);
        CPM_REQUIRE(p.cluster == 0 && (p.wave_tiles == a.n_tiles * a.m_tiles ||
                                       (a.m_tiles == 1 && p.wave_tiles == 0 && a.n_tiles % p.grid == 0)),
                    "linear: the SwiGLU epilogue needs whole tiles");
    }
    a.total_units = (static_cast<long long>(a.n_tiles) * a.m_tiles - a.wave_tiles) * a.kblocks;
    a.y = p.y; a.ldy = p.ldy; a.bias = p.bias;
    a.workspace = p.workspace; a.tickets = p.tickets;
    a.error = runtime().d_error;
    a.debug = p.debug;
    {
        static const char* dbg = tuning_env("CPMCU_LINEAR_DEBUG_ALL");
        if (dbg) a.debug = atoi(dbg);
    }
    a.prof = nullptr;
    if (kGemmProf) {
        static long long* buf = nullptr;
        if (buf == nullptr) {
            CUDA_CHECK(cudaMalloc(&buf, 256 * 4 * sizeof(long long)));
            CUDA_CHECK(cudaMemset(buf, 0, 256 * 4 * sizeof(long long)));
        }
        a.prof = buf;
        static int calls = 0;
        if (++calls % 40 == 0) {
            std::vector<long long> h(p.grid * 4);
            CUDA_CHECK(cudaMemcpy(h.data(), buf, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
            long long lo[2] = {h[0], h[1]}, hi[2] = {h[0], h[1]}, sum[2] = {0, 0};
            for (int c = 0; c < p.grid; ++c) {
                for (int k = 0; k < 2; ++k) {
                    lo[k] = std::min(lo[k], h[c * 4 + k]); hi[k] = std::max(hi[k], h[c * 4 + k]); sum[k] += h[c * 4 + k];
                }
            }
            fprintf(stderr, "gemm prof (previous launch, %d CTAs, cycles after the dependency wait): last MMA issued min %lld "
                            "mean %lld max %lld; epilogue done min %lld mean %lld max %lld\n",
                    p.grid, lo[0], sum[0] / p.grid, hi[0], lo[1], sum[1] / p.grid, hi[1]);
        }
    }
    if (p.cluster != 0 && launch_cluster_any(p, a, stream)) return;
    switch (p.mt) {
        case 16: launch_mt<16>(p, a, stream); break;
        case 32: launch_mt<32>(p, a, stream); break;
        case 64: launch_mt<64>(p, a, stream); break;
        case 128: launch_mt<128>(p, a, stream); break;
        case 256: launch_mt<256>(p, a, stream); break;
        default: throw std::invalid_argument("cpmcu_b200: bad token tile");
    }
}
