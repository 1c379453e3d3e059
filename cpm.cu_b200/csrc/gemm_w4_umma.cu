// W4A16 weight-streaming linear layer, sm_100a:  Y[M,N] = X[M,K] * dequant(Wq)[N,K]^T.
//
// Replaces the reference's vendored Marlin kernel (`gptq_marlin_gemm`,
// src/qgemm/gptq_marlin/gptq_marlin.cu:2093-2138; `Marlin<>` :457-1644) for the target's
// linears when they are GPTQ int4 (symmetric, w = (q - 8) * scale, group size 128).  The
// arithmetic is the reference's: the 4-bit value becomes an exact bf16, the scale multiply
// rounds once to bf16, products accumulate in fp32.
//
// Same mapping as the bf16 kernel (weights = UMMA A operand with M = 128, tokens = B operand,
// Y^T in TMEM, stream-K with ticketed fix-up), with one more stage in the pipeline:
//
//   W producer   one bulk copy per stage: the packed nibbles of a 128-row x 256-k super-block (16 KB)
//                and its two rows of scales are one contiguous block in HBM (re-tiled at load
//                time); ring of W stages, filled before the programmatic-dependency wait
//                (weights never depend on the previous kernel)
//   dequant      8 warps: 32 B of nibbles -> 64 bf16 per thread with the 0x4300 magic-number
//                trick (128 + q is exact in bf16), (x - 136) * scale, stored with tcgen05.st into
//                a ring of A slots in TENSOR MEMORY (row = lane, two bf16 per column): the
//                dequantised weights never touch shared memory, whose bandwidth is what bounds
//                a small-N UMMA
//   X producer   TMA: token tiles per 64-k block, one per slot
//   MMA          two issuer warps, one per parity of the k-block index, each accumulating into its own
//                accumulator (the epilogue adds the two): the single-thread issue loop (waits,
//                descriptors, four tcgen05.mma, commit) costs more cycles per k-block than the
//                tensor pipe needs, so two of them interleave.  A from tensor memory, B (tokens)
//                from shared memory; ONE commit per k-block frees the A slot and the token tile
//   epilogue     shared with the bf16 kernel
//
// HBM sees 0.5 byte per weight (+ 1/64 for scales).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

using namespace gemm;

namespace {

constexpr int BLOCK_K = 64;          // k per MMA block (128-byte swizzle row of bf16 tokens)
constexpr int SUPER_K = 256;         // k per W stage and per stream-K unit
constexpr int KB_PER_UNIT = SUPER_K / BLOCK_K;
constexpr int UMMA_K = 16;
constexpr int WQ_BYTES = BLOCK_N * SUPER_K / 2;    // 16 KB of nibbles
constexpr int WS_BYTES = 2 * BLOCK_N * 2;          // two scale rows (groups of 128 k) x 128 features
constexpr int W_STAGE_BYTES = WQ_BYTES + WS_BYTES; // one block of the streaming layout
constexpr int A_COLS = BLOCK_K / 2;                // 32 columns: 64 bf16 per lane
constexpr int DEQ_WARPS = 8;
// warp 0: W producer, warp 1: MMA (even k-blocks) + TMEM, warps 2-5: epilogue, warps 6-13: dequant,
// warp 14: X producer, warp 15: MMA (odd k-blocks)
constexpr int NUM_THREADS = (6 + DEQ_WARPS + 2) * 32;
constexpr int MAX_MT = 128;                        // 2 chains x 128 + 8 x 32 A columns = 512

// CS > 0 (cluster split-K): a reduction buffer of CS * ceil(MT / CS) tokens x 128 features fp32 that peers write,
// paid for at MT = 64 with one weight stage.
template <int MT, int CS = 0>
struct Cfg {
    static constexpr int X_BYTES = MT * BLOCK_K * 2;
    static constexpr int RED_BYTES = (CS > 0) ? (CS * ((MT + (CS > 0 ? CS : 1) - 1) / (CS > 0 ? CS : 1)) * BLOCK_N * 4 + 1023) / 1024 * 1024 : 0;
    static constexpr int W_STAGES = (MT <= 32) ? 9 : (MT <= 64) ? ((CS > 0) ? 5 : 6) : 5;
    // ring of (A slot in TMEM, token tile in smem) pairs.  A slot comes back only after the MMA that read it
    // has completed and three barrier hand-offs (about a microsecond), so the ring depth, not any role's
    // work, sets the k-block rate: tensor memory goes to slots rather than to a second accumulator stage
    static constexpr int SLOTS = (MT <= 64) ? 12 : 8;
    static constexpr int GROUPS = SLOTS / 4;  // four slots = the k-blocks of one unit, filled by one token TMA
    static constexpr int ACC_STAGES = 1;
    static constexpr int ACC_COLS = ACC_STAGES * MT;       // per chain
    static constexpr int A_COL0 = (ACC_COLS < 32) ? 32 : ACC_COLS;
    static constexpr int ACC2_OFF = A_COL0 + SLOTS * (BLOCK_K / 2);  // column offset of chain 1 from chain 0
    static constexpr int TMEM_COLS = 512;
    static constexpr int OFF_W = 0;
    static constexpr int OFF_X = (OFF_W + W_STAGES * W_STAGE_BYTES + 1023) / 1024 * 1024;
    static constexpr int OFF_RED = OFF_X + SLOTS * X_BYTES;
    static constexpr int OFF_CTRL = OFF_RED + RED_BYTES;
    static constexpr int SMEM_BYTES = OFF_CTRL + 512 + 1024;
    static_assert(ACC2_OFF + ACC_COLS <= TMEM_COLS, "tensor memory budget");
    static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct W4Args {
    LinearArgs lin;
    const uint8_t* blocks;  // [n_tiles][K/256][W_STAGE_BYTES]
    long long* prof;        // bench only: 16 clock counters per CTA, or null
};

// Role-level clock counters, compiled in only with -DCPMCU_W4_PROFILE=1 (role totals) or =2 (also the
// waits inside the loops, which lengthens the MMA issue loop).
#ifdef CPMCU_W4_PROFILE
constexpr int kProfLevel = CPMCU_W4_PROFILE;
#else
constexpr int kProfLevel = 0;
#endif
constexpr bool kProf = kProfLevel > 0;
struct Stopwatch {
    __device__ explicit Stopwatch(const void*) {}
    __device__ long long now() const { return kProfLevel > 1 ? clock64() : 0; }
    __device__ long long total() const { return kProf ? clock64() : 0; }
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return r;
}

// CS > 0: the launch runs as clusters of CS CTAs, cluster = output tile, rank = k-piece of it, and the pieces are
// summed through distributed shared memory (cluster_reduce_store) instead of the workspace and its tickets.
template <int MT, int CS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_w4_umma_kernel(const __grid_constant__ CUtensorMap tm_x, const W4Args wa) {
    using C = Cfg<MT, CS>;
    const LinearArgs& a = wa.lin;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_CTRL);
    uint64_t* w_full = bars;                       // [W_STAGES]
    uint64_t* w_empty = w_full + C::W_STAGES;      // [W_STAGES]  one arrival per dequant warp
    uint64_t* a_full = w_empty + C::W_STAGES;      // [GROUPS]    one arrival per dequant warp
    uint64_t* x_full = a_full + C::GROUPS;         // [GROUPS]
    uint64_t* grp_empty = x_full + C::GROUPS;      // [GROUPS]    one commit per MMA issuer: A slots and token tiles free
    uint64_t* acc_full = grp_empty + C::GROUPS;    // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* s_last = abort_flag + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int g = blockIdx.x;
    grid_dep_trigger();
    if constexpr (CS > 0) ptx::cluster_arrive_relaxed();   // "this CTA runs": waited for before the first write to a peer

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::W_STAGES; ++s) {
            ptx::mbar_init(&w_full[s], 1);
            ptx::mbar_init(&w_empty[s], DEQ_WARPS);
        }
        for (int s = 0; s < C::GROUPS; ++s) {
            ptx::mbar_init(&a_full[s], DEQ_WARPS);
            ptx::mbar_init(&x_full[s], 1);
            ptx::mbar_init(&grp_empty[s], 2);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&acc_full[s], 2);  // both MMA issuers commit
            ptx::mbar_init(&acc_empty[s], 128);
        }
        *abort_flag = 0;
        *s_last = 0;
        ptx::mbar_fence_init();
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

    // work units are 256-k super-blocks: a.kblocks = K / 256 units per tile
    SegIter it = make_seg_iter(a, g, G);
    const int c_rank = (CS > 0) ? static_cast<int>(ptx::cluster_ctarank()) : 0;
    const int c_tile = (CS > 0) ? g / CS : 0;
    if (CS > 0) {
        it.u = static_cast<long long>(c_tile) * a.kblocks + (a.kblocks * c_rank) / CS;
        it.u_end = static_cast<long long>(c_tile) * a.kblocks + (a.kblocks * (c_rank + 1)) / CS;
    }
    constexpr int VN = (CS > 0) ? MT : 1;
    float v[VN];   // cluster mode, epilogue threads: this CTA's partial sums of one feature, all tokens
#pragma unroll
    for (int c = 0; c < VN; ++c) v[c] = 0.f;

    if (warp == 0) {
        // ------------------------------------------------ W producer (weights only: runs ahead of the dependency wait)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int tile, u0, u1;
            bool ok = true;
            while (ok && it.next(tile, u0, u1)) {
                int m_tile, n_tile;
                tile_to_mn(a, tile, m_tile, n_tile);
                for (int u = u0; u < u1; ++u) {
                    if (!ptx::mbar_wait(&w_empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    if (CPM_EXPERIMENT(a, 64)) {  // timing experiment: no weight traffic
                        ptx::mbar_arrive(&w_full[stage]);
                    } else {
                        ptx::mbar_arrive_expect_tx(&w_full[stage], W_STAGE_BYTES);
                        ptx::bulk_load(smem + C::OFF_W + stage * W_STAGE_BYTES,
                                       wa.blocks + (static_cast<size_t>(n_tile) * a.kblocks + u) * W_STAGE_BYTES,
                                       W_STAGE_BYTES, &w_full[stage]);
                    }
                    if (++stage == C::W_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) {}
            }
        }
        grid_dep_wait();
    } else if (warp == 14) {
        // ------------------------------------------------ X producer: one 3-D TMA per unit fills a group of four slots
        grid_dep_wait();
        {
            int grp = 0;
            uint32_t phase = 0;
            int tile, u0, u1;
            bool ok = true;
            while (ok && it.next(tile, u0, u1)) {
                int m_tile, n_tile;
                tile_to_mn(a, tile, m_tile, n_tile);
                for (int u = u0; u < u1; ++u) {
                    if (!ptx::mbar_wait_warp(&grp_empty[grp], phase ^ 1, abort_flag)) { ok = false; break; }
                    if (ptx::elect_one()) {
                        if (CPM_EXPERIMENT(a, 128)) {  // timing experiment: no token traffic
                            ptx::mbar_arrive(&x_full[grp]);
                        } else {
                            ptx::mbar_arrive_expect_tx(&x_full[grp], KB_PER_UNIT * C::X_BYTES);
                            ptx::tma_load_3d(smem + C::OFF_X + grp * KB_PER_UNIT * C::X_BYTES, &tm_x, &x_full[grp], 0,
                                             m_tile * MT, u * KB_PER_UNIT);
                        }
                    }
                    __syncwarp();
                    if (++grp == C::GROUPS) { grp = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1 || warp == 15) {
        // ------------------------------------------------ MMA issuers: chain 0 takes even k-blocks, chain 1 odd ones
        // The whole warp runs the loop with warp-uniform control flow and one elected lane issues: the
        // operands of tcgen05.mma live in uniform registers, and per-thread values would be moved there
        // one by one in front of every instruction.
        grid_dep_wait();
        {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BLOCK_N, MT, 0, 0);
            const int chain = (warp == 1) ? 0 : 1;
            int grp = 0;
            uint32_t gph = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            int tile, u0, u1;
            bool ok = true;
            Stopwatch sw(wa.prof);
            long long t_acc = 0, t_a = 0, t_x = 0, t_issue = 0;
            const long long t_begin = sw.total();
            while (ok && it.next(tile, u0, u1)) {
                long long c0 = sw.now();
                if (!ptx::mbar_wait_warp(&acc_empty[acc], acc_phase ^ 1, abort_flag)) break;
                t_acc += sw.now() - c0;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + chain * C::ACC2_OFF + acc * MT;
                uint32_t accumulate = 0;
                for (int u = u0; u < u1; ++u) {
                    c0 = sw.now();
                    if (!ptx::mbar_wait_warp(&x_full[grp], gph, abort_flag)) { ok = false; break; }
                    const long long c1 = sw.now();
                    if (!ptx::mbar_wait_warp(&a_full[grp], gph, abort_flag)) { ok = false; break; }
                    const long long c2 = sw.now();
                    t_x += c1 - c0;
                    t_a += c2 - c1;
                    ptx::tc_fence_after();
                    if (ptx::elect_one()) {
                        if (!CPM_EXPERIMENT(a, 256)) {
#pragma unroll
                            for (int h = 0; h < KB_PER_UNIT / 2; ++h) {
                                const int slot = grp * KB_PER_UNIT + 2 * h + chain;
                                const uint32_t a_tmem = tmem_base + C::A_COL0 + slot * A_COLS;
                                const uint64_t db =
                                    ptx::umma_desc_sw128(ptx::smem_u32(smem + C::OFF_X + slot * C::X_BYTES), 16, 1024);
#pragma unroll
                                for (int j = 0; j < BLOCK_K / UMMA_K; ++j) {
                                    // + 2 in the descriptor's address field = 32 bytes = 16 k
                                    ptx::umma_ts(d_tmem, a_tmem + j * (UMMA_K / 2), db + 2 * j, idesc,
                                                 (h + j > 0) ? 1u : accumulate);
                                }
                            }
                        }
                        ptx::umma_commit(&grp_empty[grp]);
                    }
                    __syncwarp();
                    accumulate = 1;
                    t_issue += sw.now() - c2;
                    if (++grp == C::GROUPS) { grp = 0; gph ^= 1; }
                }
                if (!ok) break;
                if (ptx::elect_one()) ptx::umma_commit(&acc_full[acc]);
                __syncwarp();
                if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
            if (kProf && wa.prof && lane == 0) {
                long long* pr = wa.prof + g * 16 + chain * 9;
                pr[0] = sw.total() - t_begin; pr[1] = t_acc; pr[2] = t_a; pr[3] = t_x; pr[4] = t_issue;
            }
        }
    } else if (warp >= 6 && warp < 6 + DEQ_WARPS) {
        // ------------------------------------------------ dequant warps: nibbles -> bf16 A slots in tensor memory
        // A warp may only touch the TMEM lanes of its quarter (warp % 4): two warps per quarter, which take
        // alternate 64-k blocks; the thread's row is its lane and it converts the row's 64 weights.
        const int quarter = warp & 3, parity = (warp - 6) >> 2;
        const int row = quarter * 32 + lane;
        int ws = 0, grp = 0;
        uint32_t wph = 0, gph = 0;
        int tile, u0, u1;
        bool ok = true;
        const __nv_bfloat162 bias2 = __floats2bfloat162_rn(136.f, 136.f);  // 128 (magic) + 8 (zero point)
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + C::A_COL0;
        Stopwatch sw(wa.prof);
        long long t_w = 0, t_slot = 0, t_st = 0;
        (void)t_st;
        const long long t_begin = sw.total();
        while (ok && it.next(tile, u0, u1)) {
            for (int u = u0; u < u1 && ok; ++u) {
                // waits are made warp-uniform: the tensor-memory stores below are warp-collective
                long long c0 = sw.now();
                if (!ptx::mbar_wait_warp(&w_full[ws], wph, abort_flag)) { ok = false; break; }
                t_w += sw.now() - c0;
                const uint8_t* wst = smem + C::OFF_W + ws * W_STAGE_BYTES;
                const bf16* sc = reinterpret_cast<const bf16*>(wst + WQ_BYTES);
                if (CPM_EXPERIMENT(a, 32)) {  // timing experiment: barriers only
                    if (!ptx::mbar_wait_warp(&grp_empty[grp], gph ^ 1, abort_flag)) { ok = false; break; }
                } else {
#pragma unroll
                    for (int jj = 0; jj < KB_PER_UNIT / 2; ++jj) {
                        const int j = jj * 2 + parity;  // this warp's k-block of the unit: k = 64 j .. 64 j + 63
                        const uint4 lo = *reinterpret_cast<const uint4*>(wst + j * 4096 + row * 16);
                        const uint4 hi = *reinterpret_cast<const uint4*>(wst + j * 4096 + 2048 + row * 16);
                        const bf16 s1 = sc[jj * BLOCK_N + row];  // group of 128 k = blocks 2 jj, 2 jj + 1
                        const __nv_bfloat162 s2 = __halves2bfloat162(s1, s1);
                        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                        uint32_t o[32];
#pragma unroll
                        for (int w = 0; w < 8; ++w) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t bits = lop3_and_or(words[w] >> (4 * i), 0x000f000fu, 0x43004300u);
                                __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&bits);  // (128 + q_lo, 128 + q_hi)
                                v = __hmul2(__hsub2(v, bias2), s2);                                  // exact subtract, one rounding
                                o[w * 4 + i] = *reinterpret_cast<uint32_t*>(&v);
                            }
                        }
                        if (jj == 0) {  // the group's A slots are free once both issuers' MMAs on them have completed
                            c0 = sw.now();
                            if (!ptx::mbar_wait_warp(&grp_empty[grp], gph ^ 1, abort_flag)) { ok = false; break; }
                            t_slot += sw.now() - c0;
                            ptx::tc_fence_after();
                        }
                        ptx::tmem_st32(lane_addr + (grp * KB_PER_UNIT + j) * A_COLS, o);
                    }
                    if (!ok) break;
                    ptx::tmem_wait_st();
                    ptx::tc_fence_before();
                }
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&a_full[grp]);
                    ptx::mbar_arrive(&w_empty[ws]);
                }
                if (++grp == C::GROUPS) { grp = 0; gph ^= 1; }
                if (++ws == C::W_STAGES) { ws = 0; wph ^= 1; }
            }
        }
        if (kProf && wa.prof && warp == 6 && lane == 0) {
            long long* pr = wa.prof + g * 16;
            pr[5] = sw.total() - t_begin; pr[6] = t_w; pr[7] = t_slot; pr[8] = t_st;
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2-5)
        grid_dep_wait();
        if constexpr (CS == 0) {
            run_epilogue<MT, (MT < 16) ? MT : 16>(a, it, tmem_base, acc_full, acc_empty, abort_flag, s_last, warp, lane,
                                                  threadIdx.x - 64, g, G, C::ACC2_OFF, C::ACC_STAGES);
        } else {
            if (ptx::mbar_wait_warp(&acc_full[0], 0, abort_flag)) {
                ptx::tc_fence_after();
                const uint32_t t_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
#pragma unroll
                for (int c0 = 0; c0 < MT; c0 += 16) {
                    uint32_t r[16], r2[16];
                    ptx::tmem_ld16(t_addr + c0, r);
                    ptx::tmem_ld16(t_addr + C::ACC2_OFF + c0, r2);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[(c0 + c) % VN] = __uint_as_float(r[c]) + __uint_as_float(r2[c]);
                }
                ptx::tc_fence_before();
            }
        }
    }
    if constexpr (CS > 0) {
        __syncwarp();
        ptx::cluster_wait();   // every CTA of the cluster has started (arrivals at entry): its reduction buffer may be written
        const bool epi = (warp >= 2 && warp < 6);
        cluster_reduce_store<MT, CS>(a, v, reinterpret_cast<float*>(smem + C::OFF_RED), c_rank, c_tile, epi, (warp & 3) * 32 + lane);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error, ERR_GEMM_TIMEOUT);
}

// CPMCU_W4_PROF=1: per-CTA clock counters of the MMA and dequant roles, printed by linear_w4_print_prof().
long long* w4_prof_buffer() {
    static long long* buf = nullptr;
    static bool init = false;
    if (!init) {
        init = true;
        if (tuning_env("CPMCU_W4_PROF")) {
            CUDA_CHECK(cudaMalloc(&buf, 256 * 16 * sizeof(long long)));
            CUDA_CHECK(cudaMemset(buf, 0, 256 * 16 * sizeof(long long)));
        }
    }
    return buf;
}

template <int MT, int CS>
void configure_kernel() {
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(linear_w4_umma_kernel<MT, CS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<MT, CS>::SMEM_BYTES));
        configured = true;
    }
}

template <int MT>
void launch_mt(const LinearPlan& p, const W4Args& args, cudaStream_t stream) {
    configure_kernel<MT, 0>();
    launch_kernel(linear_w4_umma_kernel<MT, 0>, dim3(p.grid), dim3(NUM_THREADS), Cfg<MT>::SMEM_BYTES, stream, p.tm_x, args);
}

template <int MT, int CS>
void launch_cluster(const LinearPlan& p, const W4Args& args, cudaStream_t stream) {
    configure_kernel<MT, CS>();
    launch_kernel_cluster(linear_w4_umma_kernel<MT, CS>, dim3(p.grid), dim3(NUM_THREADS), Cfg<MT, CS>::SMEM_BYTES, stream, CS,
                          p.tm_x, args);
}

template <int MT, int CS>
int capacity() {
    static int cached = -1;
    if (cached < 0) {
        configure_kernel<MT, CS>();
        cached = max_active_clusters(linear_w4_umma_kernel<MT, CS>, dim3(NUM_THREADS), Cfg<MT, CS>::SMEM_BYTES, CS);
    }
    return cached;
}

int cluster_capacity(int mt, int cs) {
    switch (mt * 8 + cs) {
        case 16 * 8 + 2: return capacity<16, 2>();
        case 16 * 8 + 3: return capacity<16, 3>();
        case 16 * 8 + 4: return capacity<16, 4>();
        case 32 * 8 + 2: return capacity<32, 2>();
        case 32 * 8 + 3: return capacity<32, 3>();
        case 32 * 8 + 4: return capacity<32, 4>();
        case 64 * 8 + 2: return capacity<64, 2>();
        case 64 * 8 + 3: return capacity<64, 3>();
        case 64 * 8 + 4: return capacity<64, 4>();
        default: return 0;
    }
}

bool launch_cluster_any(const LinearPlan& p, const W4Args& a, cudaStream_t s) {
    switch (p.mt * 8 + p.cluster) {
        case 16 * 8 + 2: launch_cluster<16, 2>(p, a, s); return true;
        case 16 * 8 + 3: launch_cluster<16, 3>(p, a, s); return true;
        case 16 * 8 + 4: launch_cluster<16, 4>(p, a, s); return true;
        case 32 * 8 + 2: launch_cluster<32, 2>(p, a, s); return true;
        case 32 * 8 + 3: launch_cluster<32, 3>(p, a, s); return true;
        case 32 * 8 + 4: launch_cluster<32, 4>(p, a, s); return true;
        case 64 * 8 + 2: launch_cluster<64, 2>(p, a, s); return true;
        case 64 * 8 + 3: launch_cluster<64, 3>(p, a, s); return true;
        case 64 * 8 + 4: launch_cluster<64, 4>(p, a, s); return true;
        default: return false;
    }
}

}  // namespace

size_t linear_w4_workspace_bytes(int mt, int grid) { return linear_workspace_bytes(mt, grid); }

LinearPlan make_linear_plan_w4(const bf16* x, int x_rows, const void* wq, int M, int N, int K, bf16* y, int ldy,
                               float* workspace, int* tickets, int grid_limit) {
    CPM_REQUIRE(M >= 1 && N >= 1, "linear (W4A16): empty problem");
    CPM_REQUIRE(K % SUPER_K == 0 && N % BLOCK_N == 0, "linear (W4A16): K must be a multiple of 256 and N of 128");
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0,
                "linear (W4A16): operands must be 16-byte aligned");
    LinearPlan p;
    p.M = M; p.N = N; p.K = K;
    p.mt = std::min(linear_pick_mt(M), MAX_MT);
    p.y = y; p.ldy = ldy; p.bias = nullptr;
    p.workspace = workspace; p.tickets = tickets;
    p.wq = wq;
    const int n_tiles = N / BLOCK_N, m_tiles = ceil_div(M, p.mt), units_per_tile = K / SUPER_K;
    const long long units = static_cast<long long>(n_tiles) * m_tiles * units_per_tile;
    long long grid = std::min<long long>(units, grid_limit);
    if (grid < 1) grid = 1;
    if (m_tiles == 1 && grid_limit >= 64) {
        // prefer a grid whose shares end on tile boundaries or split tiles evenly (cheap fix-ups)
        long long best = grid;
        double best_t = 1e30;
        for (long long gsz = 1; gsz <= grid; ++gsz) {
            const long long per = (units + gsz - 1) / gsz;
            // measured: a CTA converts and multiplies a 256-k unit in about 0.85 us (77 GB/s of bf16-equivalent
            // weights), HBM delivers 4-bit weights at four times the bf16-equivalent rate
            const double rate = std::min(77e9, 4.0 * 6.3e12 / gsz);
            double t = per * 65536.0 / rate;
            const bool whole = (units % gsz == 0) && ((units / gsz) % units_per_tile == 0);
            if (!whole) {
                int nseg = (units % gsz == 0 && units_per_tile % (units / gsz) == 0)
                               ? static_cast<int>(units_per_tile / (units / gsz))
                               : static_cast<int>(units_per_tile / (static_cast<double>(units) / gsz)) + 2;
                t += 4.5e-6 + 1.0e-6 * ((M + 15) / 16) * ((nseg + 3) / 4);
            }
            if (t < best_t - 1e-9) { best_t = t; best = gsz; }
        }
        grid = best;
    }
    p.grid = static_cast<int>(grid);
    if (m_tiles > 1) {
        static const bool flat = tuning_env("CPMCU_LINEAR_NO_WAVES") != nullptr;   // bench only: plain stream-K
        if (!flat) plan_waves(static_cast<long long>(n_tiles) * m_tiles, units_per_tile, p.grid, p.wave_tiles, p.tail_grid);
    }
    // pieces of a tile summed inside a thread-block cluster when the device runs all the clusters at once
    // (same rule as the bf16 path; a piece is at least one 256-k unit)
    p.cluster = 0;
    {
        static const bool off = tuning_env("CPMCU_LINEAR_NO_CLUSTER") != nullptr;
        int cs = (m_tiles == 1 && grid % n_tiles == 0) ? static_cast<int>(grid / n_tiles) : 0;
        if (!off && p.mt <= 64 && cs >= 2 && cs <= 4) {
            for (; cs >= 2; --cs) {
                if (units_per_tile >= cs && cluster_capacity(p.mt, cs) >= n_tiles) {
                    p.cluster = cs;
                    p.grid = n_tiles * cs;
                    break;
                }
            }
        }
    }
    // tokens as (64 k, rows, k-blocks): one box = the four k-blocks of a unit, each a 128-byte-swizzled tile
    p.tm_x = make_tmap_3d(x, BLOCK_K, x_rows, K / BLOCK_K, static_cast<uint64_t>(K) * 2, BLOCK_K * 2, BLOCK_K, p.mt,
                          KB_PER_UNIT);
    return p;
}

void launch_linear_w4(const LinearPlan& p, cudaStream_t stream) {
    ProfileScope prof(KC_LINEAR, stream);
    W4Args wa;
    LinearArgs& a = wa.lin;
    a.M = p.M; a.N = p.N; a.K = p.K;
    a.n_tiles = p.N / BLOCK_N;
    a.m_tiles = ceil_div(p.M, p.mt);
    a.kblocks = p.K / SUPER_K;  // work units per tile
    a.wave_tiles = p.wave_tiles;
    a.tail_grid = p.tail_grid;
    a.band = raster_band(p.mt, p.K);
    a.total_units = (static_cast<long long>(a.n_tiles) * a.m_tiles - a.wave_tiles) * a.kblocks;
    a.y = p.y; a.ldy = p.ldy; a.bias = nullptr;
    a.workspace = p.workspace; a.tickets = p.tickets;
    a.error = runtime().d_error;
    static const int debug = tuning_env("CPMCU_LINEAR_DEBUG") ? atoi(tuning_env("CPMCU_LINEAR_DEBUG")) : 0;
    a.debug = debug;
    a.prof = nullptr;
    wa.blocks = static_cast<const uint8_t*>(p.wq);
    wa.prof = kProf ? w4_prof_buffer() : nullptr;
    if (p.cluster != 0 && launch_cluster_any(p, wa, stream)) return;
    switch (p.mt) {
        case 16: launch_mt<16>(p, wa, stream); break;
        case 32: launch_mt<32>(p, wa, stream); break;
        case 64: launch_mt<64>(p, wa, stream); break;
        case 128: launch_mt<128>(p, wa, stream); break;
        default: throw std::invalid_argument("cpmcu_b200: bad token tile");
    }
}

void linear_w4_print_prof() {
    long long* buf = kProf ? w4_prof_buffer() : nullptr;
    if (!buf) return;
    std::vector<long long> h(256 * 16);
    CUDA_CHECK(cudaMemcpy(h.data(), buf, h.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    for (int g : {0, 1, 64, 127}) {
        const long long* p = &h[g * 16];
        fprintf(stderr, "w4 prof cta %d: mma0 total %lld acc_wait %lld a_wait %lld x_wait %lld issue %lld | deq total %lld "
                        "w_wait %lld slot_wait %lld store %lld | mma1 total %lld a_wait %lld x_wait %lld issue %lld\n",
                g, p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], p[8], p[9], p[11], p[12], p[13]);
    }
}
