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
//   W producer   TMA: packed nibbles of a 128-row x 256-k super-block (16 KB) + its two rows of
//                scales (bulk copies), ring of W stages; the ring is filled before the
//                programmatic-dependency wait (weights never depend on the previous kernel)
//   dequant      8 warps: 16 B of nibbles -> 32 bf16 per thread with the 0x4300 magic-number
//                trick (128 + q is exact in bf16), (x - 136) * scale, written as the 128-byte
//                swizzled K-major A tile of one 64-k block (ring of A buffers)
//   X producer   TMA: token tiles per 64-k block (ring of X entries)
//   MMA          tcgen05.mma A buffer x X entry, commits free both
//   epilogue     shared with the bf16 kernel
//
// HBM sees 0.5 byte per weight; the in-flight budget is the W ring (6 x 16 KB per SM).
#include <algorithm>

#include "common.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

using namespace gemm;

namespace {

constexpr int BLOCK_K = 64;          // k per MMA block (128-byte swizzle row of bf16)
constexpr int SUPER_K = 256;         // k per W stage and per stream-K unit
constexpr int KB_PER_UNIT = SUPER_K / BLOCK_K;
constexpr int UMMA_K = 16;
constexpr int WQ_BYTES = BLOCK_N * SUPER_K / 2;   // 16 KB of nibbles
constexpr int WS_BYTES = 2 * BLOCK_N * 2;         // two scale rows (groups of 128 k) x 128 features
constexpr int W_STAGE_BYTES = WQ_BYTES + 1024;    // scales in the last KB (keeps stages 1024-aligned)
constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2;    // 16 KB bf16 A tile
constexpr int NUM_A = 3;
constexpr int DEQ_WARPS = 8;
constexpr int DEQ_THREADS = DEQ_WARPS * 32;
// warp 0: W producer, warp 1: MMA + TMEM, warps 2-5: epilogue, warps 6-13: dequant, warp 14: X producer
constexpr int NUM_THREADS = (6 + DEQ_WARPS + 1) * 32;

template <int MT>
struct Cfg {
    static constexpr int X_BYTES = MT * BLOCK_K * 2;
    static constexpr int W_STAGES = (MT <= 64) ? 6 : 3;
    static constexpr int X_STAGES = (MT <= 16) ? 12 : (MT <= 32) ? 10 : (MT <= 64) ? 8 : (MT <= 128) ? 4 : 3;
    static constexpr int TMEM_COLS = (2 * MT < 32) ? 32 : 2 * MT;
    static constexpr int OFF_W = 0;
    static constexpr int OFF_A = OFF_W + W_STAGES * W_STAGE_BYTES;
    static constexpr int OFF_X = OFF_A + NUM_A * A_BYTES;
    static constexpr int OFF_CTRL = OFF_X + X_STAGES * X_BYTES;
    static constexpr int SMEM_BYTES = OFF_CTRL + 512 + 1024;
};

struct W4Args {
    LinearArgs lin;
    const bf16* wscales;  // [K/128][N]
};

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return r;
}

template <int MT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
linear_w4_umma_kernel(const __grid_constant__ CUtensorMap tm_wq, const __grid_constant__ CUtensorMap tm_x,
                      const W4Args wa) {
    using C = Cfg<MT>;
    const LinearArgs& a = wa.lin;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_CTRL);
    uint64_t* w_full = bars;                       // [W_STAGES]
    uint64_t* w_empty = w_full + C::W_STAGES;      // [W_STAGES]  256 dequant arrivals
    uint64_t* a_full = w_empty + C::W_STAGES;      // [NUM_A]     256 dequant arrivals
    uint64_t* a_empty = a_full + NUM_A;            // [NUM_A]     MMA commit
    uint64_t* x_full = a_empty + NUM_A;            // [X_STAGES]
    uint64_t* x_empty = x_full + C::X_STAGES;      // [X_STAGES]  MMA commit
    uint64_t* acc_full = x_empty + C::X_STAGES;    // [2]
    uint64_t* acc_empty = acc_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* s_last = abort_flag + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int g = blockIdx.x;
    grid_dep_trigger();

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::W_STAGES; ++s) {
            ptx::mbar_init(&w_full[s], 1);
            ptx::mbar_init(&w_empty[s], DEQ_THREADS);
        }
        for (int s = 0; s < NUM_A; ++s) {
            ptx::mbar_init(&a_full[s], DEQ_THREADS);
            ptx::mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < C::X_STAGES; ++s) {
            ptx::mbar_init(&x_full[s], 1);
            ptx::mbar_init(&x_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_init(&acc_full[s], 1);
            ptx::mbar_init(&acc_empty[s], 128);
        }
        *abort_flag = 0;
        *s_last = 0;
        ptx::mbar_fence_init();
        ptx::prefetch_tensormap(&tm_wq);
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
    SegIter it;
    it.u = (a.total_units * g) / G;
    it.u_end = (a.total_units * (g + 1)) / G;
    it.kblocks = a.kblocks;

    if (warp == 0) {
        // ------------------------------------------------ W producer (weights only: runs ahead of the dependency wait)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int tile, u0, u1;
            bool ok = true;
            while (ok && it.next(tile, u0, u1)) {
                const int n_tile = tile % a.n_tiles;
                for (int u = u0; u < u1; ++u) {
                    if (!ptx::mbar_wait(&w_empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* dst = smem + C::OFF_W + stage * W_STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(&w_full[stage], WQ_BYTES + WS_BYTES);
                    // four 64-k sub-tiles of 128 rows x 32 B each, so that a dequant warp reads contiguous bytes
#pragma unroll
                    for (int j = 0; j < KB_PER_UNIT; ++j) {
                        ptx::tma_load_2d(dst + j * (BLOCK_N * 32), &tm_wq, &w_full[stage], u * (SUPER_K / 2) + j * 32,
                                         n_tile * BLOCK_N);
                    }
                    const bf16* srow = wa.wscales + static_cast<size_t>(u) * 2 * a.N + n_tile * BLOCK_N;
                    ptx::bulk_load(dst + WQ_BYTES, srow, BLOCK_N * 2, &w_full[stage]);
                    ptx::bulk_load(dst + WQ_BYTES + BLOCK_N * 2, srow + a.N, BLOCK_N * 2, &w_full[stage]);
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
        // ------------------------------------------------ X producer
        grid_dep_wait();
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int tile, u0, u1;
            bool ok = true;
            while (ok && it.next(tile, u0, u1)) {
                const int m_tile = tile / a.n_tiles;
                for (int kb = u0 * KB_PER_UNIT; kb < u1 * KB_PER_UNIT; ++kb) {
                    if (!ptx::mbar_wait(&x_empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(&x_full[stage], C::X_BYTES);
                    ptx::tma_load_2d(smem + C::OFF_X + stage * C::X_BYTES, &tm_x, &x_full[stage], kb * BLOCK_K, m_tile * MT);
                    if (++stage == C::X_STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        grid_dep_wait();
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(BLOCK_N, MT, 0, 0);
            int xs = 0, as = 0;
            uint32_t xph = 0, aph = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            int tile, u0, u1;
            bool ok = true;
            while (ok && it.next(tile, u0, u1)) {
                if (!ptx::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * MT;
                const int kb_begin = u0 * KB_PER_UNIT, kb_end = u1 * KB_PER_UNIT;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!ptx::mbar_wait(&a_full[as], aph, abort_flag)) { ok = false; break; }
                    if (!ptx::mbar_wait(&x_full[xs], xph, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t aa = ptx::smem_u32(smem + C::OFF_A + as * A_BYTES);
                    const uint32_t xa = ptx::smem_u32(smem + C::OFF_X + xs * C::X_BYTES);
#pragma unroll
                    for (int j = 0; j < BLOCK_K / UMMA_K; ++j) {
                        const uint64_t da = ptx::umma_desc_sw128(aa + j * UMMA_K * 2, 16, 1024);
                        const uint64_t db = ptx::umma_desc_sw128(xa + j * UMMA_K * 2, 16, 1024);
                        ptx::umma_ss(d_tmem, da, db, idesc, (kb > kb_begin || j > 0) ? 1u : 0u);
                    }
                    ptx::umma_commit(&a_empty[as]);
                    ptx::umma_commit(&x_empty[xs]);
                    if (++as == NUM_A) { as = 0; aph ^= 1; }
                    if (++xs == C::X_STAGES) { xs = 0; xph ^= 1; }
                }
                if (!ok) break;
                ptx::umma_commit(&acc_full[acc]);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (warp >= 6) {
        // ------------------------------------------------ dequant warps: nibbles -> swizzled bf16 A tiles
        const int dt = threadIdx.x - 6 * 32;  // 0..255
        const int row = dt >> 1, half = dt & 1;
        int ws = 0, as = 0;
        uint32_t wph = 0, aph = 0;
        int tile, u0, u1;
        bool ok = true;
        const __nv_bfloat162 bias2 = __floats2bfloat162_rn(136.f, 136.f);  // 128 (magic) + 8 (zero point)
        while (ok && it.next(tile, u0, u1)) {
            for (int u = u0; u < u1 && ok; ++u) {
                if (!ptx::mbar_wait(&w_full[ws], wph, abort_flag)) { ok = false; break; }
                const uint8_t* wst = smem + C::OFF_W + ws * W_STAGE_BYTES;
                const bf16* sc = reinterpret_cast<const bf16*>(wst + WQ_BYTES);
#pragma unroll 1
                for (int j = 0; j < KB_PER_UNIT; ++j) {
                    // 32 nibbles of this thread: k = 64 j + 32 half .. + 31 of row `row`
                    const uint4 pk = *reinterpret_cast<const uint4*>(wst + j * (BLOCK_N * 32) + row * 32 + half * 16);
                    const bf16 s1 = sc[(j >> 1) * BLOCK_N + row];
                    const __nv_bfloat162 s2 = __halves2bfloat162(s1, s1);
                    if (!ptx::mbar_wait(&a_empty[as], aph ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* arow = smem + C::OFF_A + as * A_BYTES + row * 128;
                    const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        uint4 o;
                        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t bits = lop3_and_or(words[w] >> (4 * i), 0x000f000fu, 0x43004300u);
                            __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&bits);  // (128 + q_lo, 128 + q_hi)
                            v = __hmul2(__hsub2(v, bias2), s2);                                  // exact subtract, one rounding
                            ow[i] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        const int chunk = half * 4 + w;  // 16-byte chunk (8 k) within the 128-byte row
                        *reinterpret_cast<uint4*>(arow + ((chunk ^ (row & 7)) << 4)) = o;
                    }
                    ptx::fence_proxy_async_smem();
                    ptx::mbar_arrive(&a_full[as]);
                    if (++as == NUM_A) { as = 0; aph ^= 1; }
                }
                ptx::mbar_arrive(&w_empty[ws]);
                if (++ws == C::W_STAGES) { ws = 0; wph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2-5)
        grid_dep_wait();
        run_epilogue<MT, (MT < 16) ? MT : 16>(a, it, tmem_base, acc_full, acc_empty, abort_flag, s_last, warp, lane,
                                              threadIdx.x - 64, g, G);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error, ERR_GEMM_TIMEOUT);
}

template <int MT>
void launch_mt(const LinearPlan& p, const W4Args& args, cudaStream_t stream) {
    using C = Cfg<MT>;
    static bool configured = false;
    if (!configured) {
        CUDA_CHECK(cudaFuncSetAttribute(linear_w4_umma_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C::SMEM_BYTES));
        configured = true;
    }
    launch_kernel(linear_w4_umma_kernel<MT>, dim3(p.grid), dim3(NUM_THREADS), C::SMEM_BYTES, stream, p.tm_w, p.tm_x, args);
}

}  // namespace

size_t linear_w4_workspace_bytes(int mt, int grid) { return linear_workspace_bytes(mt, grid); }

LinearPlan make_linear_plan_w4(const bf16* x, int x_rows, const uint32_t* wq, const bf16* wscales, int M, int N, int K,
                               bf16* y, int ldy, float* workspace, int* tickets, int grid_limit) {
    CPM_REQUIRE(M >= 1 && N >= 1, "linear (W4A16): empty problem");
    CPM_REQUIRE(K % SUPER_K == 0 && N % BLOCK_N == 0, "linear (W4A16): K must be a multiple of 256 and N of 128");
    CPM_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(wscales) & 15) == 0,
                "linear (W4A16): operands must be 16-byte aligned");
    LinearPlan p;
    p.M = M; p.N = N; p.K = K;
    p.mt = linear_pick_mt(M);
    p.y = y; p.ldy = ldy; p.bias = nullptr;
    p.workspace = workspace; p.tickets = tickets;
    p.wq = wq;
    p.wscales = wscales;
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
            const double rate = std::min(55e9, 6.3e12 / gsz) * 4.0;  // bf16-equivalent bytes per second
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
    p.tm_w = make_tmap_2d_u8(wq, static_cast<uint64_t>(K) / 2, N, static_cast<uint64_t>(K) / 2, 32, BLOCK_N);
    p.tm_x = make_tmap_2d(x, K, x_rows, static_cast<uint64_t>(K) * 2, BLOCK_K, p.mt);
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
    a.total_units = static_cast<long long>(a.n_tiles) * a.m_tiles * a.kblocks;
    a.y = p.y; a.ldy = p.ldy; a.bias = nullptr;
    a.workspace = p.workspace; a.tickets = p.tickets;
    a.error = runtime().d_error;
    a.debug = 0;
    wa.wscales = p.wscales;
    switch (p.mt) {
        case 16: launch_mt<16>(p, wa, stream); break;
        case 32: launch_mt<32>(p, wa, stream); break;
        case 64: launch_mt<64>(p, wa, stream); break;
        case 128: launch_mt<128>(p, wa, stream); break;
        case 256: launch_mt<256>(p, wa, stream); break;
        default: throw std::invalid_argument("cpmcu_b200: bad token tile");
    }
}
