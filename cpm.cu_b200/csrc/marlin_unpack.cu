// W4A16 GPTQ-Marlin checkpoints: unpacking of the Marlin tile layout and dequantisation
// `w = (q - 8) * scale` (reference src/qgemm/gptq_marlin/gptq_marlin.cu:139-162, layout
// produced by model_convert/convert_w4a16.py:17-82) into the row-major bf16 [N, K] matrix the
// streaming GEMM reads.  Runs once per tensor at load time.
#include <vector>

#include "common.cuh"

namespace {

__constant__ int16_t c_marlin_perm[1024];

// Index table of the Marlin repack: position c of a 1024-wide group holds element PERM[c] of the
// 16 x 16-tiled source (four tiles of 256).
std::vector<int16_t> build_perm() {
    std::vector<int> perm;
    for (int i = 0; i < 32; ++i) {
        std::vector<int> one;
        const int col = i / 4;
        for (int block = 0; block < 2; ++block) {
            const int rows[4] = {2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1};
            for (int r = 0; r < 4; ++r) one.push_back(16 * rows[r] + col + 8 * block);
        }
        for (int j = 0; j < 4; ++j) {
            for (int p : one) perm.push_back(p + 256 * j);
        }
    }
    static const int interleave[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    std::vector<int16_t> out(1024);
    for (int g = 0; g < 128; ++g) {
        for (int e = 0; e < 8; ++e) out[g * 8 + e] = static_cast<int16_t>(perm[g * 8 + interleave[e]]);
    }
    return out;
}

// One thread per packed 32-bit word (eight 4-bit values).
__global__ void marlin_dequant_kernel(const uint32_t* __restrict__ packed, const bf16* __restrict__ scales, int K, int N,
                                      bf16* __restrict__ dst) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long words = static_cast<long long>(K / 16) * N * 2;
    if (idx >= words) return;
    const int kt = static_cast<int>(idx / (2LL * N));
    const int wcol = static_cast<int>(idx - static_cast<long long>(kt) * 2 * N);
    const uint32_t word = packed[idx];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int col = wcol * 8 + i;
        const int g = col >> 10, c = col & 1023;
        const int src = c_marlin_perm[c];
        const int n = (g * 4 + (src >> 8)) * 16 + (src & 15);
        const int k = kt * 16 + ((src & 255) >> 4);
        // scales are stored permuted in chunks of 64: entry (i + 8 j) of a chunk sits at position 8 i + j
        const long long flat = static_cast<long long>(k >> 7) * N + n;
        const long long chunk = flat >> 6;
        const int pos = static_cast<int>(flat & 63);
        const float s = __bfloat162float(scales[chunk * 64 + (pos & 7) * 8 + (pos >> 3)]);
        const int q = static_cast<int>((word >> (4 * i)) & 0xF) - 8;
        dst[static_cast<size_t>(n) * K + k] = __float2bfloat16(static_cast<float>(q) * s);
    }
}

__constant__ int16_t c_marlin_invperm[1024];

// Streaming layout of the W4A16 GEMM: one contiguous 16896-byte block per (128-feature tile, 256-k unit),
// [4 k-blocks of 64][2 halves of 32 k][128 rows][16 B of nibbles] followed by [2 scale groups][128 rows]
// bf16, so that one untiled bulk copy fills a pipeline stage and a warp reads 512 contiguous bytes.
constexpr int W4_BLOCK_BYTES = 128 * 256 / 2 + 2 * 128 * 2;

// One thread per output word (n, j): gathers q[k = 8j .. 8j+7][n] from the Marlin tensor and packs
// them k0 k2 k4 k6 k1 k3 k5 k7 from bit 0, so that (word >> 4i) & 0x000f000f yields the pair
// (k = 2i, k = 2i + 1) in the two bf16 lanes.
__global__ void marlin_retile_kernel(const uint32_t* __restrict__ packed, int K, int N, uint8_t* __restrict__ blocks) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long words = static_cast<long long>(N) * (K / 8);
    if (idx >= words) return;
    const int n = static_cast<int>(idx / (K / 8));
    const int j = static_cast<int>(idx - static_cast<long long>(n) * (K / 8));
    uint32_t out = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int k = j * 8 + e;
        const int kt = k >> 4;
        const long long old_col = static_cast<long long>(n >> 4) * 256 + (k & 15) * 16 + (n & 15);
        const long long col = (old_col & ~1023LL) + c_marlin_invperm[old_col & 1023];
        const uint32_t word = packed[static_cast<long long>(kt) * 2 * N + (col >> 3)];
        const uint32_t q = (word >> (4 * (col & 7))) & 0xF;
        const int slot = (e & 1) ? 4 + (e >> 1) : (e >> 1);
        out |= q << (4 * slot);
    }
    const int unit = j >> 5, jw = j & 31;
    const long long block = static_cast<long long>(n >> 7) * (K / 256) + unit;
    *reinterpret_cast<uint32_t*>(blocks + block * W4_BLOCK_BYTES + (jw >> 3) * 4096 + ((jw >> 2) & 1) * 2048 + (n & 127) * 16 + (jw & 3) * 4) = out;
}

__global__ void marlin_unpermute_scales_kernel(const bf16* __restrict__ sperm, int K, int N, uint8_t* __restrict__ blocks) {
    const long long flat = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= static_cast<long long>(K / 128) * N) return;
    const int pos = static_cast<int>(flat & 63);
    const bf16 v = sperm[(flat & ~63LL) + (pos & 7) * 8 + (pos >> 3)];
    const int grp = static_cast<int>(flat / N), n = static_cast<int>(flat - static_cast<long long>(grp) * N);
    const long long block = static_cast<long long>(n >> 7) * (K / 256) + (grp >> 1);
    *reinterpret_cast<bf16*>(blocks + block * W4_BLOCK_BYTES + 16384 + (grp & 1) * 256 + (n & 127) * 2) = v;
}

void upload_tables() {
    static bool ready = false;
    if (ready) return;
    const std::vector<int16_t> perm = build_perm();
    std::vector<int16_t> inv(1024);
    for (int c = 0; c < 1024; ++c) inv[perm[c]] = static_cast<int16_t>(c);
    CUDA_CHECK(cudaMemcpyToSymbol(c_marlin_perm, perm.data(), perm.size() * sizeof(int16_t)));
    CUDA_CHECK(cudaMemcpyToSymbol(c_marlin_invperm, inv.data(), inv.size() * sizeof(int16_t)));
    ready = true;
}

}  // namespace

size_t linear_w4_weight_bytes(int N, int K) {
    return static_cast<size_t>(N / 128) * (K / 256) * W4_BLOCK_BYTES;
}

void marlin_retile_for_w4(const void* packed, const void* scales, int K, int N, void* blocks, cudaStream_t s) {
    CPM_REQUIRE(K % 256 == 0 && N % 128 == 0, "W4A16 GEMM: K must be a multiple of 256 and N a multiple of 128");
    upload_tables();
    const long long words = static_cast<long long>(N) * (K / 8);
    marlin_retile_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, s>>>(static_cast<const uint32_t*>(packed), K,
                                                                                   N, static_cast<uint8_t*>(blocks));
    CUDA_CHECK(cudaGetLastError());
    const long long count = static_cast<long long>(K / 128) * N;
    marlin_unpermute_scales_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, s>>>(
        static_cast<const bf16*>(scales), K, N, static_cast<uint8_t*>(blocks));
    CUDA_CHECK(cudaGetLastError());
}

void marlin_dequant_to_bf16(const void* packed, const void* scales, int K, int N, int group_size, bf16* dst,
                            cudaStream_t s) {
    CPM_REQUIRE(group_size == 128, "W4A16: only group_size 128 is supported");
    CPM_REQUIRE(K % 128 == 0 && N % 64 == 0, "W4A16: K must be a multiple of 128 and N a multiple of 64");
    upload_tables();
    const long long words = static_cast<long long>(K / 16) * N * 2;
    marlin_dequant_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, s>>>(
        static_cast<const uint32_t*>(packed), static_cast<const bf16*>(scales), K, N, dst);
    CUDA_CHECK(cudaGetLastError());
}
