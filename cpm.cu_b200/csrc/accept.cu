// Greedy tree acceptance and the fix-up that follows it.
//
// verify_accept_kernel restates the reference's verify_kernel
// (src/model/tree_drafter.cuh:5-46): node i is correct when its token equals
// the target's argmax at its parent; a node is accepted when every node on its
// root path is correct; the deepest accepted node wins.  Warp ballots build the
// 64-bit correct set; a 64-bit max-reduction of (depth, node) picks the winner.
//
// accept_fixup_kernel fuses what the reference does in four launches and a
// device copy (fix_kvcache_kernel_1/2 tree_drafter.cuh:48-77, remap_hidden
// eagle.cuh:108-115, embedding + make_arange minicpm4_eagle.cuh:404-412):
// compaction of the accepted K/V rows of every cache, the gather of the next
// draft hidden states, the embedding of the emitted tokens and their positions.
// A thread owns one 16-byte column of one cache, loads all accepted source rows
// and then stores them, so rows are moved without a staging buffer; hidden
// states are gathered into a separate buffer, which removes the in-place
// overwrite hazard of the reference gather.
#include "common.cuh"
#include "draft_tree.cuh"

namespace {

constexpr int MAX_PATH = 16;

__global__ void verify_accept_kernel(AcceptIO io) {
    grid_dependency_sync();
    __shared__ unsigned long long s_correct[2];
    __shared__ unsigned long long s_best[2];
    const int i = threadIdx.x;  // 64 threads
    const int T = io.tree_size;
    const int L = io.cache_length[0];
    bool correct = (i == 0);
    if (i > 0 && i < T) correct = (io.pred[i] == io.gt[io.tree_parent[i]]);
    const unsigned bal = __ballot_sync(0xffffffffu, correct);
    if ((i & 31) == 0) s_correct[i >> 5] = static_cast<unsigned long long>(bal);
    __syncthreads();
    const unsigned long long correct_mask = s_correct[0] | (s_correct[1] << 32);
    const unsigned long long my_mask = (i < T) ? io.attn_mask[i] : 0ull;
    const int my_pos = (i < T) ? io.position_ids[i] : 0;
    // key = depth * 64 + (63 - node): deepest wins; accepted nodes of equal depth cannot coexist
    unsigned long long key = (1ull << 6) | 63ull;  // root: depth 1, node 0
    if (i < T && (correct_mask & my_mask) == my_mask) {
        key = (static_cast<unsigned long long>(my_pos - L + 1) << 6) | static_cast<unsigned long long>(63 - i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = (other > key) ? other : key;
    }
    if ((i & 31) == 0) s_best[i >> 5] = key;
    __syncthreads();
    key = (s_best[0] > s_best[1]) ? s_best[0] : s_best[1];
    const int n = static_cast<int>(key >> 6);
    const int best = 63 - static_cast<int>(key & 63ull);
    const unsigned long long path_mask = io.attn_mask[best];
    // every thread has read pred[] above; safe to overwrite after the barrier
    __syncthreads();
    int slot = -1;
    if (i < T && ((path_mask >> i) & 1ull)) {
        slot = my_pos - L;
        if (slot >= 0 && slot < MAX_PATH) io.result[2 + slot] = i;
    }
    __syncthreads();
    __threadfence_block();
    if (i < n && i < MAX_PATH) {
        io.pred[i] = io.gt[io.result[2 + i]];  // emitted tokens, last one is the bonus token
    }
    if (i == 0) {
        io.result[0] = n;
        io.result[1] = best;
    }
}

__global__ void accept_fixup_kernel(FixupArgs a) {
    grid_dependency_sync();
    const int n = min(a.result[0], a.max_accept);
    const int L = a.cache_length[0];
    const int vec_per_row = a.kv_dim / 8;
    const int kv_threads = a.num_caches * vec_per_row;
    const int hid_vec = a.hidden / 8;
    const int gid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gid < kv_threads) {
        const int c = gid / vec_per_row, v = gid - c * vec_per_row;
        uint4* base = reinterpret_cast<uint4*>(a.caches[c]);
        uint4 rows[MAX_PATH];
#pragma unroll
        for (int i = 0; i < MAX_PATH; ++i) {
            if (i < n) rows[i] = base[static_cast<size_t>(L + a.result[2 + i]) * vec_per_row + v];
        }
#pragma unroll
        for (int i = 0; i < MAX_PATH; ++i) {
            if (i < n) base[static_cast<size_t>(L + i) * vec_per_row + v] = rows[i];
        }
        return;
    }
    int rest = gid - kv_threads;
    if (rest < a.max_accept * hid_vec) {  // next draft hidden states
        const int i = rest / hid_vec, v = rest - i * hid_vec;
        if (i < n) {
            reinterpret_cast<uint4*>(a.prev_hidden)[static_cast<size_t>(i) * hid_vec + v] =
                reinterpret_cast<const uint4*>(a.norm_out)[static_cast<size_t>(a.result[2 + i]) * hid_vec + v];
        }
        return;
    }
    rest -= a.max_accept * hid_vec;
    if (rest < a.max_accept * hid_vec) {  // embeddings of the emitted tokens
        const int i = rest / hid_vec, v = rest - i * hid_vec;
        if (i < n) {
            uint4 e = reinterpret_cast<const uint4*>(a.embed_table)[static_cast<size_t>(a.tokens[i]) * hid_vec + v];
            if (a.embed_scale != 1.0f) {
                bf16* p = reinterpret_cast<bf16*>(&e);
#pragma unroll
                for (int j = 0; j < 8; ++j) p[j] = __float2bfloat16(__bfloat162float(p[j]) * a.embed_scale);
            }
            reinterpret_cast<uint4*>(a.prev_embed)[static_cast<size_t>(i) * hid_vec + v] = e;
        }
        if (v == 0 && i < a.max_accept) a.eagle_pos[i] = L + i;
        return;
    }
}

}  // namespace

void launch_verify_accept(const AcceptIO& io, cudaStream_t s) {
    CPM_REQUIRE(io.tree_size >= 1 && io.tree_size <= 64, "verify: tree_size must be in [1,64]");
    launch_kernel(verify_accept_kernel, dim3(1), dim3(64), 0, s, io);
}

void launch_accept_fixup(const FixupArgs& a, cudaStream_t s) {
    CPM_REQUIRE(a.max_accept >= 1 && a.max_accept <= MAX_PATH, "fixup: accept length bound out of range");
    CPM_REQUIRE(a.kv_dim % 8 == 0 && a.hidden % 8 == 0, "fixup: row sizes must be multiples of 8 elements");
    const long long threads = static_cast<long long>(a.num_caches) * (a.kv_dim / 8) +
                              2LL * a.max_accept * (a.hidden / 8);
    launch_kernel(accept_fixup_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256), 0, s, a);
}
