// Greedy tree acceptance and the fix-up that follows it, in ONE launch.
//
// Acceptance restates the reference's verify_kernel (src/model/tree_drafter.cuh:5-46): node i is correct
// when its token equals the target's argmax at its parent; a node is accepted when every node on its root
// path is correct; the deepest accepted node wins.  Warp ballots build the 64-bit correct set; a 64-bit
// max-reduction of (depth, node) picks the winner.  It is 64 threads of work, so every CTA of the launch
// recomputes it from the tree arrays instead of waiting for a separate one-CTA kernel.
//
// The fix-up fuses what the reference does in four launches and a device copy (fix_kvcache_kernel_1/2
// tree_drafter.cuh:48-77, remap_hidden eagle.cuh:108-115, embedding + make_arange
// minicpm4_eagle.cuh:404-412): compaction of the accepted K/V rows of every cache, the gather of the next
// draft hidden states, the embedding of the emitted tokens and their positions.  A thread owns one 16-byte
// column of one cache, loads all accepted source rows and then stores them, so rows are moved without a
// staging buffer; hidden states are gathered into a separate buffer, which removes the in-place overwrite
// hazard of the reference gather.
//
// `pred` is both input (the tree's tokens) and output (the emitted tokens): the CTA that is counted last
// on the ticket, i.e. after every CTA has read the tree, writes the outputs and clears the ticket.
#include "common.cuh"
#include "draft_tree.cuh"

namespace {

constexpr int MAX_PATH = 16;

__global__ void accept_fixup_kernel(AcceptIO io, FixupArgs a, int cache_rows, int* __restrict__ error,
                                    unsigned* __restrict__ ticket) {
    grid_dependency_sync();
    __shared__ unsigned long long s_correct[2];
    __shared__ unsigned long long s_best[2];
    __shared__ int s_path[MAX_PATH];
    __shared__ int s_tok[MAX_PATH];
    __shared__ int s_last;
    const int tid = threadIdx.x;  // 256 threads; the first 64 hold one tree node each
    const int T = io.tree_size;
    const int L = io.cache_length[0];
    int n = 0, best = 0;
    {
        const int i = tid;
        bool correct = (i == 0);
        if (i > 0 && i < T) correct = (io.pred[i] == io.gt[io.tree_parent[i]]);
        const unsigned bal = __ballot_sync(0xffffffffu, correct);
        if (i < 64 && (i & 31) == 0) s_correct[i >> 5] = static_cast<unsigned long long>(bal);
        if (i < MAX_PATH) s_path[i] = 0;
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
        if (i < 64 && (i & 31) == 0) s_best[i >> 5] = key;
        __syncthreads();
        key = (s_best[0] > s_best[1]) ? s_best[0] : s_best[1];
        n = static_cast<int>(key >> 6);
        best = 63 - static_cast<int>(key & 63ull);
        const unsigned long long path_mask = io.attn_mask[best];
        if (i < T && ((path_mask >> i) & 1ull)) {
            const int slot = my_pos - L;
            if (slot >= 0 && slot < MAX_PATH) s_path[slot] = i;
        }
        __syncthreads();
        if (i < MAX_PATH) s_tok[i] = (i < n) ? io.gt[s_path[i]] : -1;  // emitted tokens, the last one is the bonus token
        __syncthreads();
    }
    const int n_fix = min(n, a.max_accept);
    const int vec_per_row = a.kv_dim / 8;
    const int kv_threads = a.num_caches * vec_per_row;
    const int hid_vec = a.hidden / 8;
    const int prev_vec = (a.prev_ld > 0 ? a.prev_ld : a.hidden) / 8;
    const int gid = blockIdx.x * blockDim.x + tid;
    if (gid < kv_threads) {
        if (L + n_fix > cache_rows) {  // host-side length checks come first; this only keeps memory intact
            if (gid == 0) atomicOr(error, ERR_KV_OVERFLOW);
        } else {
            const int c = gid / vec_per_row, v = gid - c * vec_per_row;
            uint4* base = reinterpret_cast<uint4*>(a.caches[c]);
            uint4 rows[MAX_PATH];
#pragma unroll
            for (int i = 0; i < MAX_PATH; ++i) {
                if (i < n_fix) rows[i] = base[static_cast<size_t>(L + s_path[i]) * vec_per_row + v];
            }
#pragma unroll
            for (int i = 0; i < MAX_PATH; ++i) {
                if (i < n_fix) base[static_cast<size_t>(L + i) * vec_per_row + v] = rows[i];
            }
        }
    } else if (hid_vec > 0) {
        int rest = gid - kv_threads;
        if (rest < a.max_accept * hid_vec) {  // next draft hidden states
            const int i = rest / hid_vec, v = rest - i * hid_vec;
            if (i < n_fix) {
                reinterpret_cast<uint4*>(a.prev_hidden)[static_cast<size_t>(i) * prev_vec + v] =
                    reinterpret_cast<const uint4*>(a.norm_out)[static_cast<size_t>(s_path[i]) * hid_vec + v];
            }
        } else if (rest < 2 * a.max_accept * hid_vec) {  // embeddings of the emitted tokens
            rest -= a.max_accept * hid_vec;
            const int i = rest / hid_vec, v = rest - i * hid_vec;
            if (i < n_fix) {
                uint4 e = reinterpret_cast<const uint4*>(a.embed_table)[static_cast<size_t>(s_tok[i]) * hid_vec + v];
                if (a.embed_scale != 1.0f) {
                    bf16* p = reinterpret_cast<bf16*>(&e);
#pragma unroll
                    for (int j = 0; j < 8; ++j) p[j] = __float2bfloat16(__bfloat162float(p[j]) * a.embed_scale);
                }
                reinterpret_cast<uint4*>(a.prev_embed)[static_cast<size_t>(i) * prev_vec + v] = e;
            }
            if (v == 0 && i < a.max_accept) a.eagle_pos[i] = L + i;
        }
    }
    // outputs that overwrite inputs: only after every CTA has read the tree
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        if (tid < MAX_PATH) {
            io.result[2 + tid] = s_path[tid];
            if (tid < n) io.pred[tid] = s_tok[tid];
        }
        if (tid == 0) {
            io.result[0] = n;
            io.result[1] = best;
            *ticket = 0u;
        }
    }
}

}  // namespace

void launch_accept_fixup(const AcceptIO& io, const FixupArgs& a, int cache_rows, cudaStream_t s) {
    CPM_REQUIRE(io.tree_size >= 1 && io.tree_size <= 64, "verify: tree_size must be in [1,64]");
    CPM_REQUIRE(a.max_accept >= 1 && a.max_accept <= MAX_PATH, "fixup: accept length bound out of range");
    CPM_REQUIRE(a.kv_dim % 8 == 0 && a.hidden % 8 == 0 && a.prev_ld % 8 == 0, "fixup: row sizes must be multiples of 8 elements");
    const long long threads = static_cast<long long>(a.num_caches) * (a.kv_dim / 8) +
                              2LL * a.max_accept * (a.hidden / 8);
    const unsigned grid = static_cast<unsigned>(threads > 0 ? (threads + 255) / 256 : 1);
    Runtime& rt = runtime();
    launch_kernel(accept_fixup_kernel, dim3(grid), dim3(256), 0, s, io, a, cache_rows, rt.d_error, rt.d_accept_ticket);
}
