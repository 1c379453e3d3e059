// Device-resident state of one draft tree (all pointers are device memory).
// Field names follow the reference's EagleImpl members (src/model/eagle.cuh:283-293).
#pragma once
#include "common.cuh"

struct DraftTreeState {
    int k = 0;            // topk_per_iter
    int num_iter = 0;
    int tree_size = 0;
    int total_tried = 0;  // k + k*k*(num_iter-1)
    bf16* tried_val = nullptr;            // [total_tried] cumulative log-probs (bf16)
    int32_t* tried_pos = nullptr;         // [total_tried] draft-vocabulary ids
    int32_t* tried_parent = nullptr;      // [k*(num_iter-1)] tried index of each frontier node
    bf16* fr_score = nullptr;             // [k] frontier cumulative scores
    int32_t* fr_id = nullptr;             // [k] frontier token ids (full vocabulary)
    uint64_t* fr_mask = nullptr;          // [k] frontier ancestor masks over draft keys
    int32_t* fr_src = nullptr;            // [k] row of the level's hidden states each frontier node continues from
    int32_t* sel_pos = nullptr;           // [64] tried index chosen for tree node i+1
    const int32_t* token_id_remap = nullptr;  // FR-Spec: draft id -> full-vocabulary id, or null
};

int draft_num_segments(int vocab);
size_t draft_scan_workspace_bytes(int rows, int vocab, int k);

// log-softmax + top-k of `logits` (1 row at level 0, k rows after) followed by
// the frontier bookkeeping of that level.  st.fr_src[i] receives the row of the
// level's hidden states that frontier node i continues from (*last_row_ptr at level 0,
// the selected parent afterwards).  If hid_out is not null the rows are also gathered,
// hid_out[i] = h_rows[fr_src[i]]; the engine passes null and gathers them in the next
// level's embedding kernel (launch_embedding_gather).
void launch_draft_topk_expand(const DraftTreeState& st, const bf16* logits, int ld, int vocab, int level,
                              void* scan_ws, const bf16* h_rows, int h_ld, const int32_t* last_row_ptr, bf16* hid_out,
                              int hid_ld, int hidden, cudaStream_t s);

// Pick the tree_size-1 best candidates and write tree_draft_ids[1:], positions,
// parents and packed ancestor masks.
void launch_tree_finalize(const DraftTreeState& st, const int32_t* cache_length, int32_t* tree_draft_ids,
                          int32_t* tree_pos, uint64_t* tree_mask, int32_t* tree_parent, cudaStream_t s);

// Greedy acceptance + fix-up (accept.cu).
struct AcceptIO {
    int tree_size = 0;
    int32_t* pred = nullptr;            // in: tree token ids; out: the n emitted tokens in [0,n)
    const int32_t* gt = nullptr;        // target argmax per tree node
    const int32_t* position_ids = nullptr;
    const int32_t* cache_length = nullptr;
    const uint64_t* attn_mask = nullptr;
    const int32_t* tree_parent = nullptr;
    int32_t* result = nullptr;          // [0]=accept length n, [1]=best node, [2..2+n) path node ids
};

struct FixupArgs {
    bf16* const* caches = nullptr;        // device array of num_caches K/V base pointers
    int num_caches = 0;
    int kv_dim = 0;                       // elements per cache row
    int max_accept = 0;                   // num_iter + 1
    const bf16* norm_out = nullptr;       // [tree_size, hidden] target final-norm rows
    bf16* prev_hidden = nullptr;          // [max_accept, hidden]
    const bf16* embed_table = nullptr;
    float embed_scale = 1.f;
    bf16* prev_embed = nullptr;           // [max_accept, hidden]
    int32_t* eagle_pos = nullptr;         // [max_accept] = cache_length + i
    int hidden = 0;                       // 0: caches only (no hidden-state gather, no embeddings)
    int prev_ld = 0;                      // row stride of prev_hidden / prev_embed in elements (0 = hidden)
};
// One launch: acceptance (every CTA recomputes it) + fix-up; io.pred / io.result are written by the CTA that
// is counted last.  cache_rows: rows each cache holds (compaction beyond it is skipped and flagged).
void launch_accept_fixup(const AcceptIO& io, const FixupArgs& a, int cache_rows, cudaStream_t s);
