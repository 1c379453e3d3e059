"""CPU oracle (PyTorch, host cores) for the floating-point stages and the whole
speculative step: target forward (prefill, tree verify), EAGLE draft loop,
acceptance and fix-up, and the generate loops.

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the
cpu_baseline / reference arms of bench.py.  Nothing in the product imports it.

PARITY: the integer stages this file calls (oracle/tree.py, oracle/sparse.py) are
pinned bit for bit against the reference's own kernels (tests/test_ref_golden_cpu.py).
The float composition here (layer order, where values are rounded, attention,
the generate loops) is UNPINNED: the reference's model classes include its
attention code, which needs the un-vendored CUTLASS tree, so they cannot be
compiled or run here; it is restated from the sources cited below.  The row-wise
kernels and GEMMs it is built from are compared with the reference's own on the
GPU in tests/test_ref_kernels_gpu.py.

Numerics: `dtype="bf16"` rounds to bf16 exactly where the reference stores the
model dtype (GEMM outputs, norm outputs, RoPE outputs, activation outputs,
residual adds, log-softmax, cumulative scores) and computes everything else in
fp32; `dtype="fp32"` never rounds (BASELINE config 1).
"""
import math

import numpy as np
import torch

from . import sparse as osparse
from . import tree as otree


class OracleConfig:
    def __init__(self, vocab, layers, hidden, inter, hq, hkv, head_dim, eps=1e-5, rope_theta=10000.0,
                 scale_embed=1.0, scale_lmhead=1.0, scale_residual=1.0, dtype="bf16"):
        self.vocab, self.layers, self.hidden, self.inter = vocab, layers, hidden, inter
        self.hq, self.hkv, self.head_dim = hq, hkv, head_dim
        self.eps, self.rope_theta = eps, rope_theta
        self.scale_embed, self.scale_lmhead, self.scale_residual = scale_embed, scale_lmhead, scale_residual
        self.dtype = dtype


class EagleOracleConfig:
    def __init__(self, num_iter=6, topk=10, tree_size=60, window=0, frspec_vocab=0, residual_scale=1.0,
                 use_input_norm=False, use_attn_norm=False, minicpm4_variant=False):
        self.num_iter, self.topk, self.tree_size = num_iter, topk, tree_size
        self.window, self.frspec_vocab, self.residual_scale = window, frspec_vocab, residual_scale
        self.use_input_norm, self.use_attn_norm = use_input_norm, use_attn_norm
        self.minicpm4_variant = minicpm4_variant


def default_inv_freq(head_dim, theta):
    """'default' rope initialiser of transformers (used by cpmcu/llm.py:184): theta^(-2i/d)."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def make_weights(cfg, seed, eagle=None, std=0.02, draft_from_last_layer=True, layer_scale=1.0, fc_mode="mix", fc_gain=1.0):
    """Seeded synthetic weights N(0, std) in the reference's checkpoint names
    (src/model/model.cuh:116-137; draft names without the 'eagle.' prefix as in
    an EAGLE checkpoint, src/model/minicpm4/minicpm4_eagle.cuh:187-221).

    layer_scale < 1 shrinks the decoder-layer matrices so that the next token is
    mostly a function of the current one; with fc_mode="embed" (fc = [gain*I | 0]) the
    drafter then predicts the target well and accepted paths get long.  Tests use
    this to exercise accept lengths > 1; the benchmark keeps layer_scale = 1."""
    g = torch.Generator().manual_seed(seed)
    H, I, d = cfg.hidden, cfg.inter, cfg.head_dim

    def rnd(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * std

    w = {"model.embed_tokens.weight": rnd(cfg.vocab, H), "lm_head.weight": rnd(cfg.vocab, H),
         "model.norm.weight": torch.ones(H)}
    for l in range(cfg.layers):
        p = "model.layers.%d." % l
        w[p + "self_attn.q_proj.weight"] = rnd(cfg.hq * d, H) * layer_scale
        w[p + "self_attn.k_proj.weight"] = rnd(cfg.hkv * d, H) * layer_scale
        w[p + "self_attn.v_proj.weight"] = rnd(cfg.hkv * d, H) * layer_scale
        w[p + "self_attn.o_proj.weight"] = rnd(H, cfg.hq * d) * layer_scale
        w[p + "mlp.gate_proj.weight"] = rnd(I, H) * layer_scale
        w[p + "mlp.up_proj.weight"] = rnd(I, H) * layer_scale
        w[p + "mlp.down_proj.weight"] = rnd(H, I) * layer_scale
        w[p + "input_layernorm.weight"] = torch.ones(H)
        w[p + "post_attention_layernorm.weight"] = torch.ones(H)
    ew = None
    if eagle is not None:
        ew = {}
        last = "model.layers.%d." % (cfg.layers - 1)
        for name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
                     "mlp.up_proj", "mlp.down_proj", "input_layernorm", "post_attention_layernorm"):
            src = w[last + name + ".weight"]
            ew["layers.0." + name + ".weight"] = src.clone() if draft_from_last_layer else rnd(*src.shape)
        # fc = [fc1 | fc2] over [embedding | hidden]; a small random mix keeps acceptance non-trivial
        if fc_mode == "embed":
            fc = torch.cat([torch.eye(H) * fc_gain, torch.zeros(H, H)], dim=1)
        else:
            fc = torch.cat([rnd(H, H), torch.eye(H) + rnd(H, H)], dim=1)
        ew["fc.weight"] = fc
        ew["fc.bias"] = torch.zeros(H)
        if eagle.use_input_norm:
            ew["input_norm1.weight"] = torch.ones(H)
            ew["input_norm2.weight"] = torch.ones(H)
    if cfg.dtype == "bf16":
        w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}
        if ew is not None:
            ew = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in ew.items()}
    return w, ew


class OracleModel:
    def __init__(self, cfg, weights, eagle=None, eagle_weights=None, budget=1024, token_id_remap=None, sparse=None):
        self.cfg, self.w = cfg, weights
        self.sparse = sparse  # oracle.sparse.SparseConfig: InfLLM-v2 block selection in the target layers
        self.eagle, self.ew = eagle, eagle_weights
        self.budget = budget
        self.inv_freq = default_inv_freq(cfg.head_dim, cfg.rope_theta)
        kvd = cfg.hkv * cfg.head_dim
        self.k_cache = torch.zeros(cfg.layers, budget, kvd)
        self.v_cache = torch.zeros(cfg.layers, budget, kvd)
        if eagle is not None:
            self.ek_cache = torch.zeros(budget, kvd)
            self.ev_cache = torch.zeros(budget, kvd)
            self.remap = None
            self.draft_head = weights["lm_head.weight"]
            if eagle.frspec_vocab and eagle.frspec_vocab != cfg.vocab:
                assert token_id_remap is not None
                self.remap = torch.as_tensor(np.asarray(token_id_remap), dtype=torch.long)
                self.draft_head = weights["lm_head.weight"][self.remap]  # remap_copy_kernel, tree_drafter.cuh:79-85
        self.trace = {}
        # tests may set this to a function (layer, own_mask) -> mask: the attention then uses the returned
        # block mask instead of the oracle's own selection (both are kept in trace["blockmask_pairs"])
        self.mask_override = None
        self._layer_index = 0

    # ---------------------------------------------------------------- primitives
    def rnd(self, x):
        return x.to(torch.bfloat16).to(torch.float32) if self.cfg.dtype == "bf16" else x

    def linear(self, x, w, bias=None):
        """src/model/linear.cuh:8-37 (+ batched_add of the bias, :83-85): fp32 accumulate, store T."""
        y = self.rnd(x @ w.t())
        if bias is not None:
            y = self.rnd(y + bias)
        return y

    def rms_norm(self, x, w):
        """src/model/norm.cuh:8-50."""
        rs = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.cfg.eps)
        return self.rnd(rs * x * w)

    def add(self, x, delta, scale=1.0):
        """elementwise_scale (skipped when 1) then add, each stored in T (src/model/elementwise.cuh:8-87)."""
        if scale != 1.0:
            delta = self.rnd(delta * scale)
        return self.rnd(x + delta)

    def rope(self, x, pos, nheads):
        """NeoX half-split rotary, src/model/rotary.cuh:7-34."""
        d = self.cfg.head_dim
        x = x.view(x.shape[0], nheads, d)
        freq = pos.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cos, sin = torch.cos(freq)[:, None, :], torch.sin(freq)[:, None, :]
        a, b = x[..., : d // 2], x[..., d // 2:]
        out = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
        return self.rnd(out).reshape(x.shape[0], nheads * d)

    def attention(self, q, k_cache, v_cache, kv_total, tq_valid, mask=None, mask_k=0, window=0, block_vis=None):
        """Visibility per src/flash_attn/src/mask.h:182-222 with the causal bound of
        flash_api.hpp:318-320: key c visible to row t iff c < kv_total - tq + t + 1 and,
        for the last mask_k keys, bit (c - (kv_total - mask_k)) of mask[t]."""
        cfg = self.cfg
        d, grp = cfg.head_dim, cfg.hq // cfg.hkv
        tq = q.shape[0]
        qh = q.view(tq, cfg.hq, d)
        K = k_cache[:kv_total].view(kv_total, cfg.hkv, d)
        V = v_cache[:kv_total].view(kv_total, cfg.hkv, d)
        cols = torch.arange(kv_total)
        vis = cols[None, :] < (kv_total - tq_valid + torch.arange(tq)[:, None] + 1)
        if mask is not None and mask_k > 0:
            mbeg = kv_total - mask_k
            bits = torch.zeros(tq, kv_total, dtype=torch.bool)
            for t in range(tq):
                m = int(mask[t])
                for c in range(mask_k):
                    bits[t, mbeg + c] = (m >> c) & 1
            vis = vis & ((cols[None, :] < mbeg) | bits)
        if window > 0:
            # block-granular left bound per 64-row query block (flash_blockmask.h:29-33 with the
            # loop_step_idx = m_block * 64 of flash_fwd_kernel.h:1517): key blocks of 128 below
            # ceil(q0 / 128) - window / 128 are skipped
            for blk in range(0, tq, 64):
                q0 = kv_total - tq_valid + blk
                lo_blk = (q0 + 127) // 128 - window // 128
                if lo_blk > 0:
                    vis[blk:blk + 64] = vis[blk:blk + 64] & (cols[None, :] >= lo_blk * 128)
        out = torch.zeros(tq, cfg.hq, d)
        scale = 1.0 / math.sqrt(d)
        for h in range(cfg.hq):
            s = (qh[:, h, :] @ K[:, h // grp, :].t()) * scale
            s = s.masked_fill(~(vis if block_vis is None else vis & block_vis[h // grp]), float("-inf"))
            p = torch.softmax(s, dim=-1)
            p = torch.nan_to_num(p, nan=0.0)
            out[:, h, :] = p @ V[:, h // grp, :]
        return self.rnd(out.reshape(tq, cfg.hq * d))

    # ---------------------------------------------------------------- decoder layer
    def layer(self, prefix, w, x, pending, pending_scale, res_scale, pos, k_cache, v_cache, kv_row0, kv_total,
              tq_valid, mask, mask_k, window, attn_norm=True, select=False):
        """Layer::decode / prefill (src/model/layer.cuh:47-89), Attention (attn.cuh:135-234), GatedFFN (ffn.cuh:72-90).
        Returns (x, pending_delta): the residual stream after the attention add, and the FFN output."""
        cfg = self.cfg
        rows = x.shape[0]
        if pending is not None:
            x = self.add(x, pending, pending_scale)
        normed = self.rms_norm(x, w[prefix + "input_layernorm.weight"]) if attn_norm else x
        q = self.linear(normed, w[prefix + "self_attn.q_proj.weight"])
        k = self.linear(normed, w[prefix + "self_attn.k_proj.weight"])
        v = self.linear(normed, w[prefix + "self_attn.v_proj.weight"])
        q = self.rope(q, pos, cfg.hq)
        k = self.rope(k, pos, cfg.hkv)
        nv = tq_valid if tq_valid is not None else rows
        k_cache[kv_row0:kv_row0 + nv] = k[:nv]
        v_cache[kv_row0:kv_row0 + nv] = v[:nv]
        block_vis = None
        if select and self.sparse is not None:
            # InfLLM-v2: kv_row0 is the layer's next_kv_length (rows accepted so far); the rows just appended
            # take no part in the selection (minicpm4_attn.cuh:96-166, :226-290)
            bm = osparse.select_blocks(self.sparse, q, k_cache, kv_row0, cfg.hq, cfg.hkv, cfg.head_dim, kv_total)
            if bm is not None:
                self.trace.setdefault("blockmask", []).append(bm)
                if self.mask_override is not None:
                    theirs = self.mask_override(self._layer_index, bm)
                    self.trace.setdefault("blockmask_pairs", []).append((bm, theirs))
                    bm = theirs
                block_vis = osparse.block_visibility(bm, self.sparse.block_window_size, rows, kv_total)
        a = self.attention(q, k_cache, v_cache, kv_total, nv, mask, mask_k, window, block_vis)
        o = self.linear(a, w[prefix + "self_attn.o_proj.weight"])
        x = self.add(x, o, res_scale)
        normed = self.rms_norm(x, w[prefix + "post_attention_layernorm.weight"])
        g = self.linear(normed, w[prefix + "mlp.gate_proj.weight"])
        u = self.linear(normed, w[prefix + "mlp.up_proj.weight"])
        act = self.rnd(g * torch.sigmoid(g) * u)  # gated_silu, src/model/activation.cuh:7-18
        down = self.linear(act, w[prefix + "mlp.down_proj.weight"])
        return x, down

    def embed(self, ids):
        e = self.w["model.embed_tokens.weight"][torch.as_tensor(ids, dtype=torch.long)]
        return self.rnd(e * self.cfg.scale_embed) if self.cfg.scale_embed != 1.0 else e

    def target_forward(self, ids, pos, kv_row0, kv_total, mask=None, mask_k=0):
        """ModelImpl::prefill_embed / decode_embed (src/model/model.cuh:139-165)."""
        cfg = self.cfg
        x = self.embed(ids)
        pos = torch.as_tensor(pos, dtype=torch.long)
        pending = None
        for l in range(cfg.layers):
            self._layer_index = l
            x, pending = self.layer("model.layers.%d." % l, self.w, x, pending, cfg.scale_residual, cfg.scale_residual,
                                    pos, self.k_cache[l], self.v_cache[l], kv_row0, kv_total, None, mask, mask_k, 0,
                                    select=True)
        x = self.add(x, pending, cfg.scale_residual)
        return self.rms_norm(x, self.w["model.norm.weight"])

    def lm_head(self, h, head=None, scale=True):
        if scale and self.cfg.scale_lmhead != 1.0:
            h = self.rnd(h * self.cfg.scale_lmhead)
        return self.linear(h, self.w["lm_head.weight"] if head is None else head)

    # ---------------------------------------------------------------- reference API
    def prefill(self, ids, history=0):
        """Single-chunk prefill (src/model/minicpm4/minicpm4_eagle.cuh:284-298, cpmcu/llm.py:189-261)."""
        n = len(ids)
        pos = np.arange(history, history + n)
        norm_out = self.target_forward(ids, pos, history, history + n)
        logits = self.lm_head(norm_out[-1:])
        if self.eagle is not None:
            self.prev_embed = torch.zeros(n, self.cfg.hidden)
            if n > 1:
                self.prev_embed[: n - 1] = self.embed(ids[1:])
            self.prev_hidden = norm_out.clone()
            self.eagle_pos = torch.as_tensor(pos, dtype=torch.long)
            self.num_prev, self.num_history, self.first_draft = n, history, True
        return logits[0]

    def prefill_chunked(self, ids, chunk):
        """cpmcu/llm.py:225-261: the prompt goes through prefill in chunks of `chunk` tokens; with a drafter
        the draft model's pass over a chunk is run when the next chunk (or the first draft) supplies the
        embedding of the token that follows it (src/model/eagle.cuh:405-434)."""
        logits = None
        for start in range(0, len(ids), chunk):
            logits = self.prefill_chunk(list(ids[start:start + chunk]), start)
        return logits

    def prefill_chunk(self, part, start):
        """One chunk of prefill_chunked: rows [start, start + len(part))."""
        if self.eagle is not None and start > 0:
            self.prev_embed[self.num_prev - 1] = self.embed([part[0]])[0]
            self._draft_core(self.prev_embed, self.prev_hidden, self.eagle_pos, self.num_history,
                             self.num_history + self.num_prev, None, None, 0)
        return self.prefill(part, history=start)

    def decode(self, ids, pos, cache_length, mask):
        """Tree verify forward (cpmcu/llm.py:263-283): KV rows written at [L, L+T)."""
        T = len(ids)
        norm_out = self.target_forward(ids, pos, cache_length, cache_length + T, mask, T if mask is not None else 0)
        self.norm_out = norm_out
        return self.lm_head(norm_out)

    def _draft_core(self, emb, hid, pos, kv_row0, kv_total, nv, mask, mask_k):
        e, ew, cfg = self.eagle, self.ew, self.cfg
        H = cfg.hidden
        if e.use_input_norm:
            emb = self.rms_norm(emb, ew["input_norm1.weight"])
            hid = self.rms_norm(hid, ew["input_norm2.weight"])
        # fc1 (embedding half, with bias) and fc2 (hidden half) are separate GEMMs in the reference,
        # each stored in T before the add (eagle.cuh:392-394, linear.cuh:83-85)
        y1 = self.linear(emb, ew["fc.weight"][:, :H], ew["fc.bias"])
        y2 = self.linear(hid, ew["fc.weight"][:, H:])
        x = self.rnd(y1 + y2)
        x, down = self.layer("layers.0.", ew, x, None, 1.0, e.residual_scale, pos, self.ek_cache, self.ev_cache,
                             kv_row0, kv_total, nv, mask, mask_k, e.window, attn_norm=e.use_attn_norm)
        return self.add(x, down, e.residual_scale)

    def draft(self, root_id, L):
        """EagleImpl::draft / MiniCPM4EagleImpl::draft (src/model/eagle.cuh:436-498,
        src/model/minicpm4/minicpm4_eagle.cuh:304-396)."""
        e, cfg = self.eagle, self.cfg
        k = e.topk
        if self.first_draft:
            self.prev_embed[self.num_prev - 1] = self.embed([root_id])[0]
            h = self._draft_core(self.prev_embed, self.prev_hidden, self.eagle_pos, self.num_history,
                                 self.num_history + self.num_prev, None, None, 0)
        else:
            n = self.num_prev
            h = self._draft_core(self.prev_embed[:n], self.prev_hidden[:n], self.eagle_pos[:n], L - n, L, None, None, 0)
        self.first_draft = False
        last = h[-1]
        scale = not e.minicpm4_variant
        tree = otree.DraftTree(k, e.num_iter, e.tree_size,
                               None if self.remap is None else self.remap.numpy())
        lp = otree.log_softmax_bf16(self.lm_head(last[None, :], self.draft_head, scale)[0].numpy()) \
            if cfg.dtype == "bf16" else torch.log_softmax(self.lm_head(last[None, :], self.draft_head, scale)[0], -1).numpy()
        tree.level0(lp)
        hid = last[None, :].repeat(k, 1)
        levels = [lp]
        for d in range(1, e.num_iter):
            emb = self.embed(tree.fr_id)
            pos = torch.full((k,), L + d - 1, dtype=torch.long)
            h = self._draft_core(emb, hid, pos, L + k * (d - 1), L + k * d, None, tree.fr_mask, k * d)
            logits = self.lm_head(h, self.draft_head, scale)
            if cfg.dtype == "bf16":
                lps = np.stack([otree.log_softmax_bf16(logits[r].numpy()) for r in range(k)])
            else:
                lps = torch.log_softmax(logits, -1).numpy()
            tree.level(d, lps)
            hid = h[torch.as_tensor(tree.fr_parent_row, dtype=torch.long)]
            levels.append(lps)
        ids, pos, mask, parent, sel = tree.finalize(L, root_id)
        self.trace = {"tree": tree, "sel": sel, "levels": levels}
        return ids, pos, mask, parent

    def verify_and_fix(self, tree_ids, gt, pos, L, mask, parent):
        """verify + fix-up (src/model/minicpm4/minicpm4_eagle.cuh:398-418)."""
        n, best, path = otree.verify(tree_ids, gt, pos, L, mask, parent)
        self.prev_hidden = self.norm_out[torch.as_tensor(path, dtype=torch.long)].clone()
        for l in range(self.cfg.layers):
            for cache in (self.k_cache[l], self.v_cache[l]):
                rows = cache[[L + p for p in path]].clone()
                cache[L:L + n] = rows
        out = otree.emitted_tokens(gt, path)
        self.prev_embed = self.embed(out)
        self.eagle_pos = torch.arange(L, L + n, dtype=torch.long)
        self.num_prev = n
        return n, out, path

    # ---------------------------------------------------------------- generate loops
    def generate_spec(self, prompt, num_tokens, chunk=None):
        """LLM_with_tree_drafter.generate, non-stream greedy path
        (cpmcu/speculative/tree_drafter.py:215-252).  Returns (tokens, accept_lengths, steps)."""
        P = len(prompt)
        logits = self.prefill(prompt) if chunk is None else self.prefill_chunked(prompt, chunk)
        root = int(torch.argmax(logits))
        tokens = [root]
        accept, steps = [], []
        i = 0
        while i < num_tokens - 1:
            L = P + i
            ids, pos, mask, parent = self.draft(root, L)
            logits = self.decode(ids, pos, L, mask)
            gt = torch.argmax(logits, dim=-1).numpy().astype(np.int32)
            n, out, path = self.verify_and_fix(ids, gt, pos, L, mask, parent)
            steps.append({"ids": ids, "pos": pos, "mask": mask, "parent": parent, "gt": gt, "n": n, "path": path,
                          "logits": logits})
            accept.append(n)
            tokens.extend(out[: min(n, num_tokens - 1 - i)])
            root = out[n - 1]
            i += n
        return tokens, accept, steps

    def teacher_forced_logits(self, prompt, tokens):
        """Target logits for every generated position in ONE causal pass over prompt + tokens[:-1]: row i is
        the distribution the token tokens[i] was (or should have been) picked from.  Greedy speculative decoding
        must reproduce greedy plain decoding (cpmcu/speculative/tree_drafter.py:215-252 accepts a drafted token
        only when it equals the target's argmax), so tokens[i] == argmax(row i) up to near-ties.  Dense target
        only; overwrites the KV caches."""
        assert self.sparse is None
        P = len(prompt)
        ids = list(prompt) + list(tokens[:-1])
        norm_out = self.target_forward(ids, np.arange(len(ids)), 0, len(ids))
        return self.lm_head(norm_out[P - 1:])

    def generate_plain(self, prompt, num_tokens):
        """Greedy decoding without speculation (cpmcu/llm.py:285-419, non-stream)."""
        P = len(prompt)
        logits = self.prefill(prompt)
        tok = int(torch.argmax(logits))
        tokens = [tok]
        for i in range(num_tokens - 1):
            L = P + i
            lg = self.decode([tok], [L], L, None)
            tok = int(torch.argmax(lg[0]))
            tokens.append(tok)
        return tokens
