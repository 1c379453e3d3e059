"""Shared fixtures of the GPU parity tests: tiny seeded models loaded both into
the CPU oracle and, through the reference-shaped Python classes, into the
library."""
import types

import numpy as np
import torch

from oracle.model import EagleOracleConfig, OracleConfig, OracleModel, make_weights


def bf16_bits(t):
    return t.view(torch.int16)


def tiny_configs(which="a"):
    if which == "a":   # GQA ratio 2
        cfg = OracleConfig(vocab=4096, layers=2, hidden=256, inter=704, hq=2, hkv=1, head_dim=128, dtype="bf16")
    else:              # GQA ratio 4, more heads
        cfg = OracleConfig(vocab=5000, layers=3, hidden=512, inter=1024, hq=8, hkv=2, head_dim=128, dtype="bf16")
    return cfg


def hf_config(cfg):
    return types.SimpleNamespace(vocab_size=cfg.vocab, num_hidden_layers=cfg.layers, hidden_size=cfg.hidden,
                                 intermediate_size=cfg.inter, num_attention_heads=cfg.hq,
                                 num_key_value_heads=cfg.hkv, head_dim=cfg.head_dim, rms_norm_eps=cfg.eps,
                                 rope_theta=cfg.rope_theta, torch_dtype=torch.bfloat16)


def build_pair(cfg, eagle, seed=0, chunk_length=256, layer_scale=0.6, fc_mode="embed", fc_gain=200.0,
               token_id_remap=None, fused_step=True, budget=1024, sparse=None, qk_gain=1.0):
    """Returns (oracle_model, library_model) holding identical weights.  sparse: oracle.sparse.SparseConfig
    for an InfLLM-v2 target (the reference's apply_sparse=True)."""
    from cpmcu.speculative.eagle import LLM_with_eagle
    w, ew = make_weights(cfg, seed, eagle, layer_scale=layer_scale, fc_mode=fc_mode, fc_gain=fc_gain)
    if qk_gain != 1.0:
        # peaked attention: with flat attention every block scores alike and block selection is a coin toss
        for name in w:
            if "q_proj" in name or "k_proj" in name:
                w[name] = (w[name] * qk_gain).to(torch.bfloat16).float()
    oracle = OracleModel(cfg, w, eagle, ew, budget=budget, token_id_remap=token_id_remap, sparse=sparse)
    sparse_kw = {}
    if sparse is not None:
        sparse_kw = dict(apply_sparse=True, sink_window_size=sparse.sink_window_size,
                         block_window_size=sparse.block_window_size, sparse_topk_k=sparse.sparse_topk_k,
                         sparse_switch=sparse.sparse_switch, apply_compress_lse=sparse.apply_compress_lse)
    llm = LLM_with_eagle(None, None, num_iter=eagle.num_iter, topk_per_iter=eagle.topk, tree_size=eagle.tree_size,
                         eagle_window_size=eagle.window, frspec_vocab_size=eagle.frspec_vocab,
                         use_input_norm=eagle.use_input_norm, use_attn_norm=eagle.use_attn_norm,
                         eagle_config={"num_hidden_layers": 1}, config=hf_config(cfg), dtype=torch.bfloat16,
                         chunk_length=chunk_length, memory_limit=0.5, fused_step=fused_step, **sparse_kw)
    import os
    os.environ.setdefault("CPMCU_MAX_TOKENS", "4096")
    llm.init_storage()
    if token_id_remap is not None:
        llm._load("token_id_remap", torch.as_tensor(np.asarray(token_id_remap), dtype=torch.int32), cls="eagle")
    llm.load_state_dict_tensors({k: v.to(torch.bfloat16) for k, v in ew.items()}, cls="eagle")
    llm.load_state_dict_tensors({k: v.to(torch.bfloat16) for k, v in w.items()})
    return oracle, llm


def top2_gap(logits_row):
    v = torch.topk(logits_row.float(), 2).values
    return float(v[0] - v[1])


def bf16_step(x):
    """Spacing of bf16 numbers around x."""
    return 2.0 ** (np.floor(np.log2(max(abs(float(x)), 1e-30))) - 7)


# Near-tie rule of the token-stream comparisons: the two candidates are the top two logits of the row and
# lie within NEAR_TIE_STEPS bf16 steps of the top logit of each other.  Logits are stored in bf16, whose
# spacing at the usual logit magnitude (1..8) is 0.0078..0.03, so an absolute gap of 1e-3 cannot be told
# from a tie at all; this rule is the bf16 equivalent of "top-2 gap below resolution".
NEAR_TIE_STEPS = 2


def check_greedy_stream(oracle, prompt, tokens, what):
    """Every generated token must be the argmax of the oracle's target logits given the prompt and the tokens
    before it: greedy speculative decoding reproduces greedy plain decoding.  A different token is tolerated
    only at a near-tie AT THAT POSITION: it must be the runner-up and within NEAR_TIE_STEPS bf16 steps of the
    top logit.  Every position is judged given the stream's own prefix, so the check does not stop at the first
    tolerated tie.  Returns the tolerated ties as (position, gap)."""
    rows = oracle.teacher_forced_logits(list(prompt), list(tokens))
    ties = []
    for i, tok in enumerate(tokens):
        row = rows[i].float()
        best = int(torch.argmax(row))        # lowest index among equal maxima, as the reference's argmax
        if best == tok:
            continue
        masked = row.clone()
        masked[best] = float("-inf")
        second = int(torch.argmax(masked))
        gap = float(row[best] - row[second])
        ok = second == tok and gap <= NEAR_TIE_STEPS * bf16_step(float(row[best]))
        if not ok:
            raise AssertionError(f"{what}: token {i} is {tok}, oracle argmax {best} "
                                 f"(runner-up {second}, gap {gap:.4g}); stream so far {list(tokens[:i + 1])[-6:]}")
        ties.append((i, gap))
        print(f"{what}: tolerated near-tie at output {i}: gap {gap:.4g} between {best} and {tok}")
    return ties


def quantize_target(cfg, w):
    """W4A16 view of a target: returns (weights with the four linears replaced by their dequantised
    values, for the oracle) and the Marlin checkpoint tensors the reference converter would produce
    (fused qkv_proj / gate_up_proj, int32 qweight + bf16 scales)."""
    from oracle import marlin
    w = dict(w)
    ckpt = {}
    for l in range(cfg.layers):
        p = "model.layers.%d." % l
        groups = {"self_attn.qkv_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
                  "self_attn.o_proj": ["self_attn.o_proj"], "mlp.gate_up_proj": ["mlp.gate_proj", "mlp.up_proj"],
                  "mlp.down_proj": ["mlp.down_proj"]}
        for fused, parts in groups.items():
            full = torch.cat([w[p + n + ".weight"] for n in parts], dim=0)          # [N, K]
            q, s = marlin.quantize_sym_int4(full.t().contiguous().numpy())            # [K, N]
            packed, sperm = marlin.marlin_pack(q, s)
            deq = torch.from_numpy(marlin.dequantize(q, s)).t().contiguous()          # [N, K]
            row = 0
            for n in parts:
                rows = w[p + n + ".weight"].shape[0]
                w[p + n + ".weight"] = deq[row:row + rows].clone()
                row += rows
            ckpt[p + fused + ".qweight"] = torch.from_numpy(packed.copy())
            ckpt[p + fused + ".scales"] = torch.from_numpy(sperm.copy()).to(torch.bfloat16)
    for name in ("model.embed_tokens.weight", "lm_head.weight", "model.norm.weight"):
        ckpt[name] = w[name].to(torch.bfloat16)
    for l in range(cfg.layers):
        for n in ("input_layernorm", "post_attention_layernorm"):
            ckpt["model.layers.%d.%s.weight" % (l, n)] = w["model.layers.%d.%s.weight" % (l, n)].to(torch.bfloat16)
    return w, ckpt


def quantize_eagle(cfg, ew):
    """W4A16 view of a drafter: returns (weights with fc and the layer's linears replaced by their dequantised
    values, for the oracle) and the checkpoint tensors of a quantised drafter as the reference loads them:
    `layers.0.*` fused like a target layer, `fc.qweight` / `fc.scales` = the two [H -> H] halves (embedding half,
    hidden-state half) quantised separately and concatenated along the last dimension, `fc.bias` bf16
    (cpmcu/speculative/eagle_base_quant/eagle_base_w4a16_marlin_gptq.py:80-103)."""
    from oracle import marlin
    ew = dict(ew)
    ckpt = {}
    H = cfg.hidden

    def quant(full):                                   # full: [N, K] float
        q, s = marlin.quantize_sym_int4(full.t().contiguous().numpy())
        packed, sperm = marlin.marlin_pack(q, s)
        deq = torch.from_numpy(marlin.dequantize(q, s)).t().contiguous()
        return torch.from_numpy(packed.copy()), torch.from_numpy(sperm.copy()).to(torch.bfloat16), deq

    groups = {"self_attn.qkv_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
              "self_attn.o_proj": ["self_attn.o_proj"], "mlp.gate_up_proj": ["mlp.gate_proj", "mlp.up_proj"],
              "mlp.down_proj": ["mlp.down_proj"]}
    for fused, parts in groups.items():
        qw, sc, deq = quant(torch.cat([ew["layers.0." + n + ".weight"] for n in parts], dim=0))
        row = 0
        for n in parts:
            rows = ew["layers.0." + n + ".weight"].shape[0]
            ew["layers.0." + n + ".weight"] = deq[row:row + rows].clone()
            row += rows
        ckpt["layers.0." + fused + ".qweight"] = qw
        ckpt["layers.0." + fused + ".scales"] = sc
    q1, s1, d1 = quant(ew["fc.weight"][:, :H])
    q2, s2, d2 = quant(ew["fc.weight"][:, H:])
    ew["fc.weight"] = torch.cat([d1, d2], dim=1)
    ckpt["fc.qweight"] = torch.cat([q1, q2], dim=-1)
    ckpt["fc.scales"] = torch.cat([s1, s2], dim=-1)
    for name in ew:
        if "layernorm" in name or name in ("fc.bias", "input_norm1.weight", "input_norm2.weight"):
            ckpt[name] = ew[name].to(torch.bfloat16)
    return ew, ckpt


def build_quant_pair(cfg, eagle, seed=0, chunk_length=256, layer_scale=0.6, fc_gain=200.0, budget=1024, sparse=None,
                     quant_draft=False):
    from cpmcu.speculative.eagle_base_quant.eagle_base_w4a16_marlin_gptq import W4A16GPTQMarlinLLM_with_eagle
    import os
    w, ew = make_weights(cfg, seed, eagle, layer_scale=layer_scale, fc_mode="embed", fc_gain=fc_gain)
    wq, ckpt = quantize_target(cfg, w)
    eckpt = {k: v.to(torch.bfloat16) for k, v in ew.items()}
    econfig = {"num_hidden_layers": 1}
    extra = {}
    if quant_draft:
        ew, eckpt = quantize_eagle(cfg, ew)
        econfig["quantization_config"] = {"group_size": 128, "bits": 4}
        extra = dict(apply_eagle_quant=True, use_input_norm=eagle.use_input_norm, use_attn_norm=eagle.use_attn_norm)
    oracle = OracleModel(cfg, wq, eagle, ew, budget=budget, sparse=sparse)
    hf = hf_config(cfg)
    hf.quantization_config = {"group_size": 128, "bits": 4}
    sparse_kw = {}
    if sparse is not None:
        sparse_kw = dict(apply_sparse=True, sink_window_size=sparse.sink_window_size,
                         block_window_size=sparse.block_window_size, sparse_topk_k=sparse.sparse_topk_k,
                         sparse_switch=sparse.sparse_switch, apply_compress_lse=sparse.apply_compress_lse)
    llm = W4A16GPTQMarlinLLM_with_eagle(None, None, num_iter=eagle.num_iter, topk_per_iter=eagle.topk,
                                        tree_size=eagle.tree_size, eagle_config=econfig, config=hf,
                                        dtype=torch.bfloat16, chunk_length=chunk_length, memory_limit=0.5, **sparse_kw,
                                        **extra)
    os.environ.setdefault("CPMCU_MAX_TOKENS", "4096")
    llm.init_storage()
    llm.load_state_dict_tensors(eckpt, cls="eagle")
    llm.load_state_dict_tensors(ckpt)
    return oracle, llm
