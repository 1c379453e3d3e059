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
               token_id_remap=None, fused_step=True, budget=1024):
    """Returns (oracle_model, library_model) holding identical weights."""
    from cpmcu.speculative.eagle import LLM_with_eagle
    w, ew = make_weights(cfg, seed, eagle, layer_scale=layer_scale, fc_mode=fc_mode, fc_gain=fc_gain)
    oracle = OracleModel(cfg, w, eagle, ew, budget=budget, token_id_remap=token_id_remap)
    llm = LLM_with_eagle(None, None, num_iter=eagle.num_iter, topk_per_iter=eagle.topk, tree_size=eagle.tree_size,
                         eagle_window_size=eagle.window, frspec_vocab_size=eagle.frspec_vocab,
                         use_input_norm=eagle.use_input_norm, use_attn_norm=eagle.use_attn_norm,
                         eagle_config={"num_hidden_layers": 1}, config=hf_config(cfg), dtype=torch.bfloat16,
                         chunk_length=chunk_length, memory_limit=0.5, fused_step=fused_step)
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
