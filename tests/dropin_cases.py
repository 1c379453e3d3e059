"""Tiny seeded models as on-disk checkpoints (Hugging Face style directories written by baseline/synth_ckpt.py):
the cases that the drop-in tests feed, unchanged, to the reference project's own CUDA build and to this library,
and from which tests/golden/make_ref_generate_golden.py records what the reference generated."""
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle.model import EagleOracleConfig, OracleConfig, OracleModel, make_weights  # noqa: E402

CFGS = {
    "a": dict(vocab=4096, layers=2, hidden=256, inter=704, hq=2, hkv=1, head_dim=128),
    # the reference builds o_proj as Linear(hidden, hq * head_dim) like q_proj (src/model/attn.cuh:84-88), so it
    # only works when hq * head_dim == hidden: every case keeps that
    "c": dict(vocab=5000, layers=3, hidden=1024, inter=1536, hq=8, hkv=2, head_dim=128),
    "q": dict(vocab=4096, layers=2, hidden=256, inter=768, hq=2, hkv=1, head_dim=128),
}

# The reference takes the FR-Spec vocabulary and the draft window only on its MiniCPM4 drafter, which it picks when
# one of the norm switches is on (cpmcu/speculative/eagle.py:52-74); those cases therefore carry input norms.
CASES = {
    "plain": dict(cfg="a", eagle=dict(num_iter=4, topk=4, tree_size=16), seed=2, prompt=130, gen=40,
                  layer_scale=0.6, fc_gain=200.0, chunk=256),
    "norms": dict(cfg="c", eagle=dict(num_iter=3, topk=5, tree_size=12, use_input_norm=True, use_attn_norm=True,
                                      minicpm4_variant=True), seed=2, prompt=130, gen=40, layer_scale=0.3, fc_gain=8.0,
                  chunk=256),
    "frspec": dict(cfg="a", eagle=dict(num_iter=3, topk=4, tree_size=12, frspec_vocab=1024, use_input_norm=True,
                                       minicpm4_variant=True), seed=4, prompt=100, gen=24, layer_scale=0.6,
                   fc_gain=200.0, chunk=256),
    "window": dict(cfg="a", eagle=dict(num_iter=3, topk=4, tree_size=12, window=128, use_input_norm=True,
                                       minicpm4_variant=True), seed=6, prompt=400, gen=24, layer_scale=0.6,
                   fc_gain=200.0, chunk=512),
    "quant": dict(cfg="q", eagle=dict(num_iter=4, topk=4, tree_size=16), seed=8, prompt=120, gen=30, layer_scale=0.6,
                  fc_gain=200.0, chunk=256, quant=True),
    "quant_draft": dict(cfg="q", eagle=dict(num_iter=4, topk=4, tree_size=16, minicpm4_variant=True), seed=13, prompt=120,
                        gen=36, layer_scale=0.6, fc_gain=200.0, chunk=256, quant=True, quant_draft=True),
    # muP-scaled checkpoints (MiniCPM style: scale_emb, dim_model_base -> LM-head input scale, scale_depth -> residual
    # scale).  The plain drafter scales its LM-head input like the target; the MiniCPM4 drafter does not
    # (src/model/minicpm4/minicpm4_eagle.cuh:26,95-99 holds the head as a plain Linear) and scales its residual.
    "mup_plain": dict(cfg="a", eagle=dict(num_iter=4, topk=4, tree_size=16), seed=15, prompt=110, gen=36, layer_scale=0.6,
                      fc_gain=40.0, chunk=256, mup=dict(scale_emb=6.0, dim_model_base=128, scale_depth=1.2)),
    "mup_minicpm4": dict(cfg="c", eagle=dict(num_iter=3, topk=5, tree_size=12, use_input_norm=True, use_attn_norm=True,
                                             minicpm4_variant=True), seed=16, prompt=110, gen=36, layer_scale=0.3,
                         fc_gain=8.0, chunk=256, mup=dict(scale_emb=6.0, dim_model_base=512, scale_depth=1.4)),
    "headline_tree": dict(cfg="c", eagle=dict(num_iter=6, topk=10, tree_size=60), seed=12, prompt=300, gen=48,
                          layer_scale=0.3, fc_gain=8.0, chunk=512),
    # a prompt of two prefill chunks, the first of 13 token tiles: the prefill-sized schedules (whole GEMM tiles in
    # waves, the SwiGLU epilogue, causal attention over thousands of keys) and the drafter's deferred pass over the
    # previous chunk, against the reference build's own chunked prefill
    "long_prompt": dict(cfg="c", eagle=dict(num_iter=4, topk=6, tree_size=24), seed=21, prompt=3400, gen=32,
                        layer_scale=0.3, fc_gain=8.0, chunk=3328, max_tokens=8192),
}


def oracle_chunk(name):
    """The chunk length to hand the oracle's generate_spec: None for a prompt of one chunk."""
    c = CASES[name]
    return c["chunk"] if c["prompt"] > c["chunk"] else None


def case_parts(name):
    """(OracleConfig, EagleOracleConfig, weights, eagle weights, remap or None, prompt ids) of a case."""
    c = CASES[name]
    shape = CFGS[c["cfg"]]
    mup = c.get("mup")
    scales, eagle_kw = {}, dict(c["eagle"])
    if mup:
        # the constructors' arithmetic, cpmcu/llm.py:63-67 and cpmcu/speculative/eagle.py:43
        scales = dict(scale_embed=mup["scale_emb"], scale_lmhead=mup["dim_model_base"] / shape["hidden"],
                      scale_residual=mup["scale_depth"] / math.sqrt(shape["layers"]))
        if eagle_kw.get("minicpm4_variant"):
            eagle_kw["residual_scale"] = mup["scale_depth"] / math.sqrt(shape["layers"] + 1)
    cfg = OracleConfig(dtype="bf16", **shape, **scales)
    eagle = EagleOracleConfig(**eagle_kw)
    w, ew = make_weights(cfg, c["seed"], eagle, layer_scale=c["layer_scale"], fc_mode="embed", fc_gain=c["fc_gain"])
    remap = None
    if eagle.frspec_vocab:
        rng = np.random.default_rng(7)
        counts = np.bincount(rng.zipf(1.1, 200000) % cfg.vocab, minlength=cfg.vocab)
        remap = np.lexsort((np.arange(cfg.vocab), -counts))[:eagle.frspec_vocab].astype(np.int32)
    prompt = np.random.default_rng(c["seed"]).integers(0, cfg.vocab, c["prompt"]).astype(np.int32)
    return cfg, eagle, w, ew, remap, prompt


def make_oracle(name, budget=1024):
    """A fresh CPU oracle holding the case's weights (for a quantised case: the dequantised weights)."""
    cfg, eagle, w, ew, remap, prompt = case_parts(name)
    if CASES[name].get("quant"):
        from helpers import quantize_target
        w, _ = quantize_target(cfg, w)
    if CASES[name].get("quant_draft"):
        from helpers import quantize_eagle
        ew, _ = quantize_eagle(cfg, ew)
    budget = max(budget, CASES[name].get("max_tokens", 0))
    return OracleModel(cfg, w, eagle, ew, budget=budget, token_id_remap=remap), prompt


def write_case(name, root):
    """Writes the case's checkpoint under `root`; returns (base_dir, eagle_dir, prompt ids)."""
    from baseline import synth_ckpt
    c = CASES[name]
    cfg, eagle, w, ew, remap, prompt = case_parts(name)
    extra = None
    if c.get("quant"):
        from helpers import quantize_target
        _, tensors = quantize_target(cfg, w)
        extra = {"quantization_config": {"group_size": 128, "bits": 4}}
    else:
        tensors = {k: v.to(torch.bfloat16) for k, v in w.items()}
    etensors = {k: v.to(torch.bfloat16) for k, v in ew.items()}
    eagle_config = None
    if c.get("quant_draft"):
        from helpers import quantize_eagle
        _, etensors = quantize_eagle(cfg, ew)
        eagle_config = {"quantization_config": {"group_size": 128, "bits": 4}}
    if remap is not None:
        etensors["token_id_remap"] = torch.from_numpy(remap)
    if c.get("mup"):
        extra = dict(extra or {}, **c["mup"])
    config = synth_ckpt.base_config(cfg.vocab, cfg.layers, cfg.hidden, cfg.inter, cfg.hq, cfg.hkv, cfg.head_dim, cfg.eps,
                                    cfg.rope_theta, extra)
    base_dir, eagle_dir = os.path.join(root, name, "base"), os.path.join(root, name, "eagle")
    synth_ckpt.write_checkpoint(base_dir, eagle_dir, config, tensors.items(), etensors.items(), eagle_config)
    return base_dir, eagle_dir, prompt


def reference_command(name, base_dir, eagle_dir, prompt_file, out_file, memory_limit=0.04):
    """Command line of baseline/ref_cuda.py for the case (the reference's own build and Python classes)."""
    c = CASES[name]
    e = c["eagle"]
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "ref_cuda.py"), "--base", base_dir, "--eagle", eagle_dir,
           "--prompt", prompt_file, "--gen", str(c["gen"]), "--repeat", "0", "--chunk", str(c["chunk"]),
           "--num-iter", str(e["num_iter"]), "--topk", str(e["topk"]), "--tree", str(e["tree_size"]),
           "--memory-limit", str(memory_limit), "--out", out_file]
    if e.get("use_input_norm"):
        cmd.append("--input-norm")
    if e.get("use_attn_norm"):
        cmd.append("--attn-norm")
    if e.get("frspec_vocab"):
        cmd += ["--frspec", str(e["frspec_vocab"])]
    if e.get("window"):
        cmd += ["--window", str(e["window"])]
    if c.get("quant"):
        cmd.append("--quant")
    if c.get("quant_draft"):
        cmd.append("--eagle-quant")
    return cmd
