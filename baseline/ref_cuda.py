"""Runs the reference project's own CUDA build (baseline/_ref/, produced by `python -m oracle.build_ref
--extension` from a reference checkout) through its own public API, in a process of its own:

    LLM_with_eagle / W4A16GPTQMarlinLLM_with_eagle(eagle_dir, base_dir, ...)  ->  init_storage()
    ->  load_from_hf()  ->  generate(prompt, n, teminators=[])

on a checkpoint directory written by baseline/synth_ckpt.py, and prints one JSON line with what `generate`
returned (tokens, accept lengths, its own decode and prefill wall times: decode tokens/s as the reference's
demo computes it, tests/test_generate.py:440-444).  Nothing of this repository's library is imported here.

    python baseline/ref_cuda.py --base DIR --eagle DIR --prompt FILE.json --gen N [--quant] [--sparse]
                                [--eagle-quant] [--frspec V] [--window W] [--chunk C] [--no-graph] [--repeat R] [--out FILE]

BENCHMARK / TEST INFRASTRUCTURE.  One environment shim, applied in this process only and not to the reference's
files: the installed `transformers` no longer lists a "default" entry in ROPE_INIT_FUNCTIONS, which the
reference's load_from_hf looks up (cpmcu/llm.py:178-184); the entry is put back with the standard
theta^(-2i/d) formula.
"""
import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available():
    """The path of the built reference extension, or None."""
    import glob
    hits = glob.glob(os.path.join(REF_DIR, "cpmcu", "C*.so"))
    return hits[0] if hits else None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base", required=True)
    ap.add_argument("--eagle", required=True)
    ap.add_argument("--prompt", required=True, help="JSON file holding the list of prompt token ids")
    ap.add_argument("--gen", type=int, default=256)
    ap.add_argument("--repeat", type=int, default=1, help="timed generate() calls after one warm-up call")
    ap.add_argument("--quant", action="store_true", help="W4A16 GPTQ-Marlin target")
    ap.add_argument("--sparse", action="store_true", help="InfLLM-v2 target (apply_sparse=True)")
    ap.add_argument("--sparse-topk", type=int, default=64)
    ap.add_argument("--sparse-switch", type=int, default=8192)
    ap.add_argument("--block-window", type=int, default=32)
    ap.add_argument("--no-compress-lse", action="store_true")
    ap.add_argument("--frspec", type=int, default=0)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--num-iter", type=int, default=6)
    ap.add_argument("--topk", type=int, default=10)
    ap.add_argument("--tree", type=int, default=60)
    ap.add_argument("--memory-limit", type=float, default=0.8)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--input-norm", action="store_true")
    ap.add_argument("--attn-norm", action="store_true")
    ap.add_argument("--eagle-quant", action="store_true", help="W4A16 drafter (apply_eagle_quant=True)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    if available() is None:
        print(json.dumps({"unavailable": "reference CUDA extension not built (baseline/_ref/cpmcu/C*.so missing)"}))
        return
    sys.path.insert(0, REF_DIR)
    import torch
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    if "default" not in ROPE_INIT_FUNCTIONS:
        def default_rope(config, device=None, seq_len=None, **kw):
            scaling = getattr(config, "rope_scaling", None) or {}
            theta = scaling.get("rope_theta", getattr(config, "rope_theta", None) or 10000.0)
            d = config.head_dim
            return 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d)), 1.0
        ROPE_INIT_FUNCTIONS["default"] = default_rope

    if args.quant:
        from cpmcu.speculative.eagle_base_quant.eagle_base_w4a16_marlin_gptq import W4A16GPTQMarlinLLM_with_eagle as Cls
    else:
        from cpmcu.speculative.eagle import LLM_with_eagle as Cls
    kw = dict(num_iter=args.num_iter, topk_per_iter=args.topk, tree_size=args.tree, eagle_window_size=args.window,
              frspec_vocab_size=args.frspec, use_input_norm=args.input_norm, use_attn_norm=args.attn_norm,
              apply_eagle_quant=args.eagle_quant,
              dtype=torch.bfloat16, memory_limit=args.memory_limit, chunk_length=args.chunk,
              cuda_graph=not args.no_graph)
    if args.sparse:
        kw.update(apply_sparse=True, sink_window_size=1, block_window_size=args.block_window,
                  sparse_topk_k=args.sparse_topk, sparse_switch=args.sparse_switch,
                  apply_compress_lse=not args.no_compress_lse)
    t0 = time.time()
    llm = Cls(args.eagle, args.base, **kw)
    llm.init_storage()
    llm.load_from_hf()
    torch.cuda.synchronize()
    load_s = time.time() - t0
    with open(args.prompt) as f:
        prompt = torch.tensor(json.load(f), dtype=torch.int32, device="cuda")
    runs = []
    for r in range(args.repeat + 1):
        tokens, accept, decode_s, prefill_s = llm.generate(prompt, args.gen, teminators=[])
        if r == 0 and args.repeat > 0:
            continue   # warm-up: first graph capture, lazy module loading
        runs.append({"tokens": tokens, "accept_lengths": accept, "decode_s": decode_s, "prefill_s": prefill_s})
    best = min(runs, key=lambda x: x["decode_s"] / max(len(x["tokens"]), 1))
    out = {"impl": "reference_cuda", "tokens": best["tokens"], "accept_lengths": best["accept_lengths"],
           "decode_s": best["decode_s"], "prefill_s": best["prefill_s"], "load_s": load_s,
           "tokens_per_s": len(best["tokens"]) / best["decode_s"],
           "ms_per_step": 1e3 * best["decode_s"] / max(len(best["accept_lengths"]), 1),
           "mean_accept_length": sum(best["accept_lengths"]) / max(len(best["accept_lengths"]), 1),
           "prefill_tokens_per_s": prompt.numel() / best["prefill_s"],
           "runs_tokens_per_s": [len(x["tokens"]) / x["decode_s"] for x in runs],
           "cuda_graph": not args.no_graph, "max_total_length": llm.max_total_length}
    line = json.dumps(out)
    if args.out:
        with open(args.out, "w") as f:
            f.write(line)
    print(line, flush=True)


if __name__ == "__main__":
    main()
