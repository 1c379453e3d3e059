"""Benchmark of the speculative-decoding step (draft -> tree -> verify -> accept).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload configN] [--no-extras]

Headline workload (BASELINE.json configs[1]): MiniCPM4-8B-shaped bf16 target (32 layers, hidden 4096,
32 q / 2 kv heads, head_dim 128, FFN 16384, vocab 73448), random N(0, 0.02) weights (seed 1), 1-layer EAGLE
drafter copied from the target's last layer, tree of 60 nodes (6 iterations, top-k 10), a 4096-token
Zipf(1.1) prompt, batch 1, greedy.  A "step" is one speculative step.  Synthetic data throughout.

Ours: `value` = tokens emitted by the K timed steps / their summed device time (CUDA events around each
captured step, inputs resident in HBM); `e2e` = the same K steps timed by the host clock around the public
`C.spec_step()` calls, which includes the per-step device->host read of the accepted tokens.  The line also
carries the verify half of the step in microseconds (an event node inside the captured step) with its
roofline fraction, and at N = 1 (unless --no-extras): the other BASELINE.json configurations (`workloads`),
an acceptance-bearing weight recipe (`accepting`), the reference project's own CUDA build run on the same
GPU through its own Python API (`reference_cuda`, when baseline/_ref/ holds it) and the CPU oracle
(`cpu_baseline`).  With N > 1 every rank runs an independent replica on its own GPU (no collective on the
data path); value = all ranks' tokens / the slowest rank's time, and a config-5 pass is added.

--impl reference: the reference has no CPU implementation of this path, so this arm times the CPU oracle
(oracle/, a restatement of the reference's step) on the host cores; each of its steps is one bounded sample
of the speculative step (one target layer, the LM head, one draft level), scaled by the op counts.
"""
import argparse
import contextlib
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "cpm.cu_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

CFG = dict(vocab=73448, layers=32, hidden=4096, inter=16384, hq=32, hkv=2, head_dim=128, eps=1e-5, rope_theta=10000.0)
TREE = dict(num_iter=6, topk=10, tree_size=60)
PROMPT_LEN = 4096
LONG_PROMPT_LEN = 32768   # config 5
LONG_CHUNK = 2048         # the reference's default chunk_length: the first chunk is dense, later ones select blocks
FRSPEC_VOCAB = 32768      # config 3
METRIC = "spec_decode_tokens_per_s"
UNIT = "tokens/s"

WORKLOADS = {
    "config2": dict(index=1, w4a16=False, sparse=False, frspec=False,
                    text="configs[1]: 8B-shaped bf16 target + 1-layer EAGLE, tree 60 (6 iters x top-10), "),
    "config3": dict(index=2, w4a16=False, sparse=False, frspec=True,
                    text="configs[2]: config 2 with FR-Spec (draft LM head over the 32768 most frequent ids; drafter input "
                         "norms on, as the reference's FR-Spec path requires), "),
    "config4": dict(index=3, w4a16=True, sparse=False, frspec=False,
                    text="configs[3]: config-2 architecture with W4A16 GPTQ-Marlin target linears (random int4 tensors), "
                         "bf16 embeddings / LM head / EAGLE draft, tree 60, "),
    "config5": dict(index=4, w4a16=False, sparse=True, frspec=False,
                    text="configs[4]: config-2 architecture with InfLLM-v2 block-sparse target attention (block 64, "
                         "top-64 + 1 initial block + 2048-token window), draft window 1024 (drafter input norms on, as the "
                         "reference's windowed drafter requires), chunked prefill (2048), tree 60, "),
}
# Second weight recipe (not a BASELINE.json configuration): decoder-layer matrices shrunk by ACCEPT_LAYER_SCALE and
# fc = [gain * I | 0], so that the next token is mostly a function of the current one and the 1-layer drafter can
# follow the 32-layer target; exercises accept lengths > 1 (catch-up over several rows, compaction, gathers).
ACCEPT_LAYER_SCALE = float(os.environ.get("CPMCU_BENCH_LAYER_SCALE", "0.05"))
ACCEPT_FC_GAIN = float(os.environ.get("CPMCU_BENCH_FC_GAIN", "50"))


def zipf_prompt(n, vocab, seed, s=1.1):
    import numpy as np
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    p /= p.sum()
    return rng.choice(vocab, size=n, p=p).astype(np.int32)


def frspec_remap(seed):
    """FR-Spec vocabulary: the 32768 most frequent ids of a seeded Zipf(1.1) sample of 1M tokens, in order of
    descending count, ties by id."""
    import numpy as np
    counts = np.bincount(zipf_prompt(1_000_000, CFG["vocab"], seed + 1000), minlength=CFG["vocab"])
    return np.lexsort((np.arange(CFG["vocab"]), -counts))[:FRSPEC_VOCAB].astype(np.int32)


def algorithmic_bytes(w4a16=False, draft_vocab=None):
    """Weight bytes one speculative step has to stream: every target linear once (M = 60), the draft
    fc + layer + LM head six times.  bf16 weights are 2 bytes; W4A16 target linears are half a byte per
    weight plus one bf16 scale per 128."""
    H, I, V = CFG["hidden"], CFG["inter"], CFG["vocab"]
    qkv = (CFG["hq"] + 2 * CFG["hkv"]) * CFG["head_dim"]
    layer = qkv * H + H * CFG["hq"] * CFG["head_dim"] + 2 * I * H + H * I
    per_weight = (0.5 + 2.0 / 128) if w4a16 else 2.0
    target = int(CFG["layers"] * layer * per_weight) + V * H * 2
    draft_pass = (2 * H * H + layer + (draft_vocab or V) * H) * 2
    return target, TREE["num_iter"] * draft_pass


def verify_bytes(w4a16, context):
    """Bytes the verify half has to move: target weights once, the K/V rows of the context read once per layer,
    the tree's 60 K/V rows written, the 60 x vocab logits written."""
    tgt, _ = algorithmic_bytes(w4a16)
    kv_row = CFG["hkv"] * CFG["head_dim"] * 2 * 2
    return tgt + CFG["layers"] * (context + 2 * TREE["tree_size"]) * kv_row + TREE["tree_size"] * CFG["vocab"] * 2


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[3 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


# ---------------------------------------------------------------------------- synthetic weights
def iter_weights(seed=1, w4a16=False, frspec=False, accepting=False, input_norm=False):
    """Yields (cls, name, tensor) with cls None (target) or "eagle", tensors on the GPU, in an order both
    loaders accept (token_id_remap before lm_head).  Headline recipe: N(0, 0.02) everywhere, drafter = the
    target's last layer with fc passing the hidden state through (fc1 = 0, fc2 = I, bias 0).  config 4: the
    target's linears as random GPTQ-Marlin int4 tensors (any bit pattern is a valid weight).  accepting: see
    ACCEPT_LAYER_SCALE above."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    H, I, d = CFG["hidden"], CFG["inter"], CFG["head_dim"]
    ls = ACCEPT_LAYER_SCALE if accepting else 1.0

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device="cuda", generator=g, dtype=torch.float32) * (0.02 * scale)).to(torch.bfloat16)

    ones = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    if frspec:
        yield "eagle", "token_id_remap", torch.from_numpy(frspec_remap(seed)).to("cuda")
    yield None, "model.embed_tokens.weight", rnd(CFG["vocab"], H)
    yield None, "lm_head.weight", rnd(CFG["vocab"], H)
    yield None, "model.norm.weight", ones
    last = {}
    for l in range(CFG["layers"]):
        p = "model.layers.%d." % l
        is_last = l == CFG["layers"] - 1
        if w4a16:
            for fused, (K, N) in {"self_attn.qkv_proj": (H, (CFG["hq"] + 2 * CFG["hkv"]) * d),
                                  "self_attn.o_proj": (CFG["hq"] * d, H), "mlp.gate_up_proj": (H, 2 * I),
                                  "mlp.down_proj": (I, H)}.items():
                qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 16, 2 * N), device="cuda", generator=g, dtype=torch.int64)
                sc = (torch.rand(K // 128, N, device="cuda", generator=g) * 0.002 + 0.0065).to(torch.bfloat16)
                yield None, p + fused + ".qweight", qw.to(torch.int32)
                yield None, p + fused + ".scales", sc
        if not w4a16 or is_last:
            tensors = {"self_attn.q_proj": rnd(CFG["hq"] * d, H, scale=ls), "self_attn.k_proj": rnd(CFG["hkv"] * d, H, scale=ls),
                       "self_attn.v_proj": rnd(CFG["hkv"] * d, H, scale=ls), "self_attn.o_proj": rnd(H, CFG["hq"] * d, scale=ls),
                       "mlp.gate_proj": rnd(I, H, scale=ls), "mlp.up_proj": rnd(I, H, scale=ls),
                       "mlp.down_proj": rnd(H, I, scale=ls)}
            if not w4a16:
                for name, t in tensors.items():
                    yield None, p + name + ".weight", t
            if is_last:
                last = tensors
        yield None, p + "input_layernorm.weight", ones
        yield None, p + "post_attention_layernorm.weight", ones
    for name, t in last.items():
        yield "eagle", "layers.0." + name + ".weight", t
    yield "eagle", "layers.0.input_layernorm.weight", ones
    yield "eagle", "layers.0.post_attention_layernorm.weight", ones
    eye = torch.eye(H, device="cuda")
    if accepting:
        fc = torch.cat([eye * ACCEPT_FC_GAIN, torch.zeros(H, H, device="cuda")], dim=1)
    else:
        fc = torch.cat([torch.zeros(H, H, device="cuda"), eye], dim=1)
    yield "eagle", "fc.weight", fc.to(torch.bfloat16)
    yield "eagle", "fc.bias", torch.zeros(H, device="cuda", dtype=torch.bfloat16)
    if frspec or input_norm:
        # the reference takes an FR-Spec vocabulary or a draft window only on its MiniCPM4 drafter, which it picks when a
        # norm switch is on (cpmcu/speculative/eagle.py:52-74): configs 3 and 5 run with input norms (weights of ones)
        # on both arms
        yield "eagle", "input_norm1.weight", ones
        yield "eagle", "input_norm2.weight", ones


def hf_config_dict(w4a16):
    from baseline.synth_ckpt import base_config
    extra = {"quantization_config": {"group_size": 128, "bits": 4}} if w4a16 else None
    return base_config(CFG["vocab"], CFG["layers"], CFG["hidden"], CFG["inter"], CFG["hq"], CFG["hkv"], CFG["head_dim"],
                       CFG["eps"], CFG["rope_theta"], extra)


# ---------------------------------------------------------------------------- ours
def build_model(device_index, seed=1, w4a16=False, sparse=False, frspec=False, accepting=False):
    """Random-init model generated on the GPU tensor by tensor and loaded through the reference-shaped Python
    classes (C.load_model accepts device pointers)."""
    import types

    import torch
    from cpmcu.speculative.eagle import LLM_with_eagle
    from cpmcu.speculative.eagle_base_quant.eagle_base_w4a16_marlin_gptq import W4A16GPTQMarlinLLM_with_eagle
    torch.cuda.set_device(device_index)
    os.environ["CPMCU_MAX_TOKENS"] = "40960" if sparse else "8192"
    hf = types.SimpleNamespace(vocab_size=CFG["vocab"], num_hidden_layers=CFG["layers"], hidden_size=CFG["hidden"],
                               intermediate_size=CFG["inter"], num_attention_heads=CFG["hq"],
                               num_key_value_heads=CFG["hkv"], head_dim=CFG["head_dim"], rms_norm_eps=CFG["eps"],
                               rope_theta=CFG["rope_theta"], torch_dtype=torch.bfloat16)
    if w4a16:
        hf.quantization_config = {"group_size": 128, "bits": 4}
    cls = W4A16GPTQMarlinLLM_with_eagle if w4a16 else LLM_with_eagle
    extra = {}
    if sparse:
        # config 5: InfLLM-v2 target (block 64, top-64 blocks + 1 initial block + local window of 2048 tokens),
        # draft layer with a sliding window of 1024 tokens
        extra = dict(apply_sparse=True, sink_window_size=1, block_window_size=32, sparse_topk_k=64, sparse_switch=8192,
                     apply_compress_lse=True, eagle_window_size=1024, use_input_norm=True)
    if frspec:
        extra["frspec_vocab_size"] = FRSPEC_VOCAB
        extra["use_input_norm"] = True
    llm = cls(None, None, num_iter=TREE["num_iter"], topk_per_iter=TREE["topk"],
              tree_size=TREE["tree_size"], eagle_config={"num_hidden_layers": 1}, config=hf,
              dtype=torch.bfloat16, chunk_length=LONG_CHUNK if sparse else PROMPT_LEN, memory_limit=0.8,
              fused_step=True, **extra)
    llm.init_storage()
    for kind, name, t in iter_weights(seed, w4a16, frspec, accepting, input_norm=sparse):
        llm._load(name, t, cls=kind)
    llm._load("model.rotary_emb.inv_freq", llm._rope_inv_freq(), dtype=torch.float32)
    torch.cuda.empty_cache()
    return llm


def measure(llm, prompt_len, seed, steps, warmup, local, barrier=None, profile=True):
    """Prefill + `warmup` untimed + `steps` timed speculative steps.  Returns a dict of raw measurements."""
    import torch
    import cpmcu.C as C
    prompt = torch.tensor(zipf_prompt(prompt_len, CFG["vocab"], seed), device="cuda")
    pos = torch.arange(prompt_len, dtype=torch.int32, device="cuda")
    # prefill as the reference's demo measures it: one warm-up pass, then the better of two (each pass rebuilds the
    # whole context from position 0; the generation below continues from the last one)
    prefill_runs = []
    for _ in range(3):
        torch.cuda.synchronize()
        t0 = time.time()
        logits = llm.prefill(prompt, pos)
        torch.cuda.synchronize()
        prefill_runs.append(time.time() - t0)
    prefill_s = min(prefill_runs[1:])
    C.begin_generation(prompt_len, int(logits[0].argmax()))
    for _ in range(warmup):
        C.spec_step(16)
    sampler = ClockSampler(local)
    sampler.start()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    tokens, dev_ms, draft_ms, verify_ms, accept = 0, [], [], [], []
    for _ in range(steps):
        out = C.spec_step(16)
        tokens += len(out)
        accept.append(len(out))
        dev_ms.append(C.last_step_ms())
        d, v = C.last_step_split_ms()
        draft_ms.append(d)
        verify_ms.append(v)
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if barrier is not None:
        barrier()
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    res = dict(tokens=tokens, dev_ms=dev_ms, draft_ms=draft_ms, verify_ms=verify_ms, accept=accept, wall=wall,
               prefill_s=prefill_s, prefill_first_s=prefill_runs[0], launches=int(C.launches_per_step()), clocks=sampler.summary(),
               context=prompt_len + sum(accept) // 2)
    if profile:
        # per-class device time of a few uncaptured steps (CUDA events around every launch)
        lin_ms, att_ms, sel_ms, lin_n, prof_total = [], [], [], 0, []
        for _ in range(3):
            cls, total = C.profile_step()
            lin_ms.append(cls["linear"][0])
            att_ms.append(cls["attention"][0])
            sel_ms.append(cls["selection"][0])
            lin_n = cls["linear"][1]
            prof_total.append(total)
        res["profile"] = {"total": statistics.median(prof_total), "linear": statistics.median(lin_ms),
                          "attention": statistics.median(att_ms), "block_selection": statistics.median(sel_ms),
                          "linear_launches": lin_n}
    return res


def hbm_peak():
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    return float(peaks.get("hbm_gbs", 6650.0)), ("measured" if "hbm_gbs" in peaks else "fallback")


def summarise(res, workload, peak):
    """Small per-workload record (the `workloads` / `accepting` entries of the line)."""
    w = WORKLOADS[workload]
    tgt_b, draft_b = algorithmic_bytes(w["w4a16"], FRSPEC_VOCAB if w["frspec"] else None)
    step_ms = statistics.median(res["dev_ms"])
    verify_us = 1e3 * statistics.median(res["verify_ms"])
    out = {"tokens_per_s": res["tokens"] / (sum(res["dev_ms"]) / 1e3), "ms_per_step": step_ms,
           "steps": len(res["dev_ms"]), "mean_accept_length": statistics.mean(res["accept"]),
           "max_accept_length": max(res["accept"]), "launches_per_step": res["launches"],
           "step_roofline_frac": ((tgt_b + draft_b) / 1e9 / peak) / (step_ms / 1e3),
           "verify_step_us": verify_us, "draft_us": 1e3 * statistics.median(res["draft_ms"]),
           "verify_roofline_frac": (verify_bytes(w["w4a16"], res["context"]) / 1e9 / peak) / (verify_us / 1e6),
           "prefill_tokens_per_s": (LONG_PROMPT_LEN if w["sparse"] else PROMPT_LEN) / res["prefill_s"],
           "clocks": res["clocks"]}
    if "profile" in res:
        out["linear_roofline_frac"] = ((tgt_b + draft_b) / 1e9 / (res["profile"]["linear"] / 1e3)) / peak
    return out


def run_reference_cuda(workload, gen_tokens=256, timeout_s=900, cuda_graph=True):
    """The reference project's own CUDA build on this GPU (baseline B1): writes the workload's synthetic
    checkpoint as safetensors + config.json, runs baseline/ref_cuda.py in a process of its own (the reference's
    LLM_with_eagle: init_storage, load_from_hf, generate with cuda_graph=True, one chunk), and returns what its
    generate() reported.  Call it while this process holds no model on the GPU."""
    import torch
    from baseline import ref_cuda, synth_ckpt
    if ref_cuda.available() is None:
        return {"build": "unavailable", "reason": "baseline/_ref/cpmcu/C*.so not in the tree (python -m oracle.build_ref "
                                                  "--extension builds it from a reference checkout)"}
    w = WORKLOADS[workload]
    t0 = time.time()
    root = None
    for cand in ("/dev/shm", tempfile.gettempdir()):
        try:
            if os.path.isdir(cand) and shutil.disk_usage(cand).free > 24e9:
                root = tempfile.mkdtemp(prefix="cpmcu_ckpt_", dir=cand)
                break
        except OSError:
            pass
    if root is None:
        return {"build": "ok", "run": "skipped", "reason": "no scratch space for a 17 GB checkpoint"}
    try:
        base_dir, eagle_dir = os.path.join(root, "base"), os.path.join(root, "eagle")
        gen = list_split(iter_weights(1, w["w4a16"], w["frspec"], False, input_norm=w["sparse"]))
        synth_ckpt.write_checkpoint(base_dir, eagle_dir, hf_config_dict(w["w4a16"]), gen[0], gen[1])
        torch.cuda.empty_cache()
        prompt_len = LONG_PROMPT_LEN if w["sparse"] else PROMPT_LEN
        with open(os.path.join(root, "prompt.json"), "w") as f:
            json.dump(zipf_prompt(prompt_len, CFG["vocab"], 100).tolist(), f)
        write_s = time.time() - t0
        cmd = [sys.executable, os.path.join(ROOT, "baseline", "ref_cuda.py"), "--base", base_dir, "--eagle", eagle_dir,
               "--prompt", os.path.join(root, "prompt.json"), "--gen", str(gen_tokens), "--repeat", "2",
               "--memory-limit", "0.5", "--out", os.path.join(root, "out.json"),
               "--chunk", str(LONG_CHUNK if w["sparse"] else PROMPT_LEN)]
        if w["w4a16"]:
            cmd.append("--quant")
        if w["frspec"]:
            cmd += ["--frspec", str(FRSPEC_VOCAB), "--input-norm"]
        if w["sparse"]:
            cmd += ["--sparse", "--window", "1024", "--input-norm"]   # the draft window needs the MiniCPM4 drafter
        if not cuda_graph:
            cmd.append("--no-graph")
        env = dict(os.environ)
        env.pop("CPMCU_MAX_TOKENS", None)
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=env)
        out_file = os.path.join(root, "out.json")
        if proc.returncode != 0 or not os.path.exists(out_file):
            return {"build": "ok", "run": "failed", "returncode": proc.returncode,
                    "stderr_tail": proc.stderr[-1500:], "stdout_tail": proc.stdout[-500:]}
        with open(out_file) as f:
            r = json.load(f)
        return {"build": "ok", "run": "ok", "tokens_per_s": r["tokens_per_s"], "ms_per_step": r["ms_per_step"],
                "mean_accept_length": r["mean_accept_length"], "prefill_tokens_per_s": r["prefill_tokens_per_s"],
                "runs_tokens_per_s": r["runs_tokens_per_s"], "generated": len(r["tokens"]), "cuda_graph": r["cuda_graph"],
                "first_tokens": r["tokens"][:16], "checkpoint_write_s": write_s, "total_s": time.time() - t0,
                "what": "reference LLM_with_eagle.generate(): len(tokens) / decode wall time between two "
                        "torch.cuda.synchronize() calls, its own definition (tests/test_generate.py:440-444); best of 2 "
                        "runs after one warm-up run; same synthetic weights and prompt as this line's `value`"}
    except subprocess.TimeoutExpired:
        return {"build": "ok", "run": "failed", "reason": "timed out after %d s" % timeout_s}
    finally:
        shutil.rmtree(root, ignore_errors=True)


def list_split(events):
    """Two lazy streams (target tensors, drafter tensors) out of iter_weights; the checkpoint writer consumes the
    target stream first, so the drafter's tensors (a few of them, produced at the end) are buffered."""
    base, eagle = [], []

    def base_iter():
        for kind, name, t in events:
            if kind is None:
                yield name, t
            else:
                eagle.append((name, t.to("cpu")))

    def eagle_iter():
        for item in eagle:
            yield item
    return base_iter(), eagle_iter()


def run_ours(args):
    import torch
    import cpmcu.C as C
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    C.load()  # fails loudly if the CUDA library is missing
    from cpmcu.replicas import combine_ranks, replica_seed
    w = WORKLOADS[args.workload]
    prompt_len = LONG_PROMPT_LEN if w["sparse"] else PROMPT_LEN
    with contextlib.redirect_stdout(sys.stderr):  # keep stdout for the single JSON line
        llm = build_model(local, seed=1, w4a16=w["w4a16"], sparse=w["sparse"], frspec=w["frspec"])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    res = measure(llm, prompt_len, replica_seed(100, rank), args.steps, args.warmup, local, barrier)
    dev_s = sum(res["dev_ms"]) / 1e3
    tokens_all, dev_max, wall_max = combine_ranks(res["tokens"], dev_s, res["wall"], dist, "cuda")
    peak, peak_src = hbm_peak()
    line = None
    if rank == 0:
        tgt_b, draft_b = algorithmic_bytes(w["w4a16"], FRSPEC_VOCAB if w["frspec"] else None)
        prof = res["profile"]
        achieved = (tgt_b + draft_b) / 1e9 / (prof["linear"] / 1e3)
        summ = summarise(res, args.workload, peak)
        line = {
            "metric": METRIC, "value": tokens_all / dev_max, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dev_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["text"] + "%d-token Zipf(1.1) prompt, batch 1, greedy" % prompt_len,
                       "replicas": world,
                       "l2": "inputs larger than L2 (%.1f GB of weights streamed per step)" % ((tgt_b + draft_b) / 1e9)},
            "e2e": {"value": tokens_all / wall_max, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 128,
                    "note": "host clock around C.spec_step(), the call a user makes per step, including its 128-byte "
                            "device-to-host read of (accept length, tokens); a step has no host input (root token and "
                            "lengths are device state; the prompt is copied once before prefill)"},
            "gpu_launches": res["launches"] * args.steps,
            "launches_per_step": res["launches"],
            "mean_accept_length": statistics.mean(res["accept"]),
            "step_device_ms_median": statistics.median(res["dev_ms"]),
            # verify half of the captured step (target tree forward + argmax + acceptance + compaction), split off
            # by an event node inside the graph; median over the timed steps
            "verify_step_us": summ["verify_step_us"], "draft_us": summ["draft_us"],
            "verify_roofline_frac": summ["verify_roofline_frac"],
            "verify_bytes": verify_bytes(w["w4a16"], res["context"]),
            "prefill_tokens_per_s": prompt_len / res["prefill_s"],
            "profile_eager_step_ms": prof,
            "roofline": {"bound": "hbm", "kernel": "linear_umma_kernel + linear_umma_cluster_kernel%s (all %d launches of a step)"
                                                   % (" + linear_w4_umma_kernel" if w["w4a16"] else "", prof["linear_launches"]),
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src,
                         # DRAM bytes of the step's linear launches: algorithmic bytes x the ratio one ncu capture
                         # of the gate/up GEMM gave (269.5 MB read + 5.3 MB written for 268.9 MB algorithmic;
                         # W4A16: 69.8 + 1.5 MB for 69.7 MB), see profiles/
                         "traffic": int((tgt_b + draft_b) * (1.023 if w["w4a16"] else 1.022)),
                         "traffic_source": "scaled from one ncu capture of the gate/up GEMM",
                         "algorithmic_bytes_per_step": tgt_b + draft_b},
            "step_roofline_frac": summ["step_roofline_frac"],
            "clocks": res["clocks"],
        }
    C.release()
    del llm
    torch.cuda.empty_cache()

    extras = not args.no_extras and args.workload == "config2"
    if extras and world > 1:
        # replica curve of the long-context workload (BASELINE.json configs[4]): every rank one config-5 replica
        with contextlib.redirect_stdout(sys.stderr):
            llm = build_model(local, seed=1, sparse=True)
        r5 = measure(llm, LONG_PROMPT_LEN, replica_seed(100, rank), args.extra_steps, 3, local, barrier, profile=False)
        t5, d5, w5 = combine_ranks(r5["tokens"], sum(r5["dev_ms"]) / 1e3, r5["wall"], dist, "cuda")
        if rank == 0:
            s5 = summarise(r5, "config5", peak)
            s5.update({"tokens_per_s": t5 / d5, "e2e_tokens_per_s": t5 / w5, "replicas": world})
            line["workloads"] = {"config5": s5}
        C.release()
        del llm
        torch.cuda.empty_cache()
    if extras and world == 1:
        line["workloads"] = {}
        for name in ("config3", "config4", "config5"):
            ww = WORKLOADS[name]
            try:
                with contextlib.redirect_stdout(sys.stderr):
                    llm = build_model(local, seed=1, w4a16=ww["w4a16"], sparse=ww["sparse"], frspec=ww["frspec"])
                r = measure(llm, LONG_PROMPT_LEN if ww["sparse"] else PROMPT_LEN, 100, args.extra_steps, 3, local)
                line["workloads"][name] = summarise(r, name, peak)
            except Exception as e:  # keep the headline line even if an extra fails
                line["workloads"][name] = {"error": repr(e)[:300]}
            C.release()
            llm = None
            torch.cuda.empty_cache()
        try:
            with contextlib.redirect_stdout(sys.stderr):
                llm = build_model(local, seed=1, accepting=True)
            r = measure(llm, PROMPT_LEN, 100, args.extra_steps, 3, local, profile=False)
            acc = summarise(r, "config2", peak)
            acc["recipe"] = ("config-2 shapes; decoder-layer matrices scaled by %g, fc = [%g * I | 0]: the next token is "
                             "mostly a function of the current one, so the drafter lands tokens" % (ACCEPT_LAYER_SCALE, ACCEPT_FC_GAIN))
            line["accepting"] = acc
        except Exception as e:
            line["accepting"] = {"error": repr(e)[:300]}
        C.release()
        llm = None
        torch.cuda.empty_cache()
        try:
            ref = run_reference_cuda("config2")
        except Exception as e:
            ref = {"build": "ok", "run": "failed", "reason": repr(e)[:300]}
        line["reference_cuda"] = ref
        if ref.get("run") == "ok":
            line["speedup_vs_reference_cuda"] = {"e2e": line["e2e"]["value"] / ref["tokens_per_s"],
                                                 "target": 2.0, "met": line["e2e"]["value"] / ref["tokens_per_s"] >= 2.0}
        if not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_step_baseline(line["mean_accept_length"])
            except Exception as e:
                line["cpu_baseline"] = {"error": repr(e)[:300]}
    elif rank == 0 and world == 1 and not args.no_cpu_baseline and not args.no_extras:
        line["cpu_baseline"] = cpu_step_baseline(line["mean_accept_length"])
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------- CPU oracle arm
class CpuSample:
    """One bounded sample of the speculative step on the host cores with the CPU oracle: one target layer at
    M = 60 over a 4096-token KV cache, the target LM head at M = 60, one draft level (fc + layer at M = 10 + LM
    head + log-softmax/top-k).  A whole step = 32 layers + head + 6 draft levels."""

    def __init__(self):
        import torch
        from oracle.model import EagleOracleConfig, OracleConfig, OracleModel
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        cfg = OracleConfig(vocab=CFG["vocab"], layers=1, hidden=CFG["hidden"], inter=CFG["inter"], hq=CFG["hq"],
                           hkv=CFG["hkv"], head_dim=CFG["head_dim"], dtype="bf16")
        eagle = EagleOracleConfig(**TREE)
        g = torch.Generator().manual_seed(1)
        H, I, d, V = CFG["hidden"], CFG["inter"], CFG["head_dim"], CFG["vocab"]

        def rnd(*shape):
            return (torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16).to(torch.float32)

        p = "model.layers.0."
        w = {"model.embed_tokens.weight": rnd(1024, H), "lm_head.weight": rnd(V, H), "model.norm.weight": torch.ones(H),
             p + "self_attn.q_proj.weight": rnd(CFG["hq"] * d, H), p + "self_attn.k_proj.weight": rnd(CFG["hkv"] * d, H),
             p + "self_attn.v_proj.weight": rnd(CFG["hkv"] * d, H), p + "self_attn.o_proj.weight": rnd(H, CFG["hq"] * d),
             p + "mlp.gate_proj.weight": rnd(I, H), p + "mlp.up_proj.weight": rnd(I, H), p + "mlp.down_proj.weight": rnd(H, I),
             p + "input_layernorm.weight": torch.ones(H), p + "post_attention_layernorm.weight": torch.ones(H)}
        ew = {k.replace("model.layers.0.", "layers.0."): v for k, v in w.items() if k.startswith(p)}
        ew["fc.weight"] = torch.cat([torch.zeros(H, H), torch.eye(H)], dim=1)
        ew["fc.bias"] = torch.zeros(H)
        self.L, self.T, self.k = PROMPT_LEN, TREE["tree_size"], TREE["topk"]
        m = OracleModel(cfg, w, eagle, ew, budget=self.L + 128)
        for c in (m.k_cache, m.v_cache, m.ek_cache, m.ev_cache):
            c.normal_(generator=g)
        self.m, self.w, self.p = m, w, p
        self.x = rnd(self.T, H) * 50
        self.xd = rnd(self.k, H) * 50
        self.masks = [(1 << i) | 1 for i in range(self.T)]
        self.pos = torch.full((self.T,), self.L, dtype=torch.long)

    def run(self):
        """Returns (layer_s, head_s, draft_level_s) of one sample."""
        from oracle import tree as otree
        m, L, T, k = self.m, self.L, self.T, self.k
        t0 = time.perf_counter()
        m.layer(self.p, self.w, self.x, None, 1.0, 1.0, self.pos, m.k_cache[0], m.v_cache[0], L, L + T, None, self.masks, T, 0)
        t1 = time.perf_counter()
        m.lm_head(self.x)
        t2 = time.perf_counter()
        h = m._draft_core(self.xd, self.xd, self.pos[:k], L, L + k, None, [(1 << i) for i in range(k)], k)
        lg = m.lm_head(h, m.draft_head, True)
        for r in range(k):
            otree.topk_desc(otree.log_softmax_bf16(lg[r].numpy()), k)
        t3 = time.perf_counter()
        return t1 - t0, t2 - t1, t3 - t2

    @staticmethod
    def step_seconds(parts):
        return CFG["layers"] * parts[0] + parts[1] + TREE["num_iter"] * parts[2]


def cpu_step_baseline(mean_accept, budget_s=20.0):
    """The CPU oracle on the host cores over a bounded number of samples (about budget_s seconds of CPU work),
    scaled to a whole step by the op counts."""
    t_start = time.perf_counter()
    s = CpuSample()
    s.run()
    parts = []
    while time.perf_counter() - t_start < budget_s or len(parts) < 3:
        parts.append(s.run())
    med = [statistics.median(p[i] for p in parts) for i in range(3)]
    step_s = CpuSample.step_seconds(med)
    return {"value": mean_accept / step_s, "unit": UNIT, "cores": s.cores, "kind": "port, sampled",
            "step_seconds_extrapolated": step_s, "samples": len(parts),
            "sample": "%d samples of: 1 of 32 target layers at M=60 over a 4096-token KV (%.3f s), target LM head at M=60 "
                      "(%.3f s), 1 of 6 draft levels incl. log-softmax/top-k (%.3f s); step = 32 layers + head + 6 levels; "
                      "%.0f s of CPU work" % (len(parts), med[0], med[1], med[2], time.perf_counter() - t_start)}


def run_reference(args):
    """CPU arm: W untimed + K timed samples (see CpuSample); `ms_per_step` is what one timed sample took, `value`
    the tokens/s of a whole step extrapolated from the median sample at accept length 1 (what the random-weight
    headline configuration yields)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = CpuSample()
    steps = min(args.steps, 64)
    for _ in range(min(args.warmup, 3)):
        s.run()
    parts = []
    t0 = time.perf_counter()
    for _ in range(steps):
        parts.append(s.run())
    wall = time.perf_counter() - t0
    med = [statistics.median(p[i] for p in parts) for i in range(3)]
    step_s = CpuSample.step_seconds(med)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    base = {"value": 1.0 / step_s, "unit": UNIT, "cores": s.cores, "kind": "port, sampled",
            "step_seconds_extrapolated": step_s,
            "sample": "each timed step = 1 of 32 target layers at M=60 over a 4096-token KV (%.3f s) + target LM head "
                      "(%.3f s) + 1 of 6 draft levels (%.3f s); value = 1 / (32 layers + head + 6 levels)" % tuple(med)}
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
            "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": 1e3 * wall / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOADS["config2"]["text"] + "4096-token context, batch 1, greedy; CPU oracle of the "
                                   "reference step, sampled"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference has no CPU implementation of this path; this arm times the CPU restatement (oracle/) "
                    "on the host cores.  ms_per_step is the wall time of one timed SAMPLE (a fraction of a step); the "
                    "whole-step time is step_seconds_extrapolated.  The reference's own CUDA build, run on the GPU, is "
                    "reported by the default arm as `reference_cuda`."}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement (no other workloads, no reference CUDA run, no CPU baseline)")
    ap.add_argument("--extra-steps", type=int, default=48, help="timed steps of each extra workload")
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS),
                    help="config2 = the headline bf16 workload; config3 = the same with an FR-Spec draft vocabulary of 32768; "
                         "config4 = the same with a W4A16 GPTQ-Marlin target; config5 = 32768-token prompt, InfLLM-v2 "
                         "sparse target, draft window 1024")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
