"""Drop-in evidence: the SAME checkpoint directories (config.json, tokenizer, safetensors) go through the
reference's own construction sequence on both sides,

    LLM_with_eagle(eagle_dir, base_dir, ...) -> init_storage() -> load_from_hf() -> generate(ids, n, teminators=[])

(tests/test_generate.py:217-260 of the reference builds its model this way), once with this library's classes and
once with the reference project's own CUDA build (baseline/_ref/, run in a process of its own by
baseline/ref_cuda.py).  The two token streams are each judged by the CPU oracle's teacher-forced target logits
(helpers.check_greedy_stream) and compared with each other; where the reference build is not in the tree, its
recorded output (tests/golden/ref_generate_golden.json) stands in."""
import json
import os
import subprocess
import sys

import pytest
import torch

import dropin_cases as dc
from helpers import check_greedy_stream

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD_FILE = os.path.join(HERE, "golden", "ref_generate_golden.json")


def reference_live(name, base_dir, eagle_dir, prompt, root):
    sys.path.insert(0, dc.ROOT)
    from baseline import ref_cuda
    if ref_cuda.available() is None:
        return None
    prompt_file, out_file = os.path.join(root, "prompt.json"), os.path.join(root, "out.json")
    with open(prompt_file, "w") as f:
        json.dump(prompt.tolist(), f)
    proc = subprocess.run(dc.reference_command(name, base_dir, eagle_dir, prompt_file, out_file), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0 and os.path.exists(out_file), "reference run failed:\n" + proc.stderr[-2000:]
    with open(out_file) as f:
        return json.load(f)


def library_generate(name, base_dir, eagle_dir, prompt, stream=False):
    from cpmcu.speculative.eagle import LLM_with_eagle
    from cpmcu.speculative.eagle_base_quant.eagle_base_w4a16_marlin_gptq import W4A16GPTQMarlinLLM_with_eagle
    import cpmcu.C as C
    c = dc.CASES[name]
    e = c["eagle"]
    cls = W4A16GPTQMarlinLLM_with_eagle if c.get("quant") else LLM_with_eagle
    os.environ["CPMCU_MAX_TOKENS"] = str(c.get("max_tokens", 4096))
    llm = cls(eagle_dir, base_dir, num_iter=e["num_iter"], topk_per_iter=e["topk"], tree_size=e["tree_size"],
              eagle_window_size=e.get("window", 0), frspec_vocab_size=e.get("frspec_vocab", 0),
              use_input_norm=e.get("use_input_norm", False), use_attn_norm=e.get("use_attn_norm", False),
              apply_eagle_quant=bool(c.get("quant_draft")), dtype=torch.bfloat16, memory_limit=0.3, chunk_length=c["chunk"], cuda_graph=True)
    assert llm.tokenizer is not None and llm.config.vocab_size == dc.CFGS[c["cfg"]]["vocab"]
    llm.init_storage()
    llm.load_from_hf()
    ids = torch.tensor(prompt, device="cuda")
    if stream:
        out = list(llm.generate(ids, c["gen"], teminators=[], use_stream=True))
        assert all(set(d) >= {"token", "text", "is_finished", "accept_length", "prefill_time", "decode_time"} for d in out)
        assert out[-1]["is_finished"] and not any(d["is_finished"] for d in out[:-1])
        # the reference's consumer (tests/test_generate.py:365-404) collects accept_length > 0 as one entry per step
        # and takes the last decode_time > 0 as the total: the first token reports 1, then only a step's first token
        # reports the step's accept length and only its last token a decode time
        tokens = [d["token"] for d in out]
        acc = [d["accept_length"] for d in out if d["accept_length"] > 0]
        assert acc[0] == 1 and sum(acc[1:]) >= len(tokens) - 1 and out[0]["prefill_time"] > 0
        assert all(d["prefill_time"] == 0.0 for d in out[1:]) and out[-1]["decode_time"] >= 0
        acc = acc[1:]
    else:
        tokens, acc, decode_s, prefill_s = llm.generate(ids, c["gen"], teminators=[])
        assert decode_s > 0 and prefill_s > 0
    C.release()
    return tokens, acc


@pytest.mark.parametrize("name", sorted(dc.CASES))
def test_same_checkpoint_through_load_from_hf_matches_reference(name, tmp_path):
    base_dir, eagle_dir, prompt = dc.write_case(name, str(tmp_path))
    tokens, acc = library_generate(name, base_dir, eagle_dir, prompt)
    assert len(tokens) == dc.CASES[name]["gen"]
    judge, _ = dc.make_oracle(name)
    ties = check_greedy_stream(judge, prompt, tokens, name + ": library")
    ref = reference_live(name, base_dir, eagle_dir, prompt, str(tmp_path))
    source = "live reference build"
    if ref is None:
        if not os.path.exists(GOLD_FILE):
            pytest.skip("neither the reference build nor its recorded output is in the tree")
        gold = json.load(open(GOLD_FILE))
        if name not in gold:
            pytest.skip("no recorded reference output for this case")
        ref, source = {"tokens": gold[name]["tokens"], "accept_lengths": gold[name]["accept_lengths"]}, "recorded reference output"
    r_tokens = ref["tokens"][: len(tokens)]
    judge2, _ = dc.make_oracle(name)
    r_ties = check_greedy_stream(judge2, prompt, r_tokens, name + ": reference")
    if not ties and not r_ties:
        assert tokens[: len(r_tokens)] == r_tokens, f"{name}: no near-tie on either side, yet the streams differ"
        print(f"BRANCH {name}: identical to the {source} ({len(r_tokens)} tokens); accept lengths "
              f"{'equal' if acc == ref['accept_lengths'] else 'differ: %s vs %s' % (acc, ref['accept_lengths'])}")
    else:
        print(f"BRANCH {name}: near-ties tolerated (library {ties}, reference {r_ties}) against the {source}")
    # the speculation itself must be doing work in both
    assert max(acc) > 1 and max(ref["accept_lengths"]) > 1


def test_stream_mode_yields_the_same_tokens(tmp_path):
    name = "plain"
    base_dir, eagle_dir, prompt = dc.write_case(name, str(tmp_path))
    tokens, acc = library_generate(name, base_dir, eagle_dir, prompt)
    s_tokens, s_acc = library_generate(name, base_dir, eagle_dir, prompt, stream=True)
    assert s_tokens == tokens
    assert s_acc == acc      # one accept length per step, as the non-stream call returns them


def test_minicpm4_yarn_is_refused(tmp_path):
    from cpmcu.llm import LLM
    base_dir, eagle_dir, prompt = dc.write_case("plain", str(tmp_path))
    with pytest.raises(NotImplementedError):
        LLM(base_dir, dtype=torch.bfloat16, minicpm4_yarn=True)


def test_generation_longer_than_the_cache_is_refused(tmp_path):
    """Every pass checks on the host that the K/V rows it appends fit the budget, before anything is launched."""
    import cpmcu.C as C
    from cpmcu.speculative.eagle import LLM_with_eagle
    name = "plain"
    base_dir, eagle_dir, prompt = dc.write_case(name, str(tmp_path))
    os.environ["CPMCU_MAX_TOKENS"] = "256"
    try:
        llm = LLM_with_eagle(eagle_dir, base_dir, num_iter=4, topk_per_iter=4, tree_size=16, dtype=torch.bfloat16,
                             memory_limit=0.3, chunk_length=256)
        llm.init_storage()
        assert llm.max_total_length == 256
        llm.load_from_hf()
        ids = torch.tensor(prompt, device="cuda")          # 130 tokens
        with pytest.raises(ValueError):
            llm.generate(ids, 200, teminators=[])           # 130 + 200 + 16 > 256
        # below the Python check: drive the C ABI to the edge of the cache
        pos = torch.arange(len(prompt), dtype=torch.int32, device="cuda")
        logits = llm.prefill(ids, pos)
        C.begin_generation(len(prompt), int(logits[0].argmax()))
        emitted = 0
        with pytest.raises(RuntimeError, match="cache holds 256 rows"):
            for _ in range(200):
                emitted += len(C.spec_step(16))
        assert len(prompt) + emitted + 16 > 256 and len(prompt) + emitted <= 256
    finally:
        os.environ["CPMCU_MAX_TOKENS"] = "4096"
        C.release()
