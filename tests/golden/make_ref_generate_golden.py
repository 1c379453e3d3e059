"""Records what the reference project's own CUDA build generates for the drop-in cases (tests/dropin_cases.py).

Needs a GPU and baseline/_ref/ (python -m oracle.build_ref --extension, from a reference checkout).  For every
case it writes the checkpoint directories, runs baseline/ref_cuda.py (the reference's LLM_with_eagle /
W4A16GPTQMarlinLLM_with_eagle: init_storage, load_from_hf, generate) in a process of its own and stores the token
stream and the accept lengths:

    python tests/golden/make_ref_generate_golden.py [OUT.json] [--only case,case]
                                                     (default: every case into tests/golden/ref_generate_golden.json;
                                                      --only records the named cases and keeps the others' entries)

tests/test_ref_generate_golden_cpu.py holds the CPU oracle against these vectors; tests/test_dropin_gpu.py holds
the library against them (and against the live reference when its build is in the tree)."""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import dropin_cases as dc  # noqa: E402


def run_reference(name, root):
    base_dir, eagle_dir, prompt = dc.write_case(name, root)
    prompt_file = os.path.join(root, name, "prompt.json")
    out_file = os.path.join(root, name, "out.json")
    with open(prompt_file, "w") as f:
        json.dump(prompt.tolist(), f)
    proc = subprocess.run(dc.reference_command(name, base_dir, eagle_dir, prompt_file, out_file), capture_output=True,
                          text=True, timeout=600)
    if proc.returncode != 0 or not os.path.exists(out_file):
        raise RuntimeError("reference run failed for %s:\n%s\n%s" % (name, proc.stdout[-2000:], proc.stderr[-2000:]))
    with open(out_file) as f:
        r = json.load(f)
    if "unavailable" in r:
        raise RuntimeError(r["unavailable"])
    return {"tokens": r["tokens"], "accept_lengths": r["accept_lengths"], "case": dc.CASES[name]}


def main():
    args = sys.argv[1:]
    only = None
    if "--only" in args:
        i = args.index("--only")
        only = args[i + 1].split(",")
        del args[i:i + 2]
    out = args[0] if args else os.path.join(HERE, "ref_generate_golden.json")
    gold = {}
    if only is not None and os.path.exists(out):
        with open(out) as f:
            gold = json.load(f)
    with tempfile.TemporaryDirectory() as root:
        for name in (only if only is not None else dc.CASES):
            try:
                gold[name] = run_reference(name, root)
                print(name, "tokens", len(gold[name]["tokens"]), "accept", gold[name]["accept_lengths"], flush=True)
            except Exception as e:  # record and go on: one unsupported case must not lose the others
                print(name, "FAILED:", str(e)[-1500:], flush=True)
    with open(out, "w") as f:
        json.dump(gold, f, indent=1)
    print("wrote", out)


if __name__ == "__main__":
    main()
