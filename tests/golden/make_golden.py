"""Regenerates tests/golden/*.json from the CPU oracle (run from the repo root:
`python tests/golden/make_golden.py`).  The reference has no vectors of its own
for this path, so these fixtures pin the oracle against regressions only."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import tree as otree  # noqa: E402
from oracle.model import EagleOracleConfig, OracleConfig, OracleModel, make_weights  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def tree_case(seed, V, k, num_iter, T, coarse):
    g = torch.Generator().manual_seed(seed)
    rows = 1 + (num_iter - 1) * k
    logits = torch.randn(rows, V, generator=g) * 3.0
    if coarse:
        logits = torch.round(logits * 2) / 2
    lf = logits.to(torch.bfloat16).float().numpy()
    tree = otree.DraftTree(k, num_iter, T)
    tree.level0(otree.log_softmax_bf16(lf[0]))
    for d in range(1, num_iter):
        tree.level(d, np.stack([otree.log_softmax_bf16(r) for r in lf[1 + (d - 1) * k: 1 + d * k]]))
    ids, pos, mask, par, sel = tree.finalize(100, 7)
    return {"seed": seed, "V": V, "k": k, "num_iter": num_iter, "T": T, "coarse": coarse, "cache_length": 100,
            "root": 7, "ids": ids.tolist(), "pos": pos.tolist(), "mask": [int(m) for m in mask],
            "parent": par.tolist(), "sel": sel.tolist()}


def verify_case(seed, T):
    rng = np.random.default_rng(seed)
    L = 40
    parent, masks, depth = [0] * T, [1] * T, [1] * T
    for i in range(1, T):
        while True:
            p = int(rng.integers(0, i))
            if depth[p] < 7:
                break
        parent[i], depth[i], masks[i] = p, depth[p] + 1, masks[p] | (1 << i)
    pos = [L + d - 1 for d in depth]
    ids = rng.integers(0, 50, T).tolist()
    gt = rng.integers(0, 50, T).tolist()
    for i in range(1, T):
        if rng.random() < 0.6:
            ids[i] = gt[parent[i]]
    n, best, path = otree.verify(ids, gt, pos, L, masks, parent)
    return {"T": T, "L": L, "ids": ids, "gt": gt, "pos": pos, "mask": masks, "parent": parent, "n": n, "best": best,
            "path": path, "tokens": otree.emitted_tokens(gt, path)}


def generate_case(dtype, head_dim, hq, hkv, inter, seed):
    cfg = OracleConfig(vocab=4096, layers=2, hidden=256, inter=inter, hq=hq, hkv=hkv, head_dim=head_dim, dtype=dtype)
    e = EagleOracleConfig(num_iter=4, topk=4, tree_size=16)
    w, ew = make_weights(cfg, seed, e, layer_scale=0.6, fc_mode="embed", fc_gain=200.0)
    m = OracleModel(cfg, w, e, ew, budget=512)
    prompt = np.random.default_rng(seed).integers(0, 4096, 128).tolist()
    tokens, accept, steps = m.generate_spec(prompt, 32)
    plain = OracleModel(cfg, w, e, ew, budget=512).generate_plain(prompt, 32)
    return {"dtype": dtype, "head_dim": head_dim, "hq": hq, "hkv": hkv, "inter": inter, "seed": seed,
            "tokens": tokens, "accept": accept, "plain": plain,
            "first_tree": {"ids": steps[0]["ids"].tolist(), "parent": steps[0]["parent"].tolist(),
                           "mask": [int(x) for x in steps[0]["mask"]]}}


def main():
    out = {
        "trees": [tree_case(1, 4096, 4, 4, 16, False), tree_case(2, 5000, 10, 6, 60, False),
                  tree_case(3, 3000, 8, 3, 64, True), tree_case(4, 2048, 1, 5, 5, False)],
        "verify": [verify_case(s, T) for s, T in [(0, 16), (1, 60), (2, 64), (3, 2)]],
        # BASELINE config 1 (fp32, head_dim 64, FFN 688, 4 q / 2 kv heads) and the bf16 head_dim-128 test model
        "generate": [generate_case("fp32", 64, 4, 2, 688, 0), generate_case("bf16", 128, 2, 1, 704, 0)],
    }
    with open(os.path.join(HERE, "oracle_golden.json"), "w") as f:
        json.dump(out, f)
    print("wrote", os.path.join(HERE, "oracle_golden.json"))


if __name__ == "__main__":
    main()
