"""Regenerates tests/golden/sparse_golden.json from oracle/sparse.py (run from the repo root:
`python tests/golden/make_sparse_golden.py`).  The reference has no vectors for the InfLLM-v2
selection path, so the fixture pins the oracle against regressions only."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import sparse as osparse  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def selection_case(seed, T, hq, hkv, L, top, sink, window, lse):
    """Seeded q / k, the block masks the oracle selects and a checksum of its stage-1 scores."""
    g = torch.Generator().manual_seed(seed)
    d = 128
    q = torch.randn(T, hq * d, generator=g).to(torch.bfloat16).float()
    base = torch.cumsum(torch.randn(L // 64 + 2, hkv * d, generator=g), dim=0) * 0.5
    k = (base.repeat_interleave(64, dim=0)[:L + T] + torch.randn(L + T, hkv * d, generator=g)).to(torch.bfloat16).float()
    cfg = osparse.SparseConfig(sink, window, top, 256, lse)
    c1 = osparse.compress(k, L, 16)
    c_lse = osparse.compress(k, L, 64) if lse else c1
    scores = osparse.stage1_scores(q, c1, c_lse, hq, hkv, d)
    mask = osparse.select_blocks(cfg, q, k, L, hq, hkv, d, L + T)
    return {"seed": seed, "T": T, "hq": hq, "hkv": hkv, "L": L, "top": top, "sink": sink, "window": window, "lse": lse,
            "score_sum": float(scores.double().sum()), "score_max": float(scores.max()),
            "mask": [[[int(w) for w in row] for row in head] for head in mask]}


def main():
    cases = [selection_case(1, 5, 8, 2, 1500, 6, 1, 4, True), selection_case(2, 3, 4, 1, 2100, 8, 2, 3, False),
             selection_case(3, 4, 32, 2, 1000, 64, 1, 2, True)]
    with open(os.path.join(HERE, "sparse_golden.json"), "w") as f:
        json.dump({"selection": cases}, f)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
