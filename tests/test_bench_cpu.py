"""Host-side arithmetic of bench.py: the algorithmic byte counts behind the roofline figures, the FR-Spec
vocabulary order and the synthetic-checkpoint plumbing (no GPU)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def test_algorithmic_bytes_match_the_hand_count():
    # per target layer: q/k/v (4608 x 4096) + o (4096 x 4096) + gate/up (32768 x 4096) + down (4096 x 16384)
    layer = 4608 * 4096 + 4096 * 4096 + 32768 * 4096 + 4096 * 16384
    assert layer == 236_978_176
    target, draft = bench.algorithmic_bytes()
    assert target == (32 * layer + 73448 * 4096) * 2          # 15.77 GB of bf16 weights, LM head included
    assert draft == 6 * (2 * 4096 * 4096 + layer + 73448 * 4096) * 2   # six passes of fc + layer + LM head: 6.86 GB
    assert abs((target + draft) / 1e9 - 22.62) < 0.01
    t3, d3 = bench.algorithmic_bytes(draft_vocab=bench.FRSPEC_VOCAB)
    assert t3 == target and d3 == 6 * (2 * 4096 * 4096 + layer + 32768 * 4096) * 2
    t4, d4 = bench.algorithmic_bytes(w4a16=True)
    assert t4 == int(32 * layer * (0.5 + 2 / 128)) + 73448 * 4096 * 2 and d4 == draft
    # verify half at a 4096-token context: weights + K/V of 32 layers + the 60 x vocab logits = 15.92 GB
    assert abs(bench.verify_bytes(False, 4096) / 1e9 - 15.92) < 0.01


def test_frspec_vocabulary_is_ordered_by_descending_count_then_id():
    remap = bench.frspec_remap(1)
    assert remap.shape == (bench.FRSPEC_VOCAB,) and remap.dtype == np.int32 and len(set(remap.tolist())) == len(remap)
    counts = np.bincount(bench.zipf_prompt(1_000_000, bench.CFG["vocab"], 1001), minlength=bench.CFG["vocab"])
    c = counts[remap]
    assert np.all(c[:-1] >= c[1:])
    ties = c[:-1] == c[1:]
    assert np.all(remap[:-1][ties] < remap[1:][ties])
    assert c[-1] >= np.delete(counts, remap).max()            # nothing left out is more frequent than what is kept


def test_list_split_feeds_target_then_drafter():
    events = [("eagle", "token_id_remap", np.zeros(1)), (None, "a", np.ones(1)), ("eagle", "fc.weight", np.ones(2)),
              (None, "b", np.ones(3))]

    class T:  # stand-in for a tensor: list_split only calls .to("cpu") on drafter tensors
        def __init__(self, v):
            self.v = v

        def to(self, _):
            return self

    base, eagle = bench.list_split((k, n, T(v)) for k, n, v in events)
    assert [n for n, _ in base] == ["a", "b"]
    assert [n for n, _ in eagle] == ["token_id_remap", "fc.weight"]


def test_workload_table_covers_the_four_gpu_configurations():
    assert sorted(bench.WORKLOADS) == ["config2", "config3", "config4", "config5"]
    assert [bench.WORKLOADS[k]["index"] for k in sorted(bench.WORKLOADS)] == [1, 2, 3, 4]
