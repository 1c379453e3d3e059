"""The CPU oracle against golden vectors produced by the reference project's OWN device kernels
(tests/golden/ref_kernels_golden.json, written by tests/golden/make_ref_golden.py from
oracle/_ref/libcpmcu_ref_kernels.so run on a B200).  Everything here is bit-exact: draft tree from given
logits (log-softmax, top-k, frontier bookkeeping, final selection, tree build, FR-Spec remap), verify,
emitted tokens, compressed keys, max-pool + top-k + block bitmask."""
import importlib.util
import json
import os

import numpy as np
import pytest
import torch

from oracle import sparse as osparse
from oracle import tree as otree

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(HERE, "golden", "make_ref_golden.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)

with open(os.path.join(HERE, "golden", "ref_kernels_golden.json")) as f:
    GOLD = json.load(f)


def from_bits(b):
    return torch.tensor(b, dtype=torch.int16).view(torch.bfloat16).float()


def test_generator_cases_match_fixture():
    assert [c["seed"] for c in GOLD["trees"]] == [c[0] for c in gen.TREE_CASES]
    assert [c["seed"] for c in GOLD["verify"]] == [c[0] for c in gen.VERIFY_CASES]
    assert [c["seed"] for c in GOLD["select"]] == [c[0] for c in gen.SELECT_CASES]
    assert [c["seed"] for c in GOLD["compress"]] == [c[0] for c in gen.COMPRESS_CASES]


@pytest.mark.parametrize("c", GOLD["trees"], ids=lambda c: "seed%d" % c["seed"])
def test_oracle_draft_tree_equals_reference_kernels(c):
    V, k, it, T = c["V"], c["k"], c["num_iter"], c["T"]
    lg = gen.tree_logits(c["seed"], V, k, it, c["coarse"]).float().numpy()
    remap = gen.fr_remap(c["seed"], V, c["full_vocab"]) if c["full_vocab"] else None
    tree = otree.DraftTree(k, it, T, remap)
    tree.level0(otree.log_softmax_bf16(lg[0]))
    for d in range(1, it):
        tree.level(d, np.stack([otree.log_softmax_bf16(r) for r in lg[1 + (d - 1) * k: 1 + d * k]]))
    ids, pos, mask, par, _ = tree.finalize(c["cache_length"], 0)
    tt = tree.total_tried
    assert np.array_equal(from_bits(c["tried_val_bits"]).numpy(), tree.tried_val[:tt])
    assert np.array_equal(np.array(c["tried_pos"]), tree.tried_pos[:tt])
    assert np.array_equal(np.array(c["tried_parent"]), tree.tried_parent[: k * (it - 1)])
    assert ids[1:].tolist() == c["ids"]
    assert pos.tolist() == c["pos"]
    assert [int(m) for m in mask] == c["mask"]
    assert par[1:].tolist() == c["parent"]


@pytest.mark.parametrize("c", GOLD["verify"], ids=lambda c: "seed%d" % c["seed"])
def test_oracle_verify_equals_reference_kernels(c):
    ids, gt, pos, masks, parent = gen.verify_inputs(c["seed"], c["T"], c["L"])
    n, best, path = otree.verify(ids, gt, pos, c["L"], masks, parent)
    assert (n, best, path) == (c["n"], c["best"], c["path"])
    assert otree.emitted_tokens(gt, path) == c["tokens"]
    # the generator itself asserted that the reference moved whole rows L + path[i] -> L + i and nothing else,
    # which is what compact_rows restates
    rows = np.arange((c["L"] + c["T"] + 8) * 4, dtype=np.int16).reshape(-1, 4)
    want = rows.copy()
    for i, p in enumerate(path):
        want[c["L"] + i] = rows[c["L"] + p]
    assert np.array_equal(otree.compact_rows(rows.copy(), c["L"], path), want)


@pytest.mark.parametrize("c", GOLD["select"], ids=lambda c: "seed%d" % c["seed"])
def test_oracle_block_selection_equals_reference_kernels(c):
    hkv, T, L = c["hkv"], c["T"], c["cache_len"]
    n1 = max((L - 16) // 16, 0)
    scores = gen.select_scores(c["seed"], hkv, T, c["k_round"], n1).float()
    pool = osparse.maxpool_blocks(scores, T, L, c["sink"], c["window"])
    if c["pool_bits"] is not None:
        assert torch.equal(from_bits(c["pool_bits"]).view(hkv, T, -1), pool)
    mask = osparse.topk_blockmask(pool, c["top"], (L + T + 127) // 128 * 128)
    assert np.array_equal(mask, np.array(c["blockmask"], dtype=np.uint64).reshape(hkv, T, c["words"]))


@pytest.mark.parametrize("c", GOLD["compress"], ids=lambda c: "seed%d" % c["seed"])
def test_oracle_compressed_keys_equal_reference_kernels(c):
    keys = gen.compress_keys(c["seed"], c["L"], c["dim"]).float()
    for stride, key in ((16, "c1_bits"), (64, "c2_bits")):
        got = osparse.compress(keys, c["L"], stride).to(torch.bfloat16).float()
        assert torch.equal(got, from_bits(c[key]).view(-1, c["dim"]))
