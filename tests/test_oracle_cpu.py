"""CPU tests of the oracle itself: regression fixtures, ordering rules and the
invariants of the speculative step."""
import json
import os

import numpy as np
import torch

from oracle import tree as otree
from oracle.model import EagleOracleConfig, OracleConfig, OracleModel, make_weights

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "oracle_golden.json")))


def test_bf16_round_matches_torch():
    x = torch.randn(10000, generator=torch.Generator().manual_seed(0)) * 37
    assert np.array_equal(otree.bf16_round(x.numpy()), x.to(torch.bfloat16).float().numpy())
    # ties to even
    a = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8], dtype=np.float32)
    assert np.array_equal(otree.bf16_round(a), np.array([1.0, 1.0 + 2.0 ** -6], dtype=np.float32))


def test_topk_order_value_desc_then_lower_index():
    v = np.array([1.0, 3.0, 3.0, -1.0, 3.0, 2.0], dtype=np.float32)
    vals, idx = otree.topk_desc(v, 4)
    assert idx.tolist() == [1, 2, 4, 5] and vals.tolist() == [3.0, 3.0, 3.0, 2.0]


def test_golden_trees_reproduce():
    from tests_golden_helpers import tree_case
    for want in GOLD["trees"]:
        got = tree_case(want["seed"], want["V"], want["k"], want["num_iter"], want["T"], want["coarse"])
        assert got == want
        T, L = want["T"], want["cache_length"]
        for i in range(1, T):  # invariants: ancestors precede, own bit set, popcount == depth
            assert want["parent"][i] < i and (want["mask"][i] >> i) & 1
            assert bin(want["mask"][i]).count("1") == want["pos"][i] - L + 1
            assert want["mask"][i] == want["mask"][want["parent"][i]] | (1 << i)


def test_golden_verify_reproduce_and_path_is_monotone():
    for c in GOLD["verify"]:
        n, best, path = otree.verify(c["ids"], c["gt"], c["pos"], c["L"], c["mask"], c["parent"])
        assert (n, best, path) == (c["n"], c["best"], c["path"])
        assert otree.emitted_tokens(c["gt"], path) == c["tokens"]
        assert all(path[i] >= i for i in range(n)) and path[0] == 0 and 1 <= n <= 7
        # compaction never reads a row it already overwrote when done in increasing order
        cache = np.arange((c["L"] + c["T"]) * 3, dtype=np.int64).reshape(-1, 3)
        ref = cache.copy()
        otree.compact_rows(cache, c["L"], path)
        for i, p in enumerate(path):
            assert np.array_equal(cache[c["L"] + i], ref[c["L"] + p])


def test_verify_edge_cases():
    # nothing matches: only the root is accepted, the bonus token is the target's prediction at the root
    n, best, path = otree.verify([5, 6, 7], [1, 2, 3], [10, 11, 11], 10, [1, 3, 5], [0, 0, 0])
    assert (n, best, path) == (1, 0, [0])
    # a correct node below an incorrect one is not accepted
    n, best, path = otree.verify([5, 6, 9], [1, 9, 3], [10, 11, 12], 10, [1, 3, 7], [0, 0, 1])
    assert n == 1
    # full chain
    n, best, path = otree.verify([5, 1, 2], [1, 2, 3], [10, 11, 12], 10, [1, 3, 7], [0, 0, 1])
    assert (n, best, path) == (3, 2, [0, 1, 2])


def test_golden_generate_reproduce_and_speculation_is_lossless():
    from tests_golden_helpers import generate_case
    for want in GOLD["generate"]:
        got = generate_case(want["dtype"], want["head_dim"], want["hq"], want["hkv"], want["inter"], want["seed"])
        assert got == want
        assert want["tokens"] == want["plain"], "greedy speculative output must equal plain greedy decoding"
        assert max(want["accept"]) > 1 and all(1 <= a <= 5 for a in want["accept"])


def test_frspec_tree_ids_stay_inside_the_reduced_vocabulary():
    cfg = OracleConfig(vocab=4096, layers=1, hidden=256, inter=704, hq=2, hkv=1, head_dim=128, dtype="bf16")
    e = EagleOracleConfig(num_iter=3, topk=4, tree_size=12, frspec_vocab=512, minicpm4_variant=True)
    remap = np.sort(np.random.default_rng(0).permutation(4096)[:512]).astype(np.int32)
    w, ew = make_weights(cfg, 5, e, layer_scale=0.5, fc_mode="embed", fc_gain=200.0)
    m = OracleModel(cfg, w, e, ew, budget=256, token_id_remap=remap)
    prompt = np.random.default_rng(5).integers(0, 4096, 64).tolist()
    tokens, accept, steps = m.generate_spec(prompt, 12)
    for st in steps:
        assert set(st["ids"][1:].tolist()) <= set(remap.tolist())
    assert tokens == OracleModel(cfg, w, e, ew, budget=256, token_id_remap=remap).generate_plain(prompt, 12)


def test_teacher_forced_check_accepts_a_greedy_stream_and_rejects_a_wrong_token():
    """helpers.check_greedy_stream (the GPU tests' token-stream judge): the oracle's own speculative output passes
    without a tolerated tie; a stream with one token swapped for a non-runner-up fails at exactly that position,
    and the positions after a swapped-in token are judged given the swapped prefix."""
    import pytest
    from helpers import check_greedy_stream
    cfg = OracleConfig(vocab=4096, layers=2, hidden=256, inter=704, hq=2, hkv=1, head_dim=128, dtype="bf16")
    e = EagleOracleConfig(num_iter=3, topk=4, tree_size=12)
    w, ew = make_weights(cfg, 11, e, layer_scale=0.5, fc_mode="embed", fc_gain=200.0)
    prompt = np.random.default_rng(11).integers(0, 4096, 48).tolist()
    tokens, accept, steps = OracleModel(cfg, w, e, ew, budget=256).generate_spec(prompt, 14)
    judge = OracleModel(cfg, w, e, ew, budget=256)
    assert check_greedy_stream(judge, prompt, tokens, "oracle stream") == []
    bad = list(tokens)
    bad[5] = (bad[5] + 1) % 4096
    with pytest.raises(AssertionError, match="token 5"):
        check_greedy_stream(judge, prompt, bad, "swapped stream")
