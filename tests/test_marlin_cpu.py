"""W4A16 Marlin layout: the oracle's restatement against vectors produced by the reference's own
converter (tests/golden/marlin_golden.json, see make_marlin_golden.py)."""
import json
import os

import numpy as np

from oracle import marlin

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "marlin_golden.json")))


def test_permutation_tables_match_the_reference():
    assert marlin.PERM.tolist() == GOLD["perm"]
    assert marlin.SCALE_PERM.tolist() == GOLD["scale_perm"]
    assert marlin.SCALE_PERM_SINGLE.tolist() == GOLD["scale_perm_single"]
    assert sorted(marlin.PERM.tolist()) == list(range(1024))


def test_pack_matches_the_reference_converter_and_unpack_inverts_it():
    for c in GOLD["cases"]:
        K, N = c["K"], c["N"]
        q = np.array([int(ch, 16) for ch in c["q_hex"]], dtype=np.uint8).reshape(K, N)
        scales = np.array(c["scales"], dtype=np.float32)
        packed, sperm = marlin.marlin_pack(q, scales)
        want = np.array([int(c["packed_hex"][i:i + 8], 16) for i in range(0, len(c["packed_hex"]), 8)],
                        dtype=np.uint32).reshape(K // 16, 2 * N)
        assert np.array_equal(packed.view(np.uint32), want)
        assert np.array_equal(sperm, np.array(c["scales_perm"], dtype=np.float32))
        q2, s2 = marlin.marlin_unpack(packed, sperm, K, N)
        assert np.array_equal(q2, q) and np.array_equal(s2, scales)


def test_quantise_dequantise_error_bound():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((256, 128)) * 0.02).astype(np.float32)
    q, s = marlin.quantize_sym_int4(w)
    assert q.min() >= 0 and q.max() <= 15
    err = np.abs(marlin.dequantize(q, s) - w)
    assert (err <= 0.55 * np.repeat(s, 128, axis=0) + 1e-6).all()  # half a step, plus bf16 rounding of scale and product
