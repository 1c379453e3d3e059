"""The work distribution of the linear kernels (stream-K pieces, whole-tile waves, the cut tail, the band raster),
walked on the host through cpmcu_debug_linear_schedule: the iterator and raster functions are the ones the kernels
run, compiled for the host.  No GPU."""
import collections
import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "cpm.cu_b200"))


def pick_mt(M):
    return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256


def schedule(M, N, K, limit):
    import __graft_entry__ as entry
    import cpmcu.C as C
    if not os.path.exists(C.lib_path()):
        entry.build()
    cap = 1 << 16
    out = np.zeros((cap, 6), dtype=np.int32)
    n = C.call("cpmcu_debug_linear_schedule", M, N, K, limit, ctypes.c_void_p(out.ctypes.data), cap)
    return out[:n]


SHAPES = [
    # decode-sized (one token tile): plain stream-K
    (60, 4608, 4096, 148), (10, 73448, 4096, 148), (60, 1000, 2048, 3), (1, 256, 256, 148), (33, 300, 128, 148),
    # prefill-sized: whole tiles in waves, the rest cut along K
    (4096, 4608, 4096, 148), (4096, 4096, 4096, 148), (4096, 32768, 4096, 148), (4096, 4096, 16384, 148),
    (2048, 4096, 16384, 148), (4100, 1280, 256, 148), (700, 1024, 512, 7), (520, 384, 2048, 5), (257, 640, 1024, 11),
    (3328, 1536, 1024, 148), (300, 1024, 512, 148), (9000, 512, 128, 148), (4096, 128, 64, 148), (5000, 8192, 8192, 132),
]


@pytest.mark.parametrize("M,N,K,limit", SHAPES)
def test_every_k_block_of_every_tile_is_computed_exactly_once(M, N, K, limit):
    seg = schedule(M, N, K, limit)
    mt = pick_mt(M)
    n_tiles, m_tiles, kblocks = -(-N // 128), -(-M // mt), K // 64
    assert len(seg) > 0 and seg[:, 0].max() < limit
    # raster: tile number <-> (token tile, feature tile) is a bijection onto the grid of tiles
    pairs = {}
    for g, tile, m, n, kb0, kb1 in seg.tolist():
        assert 0 <= m < m_tiles and 0 <= n < n_tiles and 0 <= kb0 < kb1 <= kblocks
        assert pairs.setdefault(tile, (m, n)) == (m, n)
    assert len(pairs) == n_tiles * m_tiles == len(set(pairs.values()))
    # coverage: the pieces of a tile tile its k range, in CTA order, by consecutive CTAs
    pieces = collections.defaultdict(list)
    for g, tile, m, n, kb0, kb1 in seg.tolist():
        pieces[tile].append((kb0, kb1, g))
    for tile, ps in pieces.items():
        ps.sort()
        assert ps[0][0] == 0 and ps[-1][1] == kblocks
        for (a0, a1, ga), (b0, b1, gb) in zip(ps, ps[1:]):
            assert a1 == b0 and gb == ga + 1
    # a CTA holds at most two cut pieces (the workspace has two slots per CTA): the end of one tile and the start of
    # another, and it runs them before its whole tiles
    for g in range(int(seg[:, 0].max()) + 1):
        mine = [s for s in seg.tolist() if s[0] == g]
        cut = [s for s in mine if not (s[4] == 0 and s[5] == kblocks)]
        assert len(cut) <= 2
        assert sum(1 for s in cut if s[4] > 0) <= 1 and sum(1 for s in cut if s[4] == 0) <= 1
        if m_tiles > 1 and cut:
            last_cut = max(i for i, s in enumerate(mine) if s in cut)
            whole_after = [s for s in mine[last_cut + 1:]]
            assert all(s[4] == 0 and s[5] == kblocks for s in whole_after)
    # balance: no CTA has more than one tile's worth of k-blocks above the mean
    load = collections.Counter()
    for g, tile, m, n, kb0, kb1 in seg.tolist():
        load[g] += kb1 - kb0
    ctas = int(seg[:, 0].max()) + 1
    assert max(load.values()) <= n_tiles * m_tiles * kblocks / ctas + kblocks


def test_a_wave_of_tiles_shares_few_weight_slabs_and_one_band_of_tokens():
    """4096 tokens x 4096 x 16384 (the down projection of a prefill chunk): 256-token tiles in bands of 8, so the 148
    tiles that run together cover all 8 token tiles of a band and about 148 / 8 feature tiles."""
    seg = schedule(4096, 4096, 16384, 148)
    whole = [s for s in seg.tolist() if s[4] == 0 and s[5] == 256]
    first = {}
    for s in whole:               # the first whole tile of every CTA: one wave
        first.setdefault(s[0], s)
    wave = list(first.values())
    assert len(wave) == 148
    m_set, n_set = {s[2] for s in wave}, {s[3] for s in wave}
    assert len(m_set) == 8 and max(m_set) - min(m_set) == 7
    assert len(n_set) <= 148 // 8 + 2
