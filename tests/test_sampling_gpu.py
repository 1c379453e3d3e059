"""Device-side sampling (temperature > 0): the reference picks the target's token at every tree node with
torch.multinomial over softmax(logits / temperature) in its Python loop (cpmcu/speculative/tree_drafter.py:99-100,
230-231); here the pick is a Gumbel-max argmax with Philox noise inside the captured step.  Checked: the draws follow
the softmax distribution (chi-square), they are a pure function of (seed, row, draw), temperature -> 0 gives the
argmax, and a sampled generation is reproducible from its seed and lossless in structure (every step accepts
between 1 and num_iter + 1 tokens, accepted tokens are the sampled ones)."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import build_pair, tiny_configs
from oracle.model import EagleOracleConfig

pytestmark = pytest.mark.gpu


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def C():
    import cpmcu.C as c
    c.load()
    return c


def draw(c, logits, temperature, seed, index):
    rows, vocab = logits.shape
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    c.sample(ptr(logits), rows, vocab, temperature, seed, index, ptr(out))
    return out.cpu().numpy()


def test_draws_follow_softmax_of_scaled_logits():
    c = C()
    vocab, rows, draws, temperature = 12, 64, 500, 0.7
    g = torch.Generator().manual_seed(3)
    row = (torch.randn(vocab, generator=g) * 1.5).to(torch.bfloat16)
    logits = row[None, :].repeat(rows, 1).to("cuda").contiguous()
    counts = np.zeros(vocab)
    for d in range(draws):
        counts += np.bincount(draw(c, logits, temperature, 1234, d), minlength=vocab)
    n = rows * draws
    p = torch.softmax(row.float() / temperature, dim=-1).numpy().astype(np.float64)
    chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
    # 11 degrees of freedom: the 99.99th percentile is 37.4
    assert chi2 < 37.4, (chi2, counts, n * p)
    # rows and draws are independent streams: neighbouring rows / draws are not copies of one another
    a, b = draw(c, logits, temperature, 1234, 0), draw(c, logits, temperature, 1234, 1)
    assert not np.array_equal(a, b) and len(set(a.tolist())) > 1


def test_draws_are_a_pure_function_of_seed_row_and_draw_index():
    c = C()
    g = torch.Generator().manual_seed(4)
    logits = (torch.randn(60, 73448, generator=g) * 2).to(torch.bfloat16).to("cuda")
    a = draw(c, logits, 0.9, 77, 5)
    assert np.array_equal(a, draw(c, logits, 0.9, 77, 5))
    assert not np.array_equal(a, draw(c, logits, 0.9, 78, 5))
    assert not np.array_equal(a, draw(c, logits, 0.9, 77, 6))
    # a row's draw does not depend on which other rows are in the launch (an unaligned row start takes the scalar path)
    sub = draw(c, logits[7:19].contiguous(), 0.9, 77, 5)
    assert not np.array_equal(sub, a[7:19])          # row index is part of the key
    odd = torch.zeros(3, 73449, dtype=torch.bfloat16, device="cuda")
    odd[:, :73448] = logits[:3]
    odd[:, 73448] = -100.0
    assert np.array_equal(draw(c, odd, 0.9, 77, 5), a[:3])   # same columns, other alignment and chunk tail


def test_small_temperature_is_argmax_and_zero_is_the_greedy_entry_point():
    c = C()
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(16, 5000, generator=g) * 3).to(torch.bfloat16).to("cuda")
    want = logits.float().argmax(dim=-1).to(torch.int32).cpu().numpy()
    assert np.array_equal(draw(c, logits, 1e-4, 9, 0), want)
    assert np.array_equal(draw(c, logits, 0.0, 9, 0), want)


def test_sampled_generation_is_reproducible_and_structurally_sound():
    cfg = tiny_configs("a")
    eagle = EagleOracleConfig(num_iter=4, topk=4, tree_size=16)
    prompt = np.random.default_rng(21).integers(0, cfg.vocab, 100).astype(np.int32)
    ids = torch.tensor(prompt, device="cuda")
    runs = {}
    for seed in (5, 5, 6):
        oracle, llm = build_pair(cfg, eagle, seed=2, fused_step=True)
        llm.temperature, llm.sample_seed = 0.8, seed
        tokens, acc, _, _ = llm.generate(ids, 40)
        assert len(tokens) == 40 and all(1 <= a <= eagle.num_iter + 1 for a in acc) and sum(acc) >= 39
        assert all(0 <= t < cfg.vocab for t in tokens)
        runs.setdefault(seed, []).append((tokens, acc))
    assert runs[5][0] == runs[5][1], "same seed, different stream"
    assert runs[5][0][0] != runs[6][0][0], "different seeds gave the same stream"
    oracle, llm = build_pair(cfg, eagle, seed=2, fused_step=True)
    greedy, _, _, _ = llm.generate(ids, 40)
    assert greedy != runs[5][0][0]
    # and greedy again after a sampled run on a fresh model: the sampling mode does not leak
    oracle, llm = build_pair(cfg, eagle, seed=2, fused_step=True)
    again, _, _, _ = llm.generate(ids, 40)
    assert again == greedy
