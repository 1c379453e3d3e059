"""cpmcu_argmax_noalloc: the argmax entry point for callers that must not allocate.

A loop that samples from its own logits while the engine is live cannot use
cpmcu_argmax: that entry takes its scratch from cudaMalloc on every call, which
may not fit once the model pool owns most of the device.  The variant tested
here keeps its scratch in a fixed 16 KB array inside the library.  The file name sorts last
so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_noalloc_argmax_matches_allocating_entry_twice_in_a_row():
    import cpmcu.C as C
    C.load()
    g = torch.Generator().manual_seed(11)
    for call, (rows, vocab) in enumerate([(60, 73448), (7, 32768)]):
        # two consecutive calls with different shapes: the second one runs on top of the
        # partials the first one left in the shared scratch
        logits = (torch.randn(rows, vocab, generator=g) * 3).to(torch.bfloat16).to("cuda")
        logits[0, 5] = 40.0
        logits[0, vocab - 1] = 40.0  # exact tie: the lower index must win in both entry points
        want = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        got = torch.full((rows,), -2, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        C.call("cpmcu_argmax", ptr(logits), rows, vocab, ptr(want))
        C.call("cpmcu_argmax_noalloc", ptr(logits), rows, vocab, ptr(got))
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: {got.tolist()[:8]} vs {want.tolist()[:8]}"
        assert int(got[0]) == 5
        # and against torch directly: argmax of the float values, lowest index among equal maxima
        f = logits.float()
        first_max = (f == f.max(dim=1, keepdim=True).values).int().argmax(dim=1).to(torch.int32)
        assert torch.equal(got, first_max)


def test_noalloc_argmax_at_the_full_extent_of_its_scratch():
    """64 rows x 262144 columns: every word of the 16 KB built-in scratch is in use."""
    import cpmcu.C as C
    C.load()
    rows, vocab = 64, 262144
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = (torch.randn(rows, vocab, generator=g, device="cuda") * 3).to(torch.bfloat16)
    logits[63, vocab - 1] = 50.0     # the very last element
    want = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    got = torch.full((rows,), -2, dtype=torch.int32, device="cuda")
    C.call("cpmcu_argmax", ptr(logits), rows, vocab, ptr(want))
    C.call("cpmcu_argmax_noalloc", ptr(logits), rows, vocab, ptr(got))
    torch.cuda.synchronize()
    assert torch.equal(got, want) and int(got[63]) == vocab - 1
    f = logits.float()
    first_max = (f == f.max(dim=1, keepdim=True).values).int().argmax(dim=1).to(torch.int32)
    assert torch.equal(got, first_max)


def test_noalloc_argmax_rejects_oversize_inputs():
    import cpmcu.C as C
    C.load()
    x = torch.zeros(2, 16, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(128, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="at most 64 rows"):
        C.call("cpmcu_argmax_noalloc", ptr(x), 65, 16, ptr(out))
    with pytest.raises(RuntimeError, match="262144"):
        C.call("cpmcu_argmax_noalloc", ptr(x), 2, 262145, ptr(out))
