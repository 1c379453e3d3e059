"""Per-kernel timing of the two heavy kernels of the speculative step, through the C ABI.

    python kernel_bench.py linear [M,N,K] [iters]      bf16 weights
    python kernel_bench.py linear_w4 [M,N,K] [iters]   4-bit weights (W4A16)
    python kernel_bench.py linear_swiglu [M,inter,K] [iters]   gate/up projection with the SwiGLU epilogue
    python kernel_bench.py attention [tq,hq,hkv,kv,splits,mask] [iters]
    python kernel_bench.py select [tq,hq,hkv,L,budget] [iters]    InfLLM-v2 block selection of one layer
    python kernel_bench.py reference                   the reference project's own kernels beside the library's
    python kernel_bench.py tail [iters]                the integer tail of a step at the 8B shapes: draft tree from
                                                       logits (log-softmax, top-k, expansion, tree) and acceptance + fix-up

Each case runs `iters` back-to-back launches inside the library, timed with CUDA events on the
library's stream, rotating over enough separate weight (or KV-cache) copies that no launch finds
its operands in L2.  Prints one line per case: average microseconds per launch and the weight
(KV) bytes streamed per second.  Without a shape the shapes of the 8B verify (M=60) and draft
(M=10) passes are run.  The same command under `ncu -k regex:linear|tree_attn` is how the
summaries under profiles/ are made.
"""
import ctypes
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "cpm.cu_b200"))
import cpmcu.C as C  # noqa: E402

# qkv, o, gate_up, down, LM head of the 8B shape (hidden 4096, FFN 16384, 32 q / 2 kv heads, vocab 73448)
LINEAR_SHAPES = [(60, 4608, 4096), (60, 4096, 4096), (60, 32768, 4096), (60, 4096, 16384), (60, 73448, 4096),
                 (10, 4608, 4096), (10, 4096, 4096), (10, 32768, 4096), (10, 4096, 16384), (10, 73448, 4096),
                 (10, 4096, 8192)]
W4_SHAPES = [(60, 4608, 4096), (60, 4096, 4096), (60, 32768, 4096), (60, 4096, 16384)]
ATTN_CASES = [(60, 32, 2, 4156, 9, 1), (60, 32, 2, 4156, 4, 1), (10, 32, 2, 4116, 32, 1), (7, 32, 2, 4096, 32, 0)]


def _us(fn, *args):
    out = ctypes.c_float()
    C.call(fn, *args, ctypes.cast(ctypes.pointer(out), ctypes.c_void_p))
    return out.value


def bench_linear(shapes, iters, w4):
    for M, N, K in shapes:
        store = N * K * 2                         # bytes of one bf16 copy; the 4-bit run reads a quarter of it
        copies = max(1, min(40, (600 << 20) // store + 1))
        if w4:
            copies = min(64, 4 * copies)          # same footprint to rotate over
        us = _us("cpmcu_bench_linear_w4" if w4 else "cpmcu_bench_linear", M, N, K, copies, iters, 0)
        streamed = store // 4 + (K // 128) * N * 2 if w4 else store
        print(f"{'linear_w4' if w4 else 'linear'} M={M} N={N} K={K} copies={copies}: {us:.1f} us  "
              f"{streamed / us / 1e3:.0f} GB/s", flush=True)


def bench_linear_swiglu(shapes, iters):
    for M, inter, K in shapes:
        store = 2 * inter * K * 2                 # gate and up rows
        copies = max(1, min(40, (600 << 20) // store + 1))
        us = _us("cpmcu_bench_linear_swiglu", M, inter, K, copies, iters, 0)
        print(f"linear_swiglu M={M} inter={inter} K={K} copies={copies}: {us:.1f} us  {store / us / 1e3:.0f} GB/s", flush=True)


def bench_attention(cases, iters):
    for tq, hq, hkv, kv, splits, mask in cases:
        us = _us("cpmcu_bench_attention", tq, hq, hkv, kv, splits, mask, iters)
        kv_bytes = 2 * kv * hkv * 128 * 2
        print(f"attention tq={tq} hq={hq} hkv={hkv} kv={kv} splits={splits} mask={mask}: {us:.1f} us  "
              f"{kv_bytes / us / 1e3:.0f} GB/s", flush=True)


def bench_select(case, iters):
    """One layer's block selection (compress from scratch + stage-1 scores + max-pool / top-k / bitmask)
    through cpmcu_sparse_select; host-clock time per call, for per-kernel times run it under ncu."""
    import time

    import torch
    tq, hq, hkv, L, budget = case
    q = torch.randn(tq, (hq + 2 * hkv) * 128, device="cuda").to(torch.bfloat16)
    k = torch.randn(budget, hkv * 128, device="cuda").to(torch.bfloat16)
    score_ld = (budget // 16 + 127) // 128 * 128
    words = (budget // 64 + 63) // 64
    bm = torch.zeros(hkv, tq, words, dtype=torch.int64, device="cuda")
    kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    torch.cuda.synchronize()
    for i in range(iters + 1):
        if i == 1:
            t0 = time.time()
        C.call("cpmcu_sparse_select", p(q), q.shape[1], tq, hq, hkv, p(k), budget, p(kv_len), 0, 1, 32, 64, 8192, 1,
               None, None, None, score_ld, p(bm), words)
    us = (time.time() - t0) / iters * 1e6
    print(f"select tq={tq} hq={hq} hkv={hkv} L={L} budget={budget}: {us:.0f} us per call (host clock, "
          f"includes the compression of all {L // 16} + {L // 64} entries and the buffer set-up)", flush=True)


def bench_reference(iters=40):
    """The reference project's own kernels (oracle/_ref/, built by `python -m oracle.build_ref [--marlin] [--flash]`
    from a reference checkout) timed beside the library's on the same device: its linear<T> (a cuBLAS call), its
    Marlin W4A16 GEMM and its attention (mha_fwd_kvcache: split kernel + combine), all at the verify / draft shapes
    of the 8B configuration, operands rotating through HBM.  Prints a table; a missing library skips its rows."""
    import torch
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    rows = []
    us = ctypes.c_float(0.0)
    shapes = [("qkv", 60, 4608, 4096), ("o", 60, 4096, 4096), ("gate_up", 60, 32768, 4096), ("down", 60, 4096, 16384),
              ("lm_head", 60, 73448, 4096), ("draft lm_head", 10, 73448, 4096)]
    lib = os.path.join(ref_dir, "libcpmcu_ref_kernels.so")
    if os.path.exists(lib):
        r = ctypes.CDLL(lib)
        for name, M, N, K in shapes:
            copies = max(2, min(24, int(1.2e9 // (N * K * 2))))
            assert r.refk_bench_linear(M, N, K, copies, iters, ctypes.byref(us)) == 0
            rows.append(("bf16 %s M=%d (reference: cuBLAS)" % (name, M), us.value, _us("cpmcu_bench_linear", M, N, K, copies, iters, 0)))
    lib = os.path.join(ref_dir, "libcpmcu_ref_marlin.so")
    if os.path.exists(lib):
        m = ctypes.CDLL(lib)
        for name, M, N, K in shapes[:4]:
            copies = max(2, min(24, int(1.2e9 // (N * K // 2))))
            assert m.refk_bench_marlin(M, N, K, copies, iters, ctypes.byref(us)) == 0
            rows.append(("W4A16 %s M=%d (reference: Marlin)" % (name, M), us.value,
                         _us("cpmcu_bench_linear_w4", M, N, K, copies, iters, 0)))
    lib = os.path.join(ref_dir, "libcpmcu_ref_flash.so")
    if os.path.exists(lib):
        f = ctypes.CDLL(lib)
        for tq, kv, splits in ((60, 4156, 9), (10, 4116, 32), (60, 32828, 9)):
            hq, hkv, copies = 32, 2, 8
            padded = (kv + 127) // 128 * 128
            q = torch.randn(tq, hq * 128, device="cuda").to(torch.bfloat16)
            ks = [torch.randn(padded, hkv * 128, device="cuda").to(torch.bfloat16) for _ in range(copies)]
            vs = [torch.randn(padded, hkv * 128, device="cuda").to(torch.bfloat16) for _ in range(copies)]
            kp = (ctypes.c_void_p * copies)(*[t.data_ptr() for t in ks])
            vp = (ctypes.c_void_p * copies)(*[t.data_ptr() for t in vs])
            clen = torch.tensor([kv], dtype=torch.int32, device="cuda")
            mask = torch.tensor([(1 << i) | 1 for i in range(tq)], dtype=torch.int64, device="cuda")
            out = torch.empty(tq, hq * 128, dtype=torch.bfloat16, device="cuda")
            p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
            assert f.refk_bench_mha_fwd_kvcache(tq, padded, hq, hkv, p(q), kp, vp, copies, p(clen), p(mask), p(out), iters,
                                                ctypes.byref(us)) == 0
            rows.append(("tree attention tq=%d kv=%d (reference: 16 splits + combine)" % (tq, kv), us.value,
                         _us("cpmcu_bench_attention", tq, hq, hkv, kv, splits, 1, iters)))
    print("%-66s %12s %12s %8s" % ("kernel (CUDA events, back-to-back launches)", "reference us", "library us", "ratio"))
    for name, a, b in rows:
        print("%-66s %12.1f %12.1f %8.2f" % (name, a, b, a / b), flush=True)


def bench_tail(iters=5):
    """The latency-bound integer stages at the headline shapes, through their kernel-level entry points: the draft
    tree from given logits (V = 73448, top-k 10, 6 iterations, 60 nodes: per level log-softmax statistics, local
    top-k and expansion, then the tree) and acceptance + K/V compaction + gathers (64 caches of 256-wide rows, hidden
    4096).  Host-clock time per call (each call synchronises); run under ncu for the per-kernel device times."""
    import time

    import torch
    V, k, it, T, H = 73448, 10, 6, 60, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    logits = (torch.randn(1 + (it - 1) * k, V, generator=g, device="cuda") * 2).to(torch.bfloat16)
    tt = k + k * k * (it - 1)
    ids = torch.zeros(64, dtype=torch.int32, device="cuda")
    pos = torch.zeros(64, dtype=torch.int32, device="cuda")
    mask = torch.zeros(64, dtype=torch.int64, device="cuda")
    par = torch.zeros(64, dtype=torch.int32, device="cuda")
    tv = torch.zeros(tt + 64, dtype=torch.bfloat16, device="cuda")
    tp = torch.zeros(tt + 64, dtype=torch.int32, device="cuda")
    tpar = torch.zeros(k * it + 64, dtype=torch.int32, device="cuda")
    cl = torch.tensor([4096], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for i in range(iters + 1):
        if i == 1:
            t0 = time.time()
        C.call("cpmcu_draft_tree_from_logits", p(logits), V, k, it, T, None, p(cl), p(ids), p(pos), p(mask), p(par), p(tv),
               p(tp), p(tpar))
    print(f"draft tree from logits V={V} k={k} iters={it} T={T}: {(time.time() - t0) / iters * 1e6:.0f} us per call "
          f"(host clock, {it + 1} launches)", flush=True)
    rows, kvd, ncache = 4352, 256, 64
    caches = [torch.randn(rows, kvd, device="cuda", generator=g).to(torch.bfloat16) for _ in range(ncache)]
    cptr = torch.tensor([c.data_ptr() for c in caches], dtype=torch.int64, device="cuda")
    gt = torch.randint(0, V, (64,), device="cuda", generator=g).to(torch.int32)
    # a chain 0 -> 1 -> 2 -> 3 is drafted correctly: accept length 4
    pred = gt.clone()
    tree_par = torch.zeros(64, dtype=torch.int32, device="cuda")
    tree_pos = torch.full((64,), 4097, dtype=torch.int32, device="cuda")
    import numpy as np
    tree_mask = torch.from_numpy(np.array([(1 << i) | 1 for i in range(64)], dtype=np.uint64).view(np.int64)).to("cuda")
    for i in range(1, 4):
        tree_par[i] = i - 1
        tree_pos[i] = 4096 + i
        tree_mask[i] = (1 << (i + 1)) - 1   # i <= 3
        pred[i] = gt[i - 1]
    tree_pos[0] = 4096
    norm_out = torch.randn(64, H, device="cuda", generator=g).to(torch.bfloat16)
    prev_hidden = torch.zeros(8, H, dtype=torch.bfloat16, device="cuda")
    prev_embed = torch.zeros(8, H, dtype=torch.bfloat16, device="cuda")
    embed = torch.randn(V, H, device="cuda", generator=g).to(torch.bfloat16)
    epos = torch.zeros(8, dtype=torch.int32, device="cuda")
    result = torch.zeros(32, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for i in range(iters + 1):
        if i == 1:
            t0 = time.time()
        pr = pred.clone()
        C.call("cpmcu_accept_fixup", T, p(pr), p(gt), p(tree_pos), p(cl), p(tree_mask), p(tree_par), p(cptr), ncache, kvd, rows,
               7, H, p(norm_out), p(prev_hidden), p(embed), 1.0, p(prev_embed), p(epos), p(result))
    assert int(result[0]) == 4
    print(f"acceptance + fix-up T={T}, {ncache} caches x {kvd}, hidden {H}, accept length 4: "
          f"{(time.time() - t0) / iters * 1e6:.0f} us per call (host clock, 1 launch)", flush=True)


def main(argv):
    what = argv[1] if len(argv) > 1 else "linear"
    shape = tuple(int(v) for v in argv[2].split(",")) if len(argv) > 2 else None
    iters = int(argv[3]) if len(argv) > 3 else 50
    if what == "linear":
        bench_linear([shape] if shape else LINEAR_SHAPES, iters, False)
    elif what == "linear_w4":
        bench_linear([shape] if shape else W4_SHAPES, iters, True)
    elif what == "linear_swiglu":
        bench_linear_swiglu([shape] if shape else [(60, 16384, 4096), (10, 16384, 4096), (4096, 16384, 4096)], iters)
    elif what == "attention":
        bench_attention([shape] if shape else ATTN_CASES, iters)
    elif what == "tail":
        bench_tail(int(argv[2]) if len(argv) > 2 else 5)
    elif what == "reference":
        bench_reference(iters if len(argv) > 3 else 40)
    elif what == "select":
        bench_select(shape if shape else (60, 32, 2, 32768, 40960), iters if len(argv) > 3 else 3)
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main(sys.argv)
