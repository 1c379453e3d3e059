"""W4A16 GPTQ-Marlin weight format: quantisation, the Marlin tile repack and its inverse (numpy).

TEST INFRASTRUCTURE ONLY (see oracle/tree.py).  Restates the layout produced by the reference's
converter, model_convert/convert_w4a16.py:17-82 (`get_perms`, `marlin_repack_qweight`,
`marlin_permute_scales`), and the dequantisation of its kernel, `w = (q - 8) * scale`
(src/qgemm/gptq_marlin/gptq_marlin.cu:139-162, scalar type kU4B8).  The permutation tables are the
only constants the reference fixes for this path; the round trip quantise -> repack -> unpack is the
known-answer test of the layout.  The layout is also checked end to end against the reference's own
Marlin kernel: tests/test_ref_kernels_gpu.py packs weights with `marlin_pack`, runs the reference's
gptq_marlin_gemm (oracle/ref_marlin.cu) on them and compares with the library and with x @ dequantize().
"""
import numpy as np

from .tree import bf16_round


def marlin_perms():
    """The three index tables of the Marlin layout (convert_w4a16.py:17-43)."""
    perm = []
    for i in range(32):
        col = i // 4
        one = []
        for block in (0, 1):
            for row in (2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1):
                one.append(16 * row + col + 8 * block)
        for j in range(4):
            perm.extend(p + 256 * j for p in one)
    perm = np.array(perm).reshape(-1, 8)[:, [0, 2, 4, 6, 1, 3, 5, 7]].ravel()
    scale_perm = [i + 8 * j for i in range(8) for j in range(8)]
    scale_perm_single = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return perm, np.array(scale_perm), np.array(scale_perm_single)


PERM, SCALE_PERM, SCALE_PERM_SINGLE = marlin_perms()


def quantize_sym_int4(w_kn, group_size=128):
    """Symmetric int4 with per-group scales = absmax / 7 (BASELINE config 4).  w_kn: [K, N] float32.
    Returns q in [0, 15] (value + 8) as uint8 [K, N] and bf16-valued scales [K/group, N] float32."""
    K, N = w_kn.shape
    g = w_kn.reshape(K // group_size, group_size, N)
    scales = bf16_round(np.maximum(np.abs(g).max(axis=1), 1e-8) / 7.0)
    q = np.clip(np.rint(g / scales[:, None, :]), -8, 7).astype(np.int32) + 8
    return q.reshape(K, N).astype(np.uint8), scales.astype(np.float32)


def marlin_pack(q_kn, scales, group_size=128):
    """[K, N] 4-bit values -> int32 [K/16, N*2] in Marlin order; scales -> permuted [K/group, N]."""
    K, N = q_kn.shape
    t = q_kn.astype(np.uint32).reshape(K // 16, 16, N // 16, 16).transpose(0, 2, 1, 3).reshape(K // 16, N * 16)
    t = t.reshape(-1, PERM.size)[:, PERM].reshape(K // 16, N * 16)
    packed = np.zeros((K // 16, N * 2), dtype=np.uint32)
    for i in range(8):
        packed |= t[:, i::8] << np.uint32(4 * i)
    sp = SCALE_PERM if group_size < K and group_size != -1 else SCALE_PERM_SINGLE
    s = scales.reshape(-1, sp.size)[:, sp].reshape(-1, N)
    return packed.view(np.int32), np.ascontiguousarray(s)


def marlin_unpack(packed, scales_perm, K, N, group_size=128):
    """Inverse of marlin_pack: returns q [K, N] uint8 and scales [K/group, N]."""
    p = packed.view(np.uint32)
    t = np.zeros((K // 16, N * 16), dtype=np.uint32)
    for i in range(8):
        t[:, i::8] = (p >> np.uint32(4 * i)) & 0xF
    inv = np.argsort(PERM)
    t = t.reshape(-1, PERM.size)[:, inv].reshape(K // 16, N // 16, 16, 16).transpose(0, 2, 1, 3).reshape(K, N)
    sp = SCALE_PERM if group_size < K and group_size != -1 else SCALE_PERM_SINGLE
    s = scales_perm.reshape(-1, sp.size)[:, np.argsort(sp)].reshape(-1, N)
    return t.astype(np.uint8), s


def dequantize(q_kn, scales, group_size=128):
    """bf16((q - 8) * scale) as float32 [K, N] (one rounding, as the kernel's bf16 multiply)."""
    K, N = q_kn.shape
    w = (q_kn.astype(np.float32) - 8.0).reshape(K // group_size, group_size, N) * scales[:, None, :]
    return bf16_round(w.reshape(K, N))
