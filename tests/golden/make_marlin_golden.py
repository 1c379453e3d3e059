"""Golden vectors of the W4A16 Marlin layout, produced by the REFERENCE's own converter functions
(model_convert/convert_w4a16.py: get_perms, marlin_repack_qweight, marlin_permute_scales), which are
plain Python/numpy and run without a GPU.  Run from the repo root in a container that has the
reference mounted:  python tests/golden/make_marlin_golden.py /path/to/reference
The committed JSON is what the tests read; the reference is not needed at test time."""
import json
import os
import sys

import numpy as np
import torch


def load_reference_functions(ref_root):
    src = open(os.path.join(ref_root, "model_convert", "convert_w4a16.py")).read()
    head = src.split("parser = argparse.ArgumentParser()")[0]          # imports
    body = "def get_perms" + src.split("def get_perms", 1)[1].split("def convert_w4a16_checkpoint")[0]
    ns = {}
    exec(compile(head + body, "reference_convert_w4a16", "exec"), ns)
    return ns


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_marlin_golden.py <path of the reference checkout>")
    ref_root = sys.argv[1]
    ns = load_reference_functions(ref_root)
    rng = np.random.default_rng(123)
    cases = []
    for K, N in [(128, 64), (256, 128)]:
        q = rng.integers(0, 16, (K, N)).astype(np.uint32)
        scales = (rng.random((K // 128, N)).astype(np.float32) * 0.01 + 0.001)
        scales = torch.from_numpy(scales).to(torch.bfloat16).float().numpy()
        auto = np.zeros((K // 8, N), dtype=np.uint32)   # AutoGPTQ packing: 8 consecutive k per word
        for i in range(8):
            auto |= q[i::8, :] << np.uint32(4 * i)
        packed = ns["marlin_repack_qweight"](torch.from_numpy(auto.view(np.int32)), 4, K, N).numpy()
        sperm = ns["marlin_permute_scales"](torch.from_numpy(scales), K, N, 128).numpy()
        # compact text encodings: one hex digit per 4-bit value, eight per packed word
        cases.append({"K": K, "N": N, "q_hex": "".join("%x" % v for v in q.ravel()),
                      "scales": scales.tolist(),
                      "packed_hex": "".join("%08x" % (int(v) & 0xFFFFFFFF) for v in packed.ravel()),
                      "scales_perm": sperm.tolist()})
    perm, scale_perm, scale_perm_single = ns["get_perms"]()
    out = {"perm": [int(x) for x in perm], "scale_perm": [int(x) for x in scale_perm],
           "scale_perm_single": [int(x) for x in scale_perm_single], "cases": cases}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "marlin_golden.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path)


if __name__ == "__main__":
    main()
