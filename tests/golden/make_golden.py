"""Generates the golden vectors under tests/golden/ from the reference project's own code.

Run where the reference tree is available (the oracle/_ref library built by oracle/build_ref.sh):

    python tests/golden/make_golden.py

For a handful of small seeded matrices it records, as .npz, the input, the reference's row-major
quantised tensor, its preprocessed tensor and its scales for int8 and int4, produced by the
reference's symmetric_quantize / preprocess_weights_for_mixed_gemm compiled from its sources with
the device reported as compute capability 10.0. The files are small (tens of KB) and committed;
tests/test_oracle.py and tests/test_host_ops.py compare the CPU oracle and the product's host ops
with them on every machine, with or without the reference tree.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import woq_oracle as o  # noqa: E402

CASES = [  # (name, K, N, weight dtype, seed)
    ("f32_64x64", 64, 64, torch.float32, 0),
    ("f32_64x192", 64, 192, torch.float32, 1),
    ("f16_192x64", 192, 64, torch.float16, 2),
    ("bf16_128x128", 128, 128, torch.bfloat16, 3),
]


def main():
    assert o.ref_lib() is not None, "build oracle/_ref first (oracle/build_ref.sh)"
    for name, K, N, dt, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        w = (torch.randn(K, N, generator=g) * 0.02).to(dt)
        w[:, 5] = 0  # an all-zero column exercises the scale == 0 branch
        w[3, 7] = w[:, 7].abs().max() * -1.0  # exact -amax: clamps at the negative end
        out = {"weight_f32": w.to(torch.float32).numpy()}
        for bits in (8, 4):
            u, p, s = o.ref_symmetric_quantize(w, bits)
            out[f"unprocessed_int{bits}"] = u.numpy()
            out[f"processed_int{bits}"] = p.numpy()
            out[f"scales_int{bits}_f32"] = s.to(torch.float32).numpy()
        # raw random bytes through the layout transform alone (every nibble/byte value occurs)
        rng = np.random.default_rng(seed)
        for bits in (8, 4):
            q = rng.integers(-128, 128, size=(K, N * bits // 8), dtype=np.int8)
            out[f"raw_int{bits}"] = q
            out[f"raw_processed_int{bits}"] = o.ref_preprocess_weights(q, bits)
        np.savez_compressed(os.path.join(HERE, f"quant_{name}.npz"), dtype=str(dt), **out)
        print("wrote", name)
    # int4 weights laid out for fp8 activations (W4A8): raw bytes through the reference's transform
    out = {}
    for K, N, seed in ((128, 64, 10), (256, 192, 11)):
        q = np.random.default_rng(seed).integers(-128, 128, size=(K, N // 2), dtype=np.int8)
        out[f"raw_{K}x{N}"] = q
        out[f"w4a8_{K}x{N}"] = o.ref_preprocess_weights_w4a8(q)
    np.savez_compressed(os.path.join(HERE, "layout_w4a8.npz"), **out)
    print("wrote layout_w4a8")


if __name__ == "__main__":
    main()
