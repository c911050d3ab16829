"""Writes kquant_fixtures.npz: small seeded Q4_K / Q6_K (and Q8_0 / Q4_0) packed weights with their
dequantized f32 values and dense outputs as produced by the CPU oracle (oracle/ggml_oracle.c).

These pin the oracle against accidental change and give the GPU tests byte-for-byte fixtures.  For
Q4_K / Q6_K they are NOT reference outputs: the reference holds no test vector for the k-quants and
cannot run here, so parity for those two formats is unpinned.
Run: python tests/golden/make_kquant_fixtures.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import oracle as o  # noqa: E402

if __name__ == "__main__":
    out = {}
    rng = np.random.default_rng(20240607)
    for t, (n, k) in {o.Q8_0: (5, 96), o.Q4_0: (5, 96), o.Q4_K: (3, 512), o.Q6_K: (3, 512)}.items():
        name = o.TYPE_NAMES[t]
        w = o.quantize(t, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02), threads=1)
        # sprinkle raw random bytes into one row so every bit pattern of the header fields is exercised
        raw = rng.integers(0, 256, size=w.shape[1], dtype=np.uint8)
        w[n - 1] = raw
        if t in (o.Q4_K,):  # keep fp16 d / dmin finite in the random row
            for b in range(k // 256):
                w[n - 1, b * 144 + 1] &= 0x3B
                w[n - 1, b * 144 + 3] &= 0x3B
        if t == o.Q6_K:
            for b in range(k // 256):
                w[n - 1, b * 210 + 209] &= 0x3B
        if t in (o.Q8_0, o.Q4_0):
            bpb = o.BYTES_PER_BLOCK[t]
            for b in range(k // 32):
                w[n - 1, b * bpb + 1] &= 0x3B
        x = rng.standard_normal((2, k), dtype=np.float32)
        out[f"{name}_w"] = w
        out[f"{name}_x"] = x
        out[f"{name}_deq"] = o.dequantize(t, w, threads=1)
        out[f"{name}_y"] = o.dense(t, w, x, route="decomposed", threads=1)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kquant_fixtures.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path))
