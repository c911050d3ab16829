"""Runs one quantized-dense shape repeatedly so that a profiler can capture its kernel.

    python -m gomlx_b200.profile_case Q4_K 14336 4096 1 [--copies 6] [--rounds 2] [--dtype f32|bf16]

Uploads `copies` device copies of a synthetic [N, K] weight (so consecutive launches stream
different HBM addresses and the L2 cannot serve them) and calls the dense op on each, `rounds`
times.  Small enough for `ncu --set full -k regex:gemv_mma -c 2` to finish in under a minute.
"""
from __future__ import annotations

import argparse

import torch

import gomlx_b200 as g
from gomlx_b200.quantize import synthetic_weights


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("type", choices=["Q8_0", "Q4_0", "Q4_K", "Q6_K"])
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("m", type=int)
    ap.add_argument("--copies", type=int, default=6)
    ap.add_argument("--rounds", type=int, default=2)
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    a = ap.parse_args()
    t = g.GGMLQuantType[a.type]
    w = synthetic_weights(t, a.n, a.k)
    ws = [g.upload(w, t) for _ in range(a.copies)]
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.float32 if a.dtype == "f32" else torch.bfloat16)
    y = torch.empty(a.m, a.n, device="cuda")
    q = g.Quantization(g.QuantizationScheme.GGML, t)
    for _ in range(a.rounds):
        for wr in ws:
            g.backend_fused_quantized_dense(x, wr, None, q, out=y)
    torch.cuda.synchronize()
    print("ok", a.type, a.n, a.k, a.m, float(y.abs().max()))


if __name__ == "__main__":
    main()
