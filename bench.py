#!/usr/bin/env python
"""Headline benchmark: decode weight-GB/s of the Llama-3-8B-shaped stack of quantized projections.

Workload (BASELINE.json configs[3]): 32 layers x {q 4096->4096, k 4096->1024, o 4096->4096,
gate 4096->14336 (+SiLU), up 4096->14336 in Q4_K; v 4096->1024, down 14336->4096 in Q6_K}, one
decode token (batch 1, override with --batch), weights from N(0, 0.02) quantized row-wise,
4,444,913,664 packed weight bytes read per step.  With N GPUs every matrix is split by output rows,
each rank computes its slice and the outputs are all-gathered (NCCL); total work is fixed (strong
scaling).  One step = the 224 projections of one token pass, replayed as one CUDA graph.

Prints ONE JSON line (rank 0).  `value` = weight bytes of the whole job / max-over-ranks device
time with inputs resident in HBM; `e2e` = same metric with the step's activations copied from
pinned host memory and the results copied back inside the timed region.

`--impl reference` times the CPU restatement of the reference's algorithm (oracle/, the one place
besides the `cpu_baseline` leg where this file executes it) on the box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = 32
# name, ggml type id, N (output rows), K, fused activation
PROJECTIONS = [
    ("q", 12, 4096, 4096, "none"), ("k", 12, 1024, 4096, "none"), ("v", 14, 1024, 4096, "none"),
    ("o", 12, 4096, 4096, "none"), ("gate", 12, 14336, 4096, "silu"), ("up", 12, 14336, 4096, "none"),
    ("down", 14, 4096, 14336, "none"),
]
BPB = {12: 144, 14: 210}
WORKLOAD = "llama3-8b-shaped decoder stack, 32 layers x 7 quantized projections (Q4_K; v/down Q6_K)"


def host_threads() -> int:
    """Host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which is not the box's size)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def layer_weight_bytes() -> int:
    return sum(n * (k // 256) * BPB[t] for _, t, n, k, _ in PROJECTIONS)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "source": "fallback (6.65 TB/s, earlier measurement on this pool)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.path = device, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [c.strip() for c in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except (OSError, ValueError, TypeError):
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------- reference arm
def cpu_sample(batch: int, repeats: int, threads: int):
    """Times `repeats` passes of ONE decoder layer (7 projections) through the CPU restatement of the
    reference's fused route.  Returns (seconds per layer pass, weight bytes per layer pass)."""
    from oracle import oracle as o
    from gomlx_b200.quantize import synthetic_weights
    from gomlx_b200 import GGMLQuantType
    o.build()
    rng = np.random.default_rng(0)
    ws = [(t, synthetic_weights(GGMLQuantType(t), n, k, 0.02, seed=i)) for i, (_, t, n, k, _) in enumerate(PROJECTIONS)]
    xs = {k: rng.standard_normal((batch, k)).astype(np.float32) for k in (4096, 14336)}
    acts = {"none": o.ACT_NONE, "silu": o.ACT_SILU}

    def layer():
        for (t, w), (_, _, _, k, act) in zip(ws, PROJECTIONS):
            o.dense(t, w, xs[k], None, acts[act], route="fused", threads=threads)

    layer()
    t0 = time.perf_counter()
    for _ in range(repeats):
        layer()
    return (time.perf_counter() - t0) / repeats, layer_weight_bytes()


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as o
    threads = host_threads()
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sample(args.batch, 1, threads)
    times = []
    for _ in range(args.steps):
        sec, nbytes = cpu_sample(args.batch, 1, threads)
        times.append(sec)
    sec = float(np.mean(times))
    value = nbytes / sec / 1e9
    sample = f"1 of {LAYERS} layers (7 projections, {nbytes} weight bytes) per step, batch {args.batch}, fused CPU route"
    print(json.dumps({
        "impl": "reference", "metric": "decode_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": args.batch, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------------- CUDA arm
def run_cuda(args) -> None:
    import torch
    import torch.distributed as dist

    import gomlx_b200 as g
    from gomlx_b200 import _native as nat
    from gomlx_b200.quantize import synthetic_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: gomlx_b200 has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    nat.lib()  # fails loudly if libb200q.so is missing

    batch = args.batch
    acts = {"none": g.ActivationType.NONE, "silu": g.ActivationType.SILU}
    quant = {t: g.Quantization(g.QuantizationScheme.GGML, g.GGMLQuantType(t)) for t in (12, 14)}

    # One seeded layer; every layer gets its own device copy so each step really streams all bytes.
    packed = [synthetic_weights(g.GGMLQuantType(t), n, k, 0.02, seed=i) for i, (_, t, n, k, _) in enumerate(PROJECTIONS)]
    weights = []  # [layer][proj] -> ResidentWeight holding this rank's rows
    for _ in range(LAYERS):
        weights.append([g.upload(w, g.GGMLQuantType(t), local, shard=(rank, world) if world > 1 else None)
                        for w, (_, t, _, _, _) in zip(packed, PROJECTIONS)])
    local_bytes = sum(w.device_bytes for layer in weights for w in layer)

    # N > 1: the all-gather of every projection's output is fused into the GEMV epilogue (peer stores
    # over NVLink into one symmetric buffer per rank); NCCL all-gather is the fallback / comparison.
    gather = "none" if world == 1 else args.gather
    peer_layers = None
    if gather == "peer":
        try:
            from gomlx_b200.sharded import PeerScatterBuffers, PeerScatterDense, peer_scatter_batch
            per_layer = sum(n for _, _, n, _, _ in PROJECTIONS) * batch
            bufs = PeerScatterBuffers(LAYERS * per_layer, local)
            peer_layers, off = [], 0
            for li in range(LAYERS):
                row = []
                for pi, (_, t, n, _, _) in enumerate(PROJECTIONS):
                    row.append(PeerScatterDense(weights[li][pi], quant[t], bufs, off, batch, local, n_total=n))
                    off += batch * n
                peer_layers.append(row)
        except Exception as e:  # symmetric memory unavailable: fall back to NCCL
            print(f"[bench] peer scatter unavailable ({e!r}); using NCCL all-gather", file=sys.stderr)
            gather, peer_layers = "nccl", None

    gen = torch.Generator(device="cpu").manual_seed(1234)
    x_host = {k: torch.randn(batch, k, generator=gen).pin_memory() for k in (4096, 14336)}
    x_dev = {k: v.to(dev) for k, v in x_host.items()}
    y_loc = [[torch.empty(batch, w.n, device=dev) for w in layer] for layer in weights]
    if gather == "peer":
        y_full = [[d.y for d in row] for row in peer_layers]
    elif gather == "nccl":
        y_full = [[torch.empty(world * batch, w.n, device=dev) for w in layer] for layer in weights]
    else:
        y_full = y_loc
    y_host = torch.empty_like(y_full[-1][-1], device="cpu").pin_memory()

    act_types = {"none": g.Activation.NONE, "silu": g.Activation.SILU}
    # ranks are ordered where a real decoder layer consumes gathered outputs: after q/k/v, o, gate/up, down
    sync_after = {"v", "o", "up", "down"}

    def step():
        pending = False  # a signal has been published that the next launch has to wait for
        for li in range(LAYERS):
            for pi, (name, t, _, k, act) in enumerate(PROJECTIONS):
                qkv = args.fuse_shared_input >= 2 and args.order == "barrier"  # v beside q+k (no sync words on mixed calls)
                if gather == "peer" and args.fuse_shared_input and (name in ("k", "up") or (name == "v" and qkv)):
                    continue  # computed together with q / gate
                if gather == "peer":
                    sig = args.order == "kernel" and name in sync_after
                    if args.fuse_shared_input and name in ("q", "gate"):  # q+k(+v), gate+up: one call each
                        group = [pi, pi + 1] + ([pi + 2] if (name == "q" and qkv) else [])
                        sig = sig or (args.order == "kernel" and any(PROJECTIONS[pj][0] in sync_after for pj in group))
                        peer_scatter_batch([peer_layers[li][pj] for pj in group], x_dev[k], None,
                                           [act_types[PROJECTIONS[pj][4]] for pj in group], wait=pending, signal=sig)
                        last = PROJECTIONS[group[-1]][0]
                    else:
                        peer_layers[li][pi](x_dev[k], None, act_types[act], wait=pending, signal=sig)
                        last = name
                    pending = sig
                    if args.order == "barrier" and last in sync_after:
                        bufs.barrier(native=args.barrier == "native")
                elif gather == "nccl":
                    g.backend_fused_quantized_dense(x_dev[k], weights[li][pi], None, quant[t], acts[act], out=y_loc[li][pi])
                    dist.all_gather_into_tensor(y_full[li][pi], y_loc[li][pi])
                elif args.fuse_shared_input and name in ("q", "gate"):
                    # q, k, v and gate, up read the same activations: one call each.  Matrices of one format
                    # share a launch (q+k, gate+up); v (Q6_K) runs next to q+k on its share of the SMs.
                    group = [pi, pi + 1] + ([pi + 2] if (name == "q" and args.fuse_shared_input >= 2) else [])
                    g.backend_fused_quantized_dense_batch(
                        x_dev[k], [weights[li][pj] for pj in group], None, [quant[PROJECTIONS[pj][1]] for pj in group],
                        [acts[PROJECTIONS[pj][4]] for pj in group], outs=[y_loc[li][pj] for pj in group])
                elif args.fuse_shared_input and (name in ("k", "up") or (name == "v" and args.fuse_shared_input >= 2)):
                    pass  # computed together with q / gate
                else:
                    g.backend_fused_quantized_dense(x_dev[k], weights[li][pi], None, quant[t], acts[act], out=y_loc[li][pi])

    if gather == "peer" and args.order == "kernel":
        _inner = step

        def step():  # close the step: the last signal is consumed by a device barrier, not by a next launch
            _inner()
            bufs.barrier(native=args.barrier == "native")

    def select(pred):
        def run():
            for li in range(LAYERS):
                for pi, (name, t, _, k, act) in enumerate(PROJECTIONS):
                    if pred(name):
                        g.backend_fused_quantized_dense(x_dev[k], weights[li][pi], None, quant[t], acts[act],
                                                        out=y_loc[li][pi])
        return run

    def capture(fn):
        fn()
        torch.cuda.synchronize()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps: int) -> float:
        """ms per step: CUDA events on the launching stream, barrier + synchronize on both sides."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    graph = capture(step)
    for _ in range(max(args.warmup, 3)):
        graph.replay()

    with ClockSampler(local) as clocks:
        ms = timed(graph.replay, args.steps)

        def e2e_step():
            for k in x_dev:
                x_dev[k].copy_(x_host[k], non_blocking=True)
            graph.replay()
            y_host.copy_(y_full[-1][-1], non_blocking=True)
            torch.cuda.current_stream().synchronize()

        e2e_step()
        ms_e2e = timed(e2e_step, args.steps)

        # Dominant kernel: the Q4_K decode GEMV on the gate/up matrices (64 of the 224 launches,
        # 47 % of the bytes).  Its launches over all 32 layers are replayed alone and timed.
        gu = capture(select(lambda name: name in ("gate", "up")))
        gu.replay()
        ms_gu = timed(gu.replay, max(3, args.steps))
    clk = clocks.summary()

    total_bytes = LAYERS * layer_weight_bytes()
    value = total_bytes / (ms * 1e-3) / 1e9
    e2e_value = total_bytes / (ms_e2e * 1e-3) / 1e9
    gu_weights = [weights[li][pi] for li in range(LAYERS) for pi in (4, 5)]
    gu_bytes = sum(w.n * (w.k // 256) * 144 for w in gu_weights) / len(gu_weights)  # algorithmic bytes / launch
    gu_us = ms_gu * 1e3 / len(gu_weights)
    pk = peaks()
    achieved = gu_bytes / (gu_us * 1e-6) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "gemv_mma_kernel<Q4_K> (gate/up 14336x4096 rows/%d)" % world,
        "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
        "peak_source": pk["source"], "us_per_launch": gu_us, "bytes_per_launch": gu_bytes,
        # dram__bytes_read + dram__bytes_write per launch: ncu measured 33.10 MB for the 33.03 MB launch
        # at N = 1 (profiles/gemv_q4k_14336x4096_m1.md); traffic grows in proportion to the rows a rank holds
        "traffic": args.traffic if args.traffic is not None else gu_bytes * (33089792.0 / 33030144.0),
        "traffic_source": "ncu capture of the N=1 launch, scaled by bytes per launch",
    }

    out = {
        "metric": "decode_weight_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": ("u4/u6 codes x 15-bit activations in int8 tensor-core MMAs (s32), block scales in f32" if batch == 1 else "f16 multiply / f32 accumulate on packed u8 blocks"), "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": batch, "weight_bytes_per_step": total_bytes,
                   "parallelism": f"rows/{world}" + {"none": "", "nccl": " + NCCL all-gather per projection",
                                                           "peer": " + all-gather fused into the GEMV epilogue (NVLink peer stores), " +
                                                                   ("4 device barriers per layer (" + args.barrier + ")" if args.order == "barrier" else "ranks ordered inside the kernels at 4 points per layer")}[gather],
                   "inputs": "fixed N(0,1) activations per projection (outputs not chained)",
                   "l2": f"no flush: {local_bytes / 1e6:.0f} MB of weights per GPU per step exceed the 126 MB L2",
                   "launch": (("one CUDA graph per step; q+k and gate+up of a layer share one launch each (160 launches)" +
                               ("; v runs next to q+k on its share of the SMs" if (args.fuse_shared_input >= 2 and (gather == "none" or (gather == "peer" and args.order == "barrier"))) else ""))
                              if (args.fuse_shared_input and gather in ("none", "peer")) else "one CUDA graph of 224 GEMV launches per step")},
        "roofline": roofline,
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(sum(v.numel() * 4 for v in x_host.values())),
                "d2h_bytes_per_step": int(y_host.numel() * 4)},
        "gpu_launches": int(args.steps * LAYERS * (5 if (args.fuse_shared_input and gather in ("none", "peer")) else len(PROJECTIONS))),
        "clocks": clk,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as o  # checker timed as the CPU baseline; never on the product path
            threads = host_threads()
            sec, nbytes = cpu_sample(batch, 2, threads)
            out["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                   "sample": f"1 of {LAYERS} layers (7 projections, {nbytes} weight bytes), 2 passes, "
                                             f"batch {batch}, fused CPU route"}
        print(json.dumps(out))
    for layer in weights:
        for w in layer:
            w.free()
    if world > 1:
        # Tearing the NCCL communicator down (destroy_process_group) has been seen to block for
        # minutes on multi-GPU boxes; every rank is past its last collective here, so leave directly.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fuse-shared-input", type=int, default=2,
                    help="1: q+k and gate+up (same activations, format and K) run as one launch each; "
                         "2: also v (Q6_K) in the q+k call, side by side on its share of the SMs")
    ap.add_argument("--order", default="barrier", choices=["barrier", "kernel"],
                    help="N > 1 with --gather peer: order the ranks with device barriers between launches (default) "
                         "or with completion counters inside the GEMV kernels (experimental)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"], help="N > 1: how outputs are all-gathered")
    ap.add_argument("--barrier", default="torch", choices=["native", "torch"],
                    help="N > 1 with --gather peer: the library's one-CTA barrier kernel or torch's symmetric-memory barrier")
    ap.add_argument("--traffic", type=float, default=None, help="dram bytes per launch of the dominant kernel (ncu)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
