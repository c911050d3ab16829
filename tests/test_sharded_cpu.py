"""N-sharding + all-gather host logic on two gloo ranks (CPU).  The per-rank compute is injected
(the CPU oracle) because the CUDA library cannot run without a GPU; what is under test is the row
partition, bias slicing and the reassembly of y from the ranks' slices."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import gomlx_b200 as g
        from gomlx_b200.sharded import ShardedQuantizedDense
        from oracle import oracle as o
        t, k = o.Q4_K, 512
        w = o.make_weights(t, n, k, seed=1)
        rng = np.random.default_rng(2)
        bias = rng.standard_normal(n).astype(np.float32)

        def compute(local_w, x, b, act):
            return torch.from_numpy(o.dense(t, local_w, x.numpy(), None if b is None else b.numpy(),
                                            int(act.to_backend()), threads=1))

        layer = ShardedQuantizedDense(w, g.Quantization(g.QuantizationScheme.GGML, g.GGMLQuantType.Q4_K), compute=compute)
        assert sum(c for _, c in layer.ranges) == n
        for m in (1, 3):
            x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
            y = layer(x, torch.from_numpy(bias), g.Activation.SILU)
            want = o.dense(t, w, x.numpy(), bias, o.ACT_SILU, threads=1)
            assert y.shape == (m, n)
            assert np.array_equal(y.numpy(), want), (rank, m, n)
        q.put((rank, "ok"))
    except Exception as e:  # surface the failure in the parent
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n", [64, 48])  # equal shards (all_gather_into_tensor) and ragged shards (list all_gather)
def test_two_rank_all_gather(n, oracle):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
