"""Output-feature (N) sharding of a quantized dense layer over the ranks of one node.

Rows of the packed ``[N, bytesPerRow]`` weight are independent output features and blocks never
straddle rows (gomlx/gomlx ml/ggml/dequant.go:31-35), so rank r keeps a contiguous row range,
computes ``y[:, rows_r]`` from the replicated activations, and one all-gather along N rebuilds
``y`` on every rank.  The reference's graph layer offers only AllReduce
(core/graph/distributed.go:217-248); the gather here is new functionality below its API.

One process per GPU; the collective is ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in
the CPU tests, where ``compute`` is injected because the CUDA library cannot run there).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from .activation import Type as Activation
from .nn import Quantization, ResidentWeight, backend_fused_quantized_dense, shard_rows, upload


class ShardedQuantizedDense:
    """``y = act(x @ dequant(W)^T + bias)`` with W split by rows over ``group``.

    ``weights`` is the full packed matrix (every rank passes the same bytes, only its own rows are
    uploaded).  ``compute(local_weight, x, bias_slice, activation) -> y_local [M, n_local]`` may be
    injected for tests; by default the resident weight runs through the CUDA library.
    """

    def __init__(self, weights, quant: Quantization, group: Optional[dist.ProcessGroup] = None, device: int = 0,
                 compute: Optional[Callable] = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.quant = quant
        self.n_total = int(weights.shape[0])
        self.ranges = [shard_rows(self.n_total, r, self.world) for r in range(self.world)]
        self.begin, self.count = self.ranges[self.rank]
        self.equal = len({c for _, c in self.ranges}) == 1
        self._compute = compute
        if compute is None:
            self.local: object = upload(weights, quant.ggml_type, device, shard=(self.rank, self.world))
        else:
            self.local = weights[self.begin:self.begin + self.count]

    def local_forward(self, x, bias=None, activation: Activation = Activation.NONE):
        b = None if bias is None else bias[self.begin:self.begin + self.count]
        if self._compute is not None:
            return self._compute(self.local, x, b, activation)
        return backend_fused_quantized_dense(x, self.local, b, self.quant, activation.to_backend())

    def __call__(self, x, bias=None, activation: Activation = Activation.NONE) -> torch.Tensor:
        y_local = self.local_forward(x, bias, activation)
        y_local = y_local.reshape(-1, self.count).contiguous()
        if self.world == 1:
            return y_local
        m = y_local.shape[0]
        if self.equal:
            gathered = torch.empty((self.world * m, self.count), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(gathered, y_local, group=self.group)
            if m == 1:
                return gathered.reshape(1, self.n_total)
            return gathered.reshape(self.world, m, self.count).permute(1, 0, 2).reshape(m, self.n_total)
        # Ragged shards (N not a multiple of 16 * world): pad to the widest shard, gather, trim.
        widest = max(c for _, c in self.ranges)
        padded = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
        padded[:, :self.count] = y_local
        gathered = torch.empty((self.world * m, widest), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, padded, group=self.group)
        gathered = gathered.reshape(self.world, m, widest)
        return torch.cat([gathered[r, :, :c] for r, (_, c) in enumerate(self.ranges)], dim=1)

    def free(self) -> None:
        if isinstance(self.local, ResidentWeight):
            self.local.free()
