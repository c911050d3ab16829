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

from typing import Callable, Optional, Sequence

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


class PeerScatterBuffers:
    """One symmetric-memory buffer per rank, mapped into every rank of ``group`` (CUDA peer memory over
    NVLink), for layers whose kernels write their output slice straight into all peers.

    Allocate one instance per process group and carve the regions of all layers out of it (one rendezvous,
    one set of sync words).

    ``floats`` float32 values are allocated on every rank; ``ptr(rank, offset)`` is the device address,
    in this process, of element ``offset`` of ``rank``'s buffer, and ``local`` is this rank's buffer as a
    tensor.  ``barrier()`` enqueues a device-side barrier of all ranks on the current stream: after it,
    every store issued before it on any rank is visible to every rank.
    """

    SYNC_WORDS = 64  # the first 256 bytes of every rank's buffer hold the cross-GPU sync words

    def __init__(self, floats: int, device: int, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._all = symm_mem.empty(floats + self.SYNC_WORDS, dtype=torch.float32, device=torch.device("cuda", device))
        self.handle = symm_mem.rendezvous(self._all, group.group_name)
        self._ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._all.zero_()
        self._sync_peers = None
        self.local = self._all[self.SYNC_WORDS:]
        torch.cuda.synchronize()
        self.handle.barrier(channel=0)  # every rank's sync words are zero before anyone signals
        torch.cuda.synchronize()

    def ptr(self, rank: int, offset: int = 0) -> int:
        return self._ptrs[rank] + 4 * (self.SYNC_WORDS + offset)

    def sync_ptr(self, rank: int) -> int:
        return self._ptrs[rank]

    def barrier(self, native: bool = False) -> None:
        """Device-side rendezvous of all ranks on the current stream.  ``native``: the library's one-CTA barrier
        kernel (``b200q_peer_barrier``, overlaps the next launch's prologue); otherwise the symmetric-memory
        barrier of torch."""
        if not native:
            self.handle.barrier(channel=0)
            return
        import ctypes
        from . import _native as nat
        if self._sync_peers is None:
            peers = [self.sync_ptr(r) for r in range(self.world) if r != self.rank]
            self._sync_peers = (ctypes.c_void_p * max(1, len(peers)))(*peers)
        nat.check(nat.lib().b200q_peer_barrier(self._all.device.index, ctypes.c_void_p(self.sync_ptr(self.rank)), self._sync_peers,
                                               self.world - 1, self.rank, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def barrier_timed_out(self) -> bool:
        """True if a native barrier gave up waiting for a peer (synchronizes the device)."""
        torch.cuda.synchronize()
        return int(self._all[:self.SYNC_WORDS].view(torch.int32)[25].item()) == 2


class PeerScatterDense:
    """Row-sharded decode dense whose all-gather is fused into the GEMV epilogue: each rank's kernel
    stores its slice of ``y`` into its own and every peer's result buffer (``b200q_dense_scatter``).
    The result region is ``[max_m, N_total]`` float32 at ``offset`` of a shared ``PeerScatterBuffers``;
    call ``buffers.barrier()`` before any rank reads it."""

    def __init__(self, weights, quant: Quantization, buffers: PeerScatterBuffers, offset: int, max_m: int, device: int,
                 n_total: Optional[int] = None):
        """``weights``: the full packed matrix (this rank's rows are uploaded), or a ResidentWeight that
        already holds this rank's shard together with ``n_total``."""
        import ctypes
        self.quant, self.buffers, self.offset, self.max_m = quant, buffers, offset, max_m
        if isinstance(weights, ResidentWeight):
            self.local, self.n_total = weights, int(n_total if n_total is not None else weights.n_total)
        else:
            self.n_total = int(weights.shape[0])
            self.local = upload(weights, quant.ggml_type, device, shard=(buffers.rank, buffers.world))
        peers = [buffers.ptr(r, offset) for r in range(buffers.world) if r != buffers.rank]
        self._peer_arr = (ctypes.c_void_p * max(1, len(peers)))(*peers)
        self._n_peers = len(peers)
        self._sync_arr = (ctypes.c_void_p * max(1, len(peers)))(
            *[buffers.sync_ptr(r) for r in range(buffers.world) if r != buffers.rank])
        self.y = buffers.local[offset:offset + max_m * self.n_total].view(max_m, self.n_total)

    def __call__(self, x: torch.Tensor, bias=None, activation: Activation = Activation.NONE, wait: bool = False,
                 signal: bool = False) -> torch.Tensor:
        """``signal``: publish this kernel's completion to all ranks; ``wait``: do not start until every rank
        has published as many completions as this rank (in-kernel ordering, no extra launch)."""
        import ctypes
        from . import _native as nat
        x2 = x.reshape(-1, self.local.k).contiguous()
        m = x2.shape[0]
        if m > self.max_m:
            raise ValueError(f"batch {m} exceeds the {self.max_m} rows reserved for this layer")
        b = None if bias is None else bias[self.local.row_begin:self.local.row_begin + self.local.n].contiguous()
        nat.check(nat.lib().b200q_dense_scatter(
            self.local.handle, ctypes.c_void_p(x2.data_ptr()), nat.F32 if x2.dtype == torch.float32 else nat.BF16, m,
            ctypes.c_void_p(b.data_ptr()) if b is not None else None, int(activation.to_backend()),
            ctypes.c_void_p(self.buffers.ptr(self.buffers.rank, self.offset)), self._peer_arr, self._n_peers,
            self.n_total, self.local.row_begin, ctypes.c_void_p(self.buffers.sync_ptr(self.buffers.rank)), self._sync_arr,
            self.buffers.rank, (1 if wait else 0) | (2 if signal else 0),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.y[:m]

    def free(self) -> None:
        self.local.free()


def peer_scatter_batch(layers: Sequence["PeerScatterDense"], x: torch.Tensor, biases=None, activations=None,
                       wait: bool = False, signal: bool = False):
    """Several row-sharded projections on the same ``x`` in one launch (``b200q_dense_batch_scatter``): q+k or
    gate+up of a decoder layer.  The layers must share one ``PeerScatterBuffers``, format and K.  Returns the
    list of gathered result views (valid on every rank after the next ``buffers.barrier()``)."""
    import ctypes
    from . import _native as nat
    first = layers[0]
    bufs, n = first.buffers, len(layers)
    if any(l.buffers is not bufs for l in layers):
        raise ValueError("peer_scatter_batch: the layers must share one PeerScatterBuffers")
    x2 = x.reshape(-1, first.local.k).contiguous()
    m = x2.shape[0]
    if any(m > l.max_m for l in layers):
        raise ValueError(f"batch {m} exceeds the rows reserved for a layer")
    acts = list(activations) if activations is not None else [Activation.NONE] * n
    bs = []
    for l, b in zip(layers, biases if biases is not None else [None] * n):
        bs.append(None if b is None else b[l.local.row_begin:l.local.row_begin + l.local.n].contiguous())
    peers_of = [r for r in range(bufs.world) if r != bufs.rank]
    handles = (ctypes.c_uint64 * n)(*[l.local.handle for l in layers])
    bias_arr = (ctypes.c_void_p * n)(*[b.data_ptr() if b is not None else None for b in bs])
    act_arr = (ctypes.c_int * n)(*[int(a.to_backend()) for a in acts])
    y_loc = (ctypes.c_void_p * n)(*[bufs.ptr(bufs.rank, l.offset) for l in layers])
    y_peer = (ctypes.c_void_p * max(1, n * len(peers_of)))(*[bufs.ptr(r, l.offset) for l in layers for r in peers_of])
    lds = (ctypes.c_int64 * n)(*[l.n_total for l in layers])
    offs = (ctypes.c_int64 * n)(*[l.local.row_begin for l in layers])
    nat.check(nat.lib().b200q_dense_batch_scatter(
        n, handles, ctypes.c_void_p(x2.data_ptr()), nat.F32 if x2.dtype == torch.float32 else nat.BF16, m, bias_arr, act_arr,
        y_loc, y_peer, len(peers_of), lds, offs, ctypes.c_void_p(bufs.sync_ptr(bufs.rank)), first._sync_arr, bufs.rank,
        (1 if wait else 0) | (2 if signal else 0), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return [l.y[:m] for l in layers]
