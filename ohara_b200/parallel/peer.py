"""Peer-memory buffers and collectives for GPUs on one NVLink / NVSwitch node.

``SymmetricBuffer`` is one logical buffer that exists on every rank of a process group: each rank
allocates its copy outside the caching allocator, exports a CUDA IPC handle, and opens the handles
of its peers (exchanged through the c10d object collective, i.e. the control plane). Kernels then
take the table of per-rank base addresses and move data with plain loads and stores over NVLink.

``PeerBuffers`` applies this to the sharded optimizer: the flat gradient and weight buffers become
symmetric, and the per-step reduce-scatter (bf16 -> fp32 sum, mean) and all-gather run as the
kernels in ``csrc/peer.cu`` instead of c10d collectives. Cross-rank ordering is the flag barrier
executed at the start of each kernel; its wait is bounded (``wait_limit_s``) and a timeout
surfaces through ``ops.check_status()`` rather than hanging the device.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ohara_b200.ops._ext import ext


# Stream-ordered waits compare cyclically ("flag - awaited >= 0" as a signed 32-bit number), so
# this value satisfies a wait for any epoch a job can reach.
RELEASE_EPOCH = 0x7FFFFFFF


def release_stream_waits(addresses, device=None, value: int = RELEASE_EPOCH) -> None:
    """Write ``value`` into the 32-bit flags at ``addresses`` (device memory of *this* GPU) with
    stream-ordered stores on a stream of their own.

    A copy stream that is parked in a stream-ordered wait for a flag a lost peer will never write
    holds up every later ``wait_event`` / ``synchronize`` of the process. The awaited flags live in
    this rank's own memory, so the host can always satisfy them; the queued copies then run (on
    stale data, the step is lost anyway) and the streams drain. Safe to call from another thread
    (the step watchdog) while the main thread is blocked in ``synchronize``."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(device):
        stream = torch.cuda.Stream(device=device)
        with torch.cuda.stream(stream):
            for address in addresses:
                ext().stream_write_value32(int(address), int(value))


class SymmetricBuffer:
    """``nbytes`` of device memory per rank, addressable from every rank of ``group``."""

    def __init__(self, nbytes: int, group=None, device: torch.device | None = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(nbytes)
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.local, handle = ext().peer_alloc(self.nbytes, index)
        handles: list[bytes | None] = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.views: list[torch.Tensor] = []
        for r, peer_handle in enumerate(handles):
            if r == self.rank:
                self.views.append(self.local)
            else:
                self.views.append(ext().peer_open(peer_handle, self.nbytes, index))
        self.pointers = [v.data_ptr() for v in self.views]

    def typed(self, dtype: torch.dtype, rank: int | None = None) -> torch.Tensor:
        """This rank's (or ``rank``'s) copy viewed as a 1-D tensor of ``dtype``."""
        view = self.local if rank is None else self.views[rank]
        return view.view(dtype)


class PeerRuntime:
    """Signal pads + a monotonically increasing barrier epoch shared by all collectives of a
    group. Every rank must issue the same sequence of collectives."""

    ONE_SHOT_BYTES = 1 << 20
    # Up to this size the all-reduce is a single-block kernel whose epoch lives on the device: it
    # can be captured in a CUDA graph and replayed (decode-time tensor parallelism).
    SMALL_BYTES = 256 << 10

    def __init__(self, group=None, wait_limit_s: float = 10.0) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.wait_limit_s = wait_limit_s
        self.pads = SymmetricBuffer(4096, group)
        self.epoch = 0
        self._reduce_buffers = None
        self._small = None
        # Everyone has opened everyone's pad before the first kernel may signal.
        dist.barrier(group=group)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def barrier(self) -> None:
        ext().peer_barrier(self.pads.pointers, self.rank, self.next_epoch(), self.wait_limit_s)

    def all_reduce_(self, tensor: torch.Tensor, average: bool = False) -> torch.Tensor:
        """In-place one-shot all-reduce of a small contiguous bf16 / fp32 CUDA tensor: every rank
        writes its values into a symmetric buffer and, after the flag barrier, sums all copies
        itself (a single NVLink round trip). Falls back to the c10d collective for tensors larger
        than ``ONE_SHOT_BYTES``, where a bandwidth-optimal algorithm wins."""
        nbytes = tensor.numel() * tensor.element_size()
        if (nbytes <= self.SMALL_BYTES and tensor.is_contiguous()
                and tensor.dtype in (torch.bfloat16, torch.float32)):
            return self._all_reduce_small(tensor, average)
        if (nbytes > self.ONE_SHOT_BYTES or not tensor.is_contiguous()
                or tensor.dtype not in (torch.bfloat16, torch.float32)):
            dist.all_reduce(tensor, group=self.group)
            if average:
                tensor /= self.world
            return tensor
        if self._reduce_buffers is None:
            self._reduce_buffers = [SymmetricBuffer(self.ONE_SHOT_BYTES, self.group) for _ in range(2)]
            self._reduce_count = 0
            dist.barrier(group=self.group)
        self._reduce_count += 1
        # Two buffers alternate: a rank can only be one call ahead of a peer (the barrier inside
        # the kernel), so the buffer it overwrites was last read two calls ago.
        buffer = self._reduce_buffers[self._reduce_count % 2]
        buffer.typed(tensor.dtype)[: tensor.numel()].copy_(tensor.view(-1))
        ext().peer_all_reduce(buffer.pointers, self.pads.pointers, tensor,
                              1.0 / self.world if average else 1.0, self.rank, self.next_epoch(),
                              self.wait_limit_s)
        return tensor


    def _all_reduce_small(self, tensor: torch.Tensor, average: bool) -> torch.Tensor:
        if self._small is None:
            # Set-up is collective; it happens at the first small all-reduce, which every rank
            # reaches at the same point of the program (never inside a graph capture: warm up
            # one step first).
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("run one eager step before capturing a graph that all-reduces")
            buffers = SymmetricBuffer(2 * self.SMALL_BYTES, self.group)
            pads = SymmetricBuffer(4096, self.group)
            counter = torch.zeros(1, dtype=torch.int32, device=buffers.device)
            self._small = (buffers, pads, counter)
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        buffers, pads, counter = self._small
        slot_elems = self.SMALL_BYTES // tensor.element_size()
        ext().peer_all_reduce_small(buffers.pointers, pads.pointers, counter, tensor, slot_elems,
                                    1.0 / self.world if average else 1.0, self.rank,
                                    self.wait_limit_s)
        return tensor


class PeerBuffers:
    """Symmetric gradient / weight buffers of a :class:`ShardedOptimizer` and their collectives."""

    def __init__(self, optimizer, group) -> None:
        self.runtime = PeerRuntime(group)
        self.region = optimizer.region
        self.world = optimizer.world
        self.rank = optimizer.rank
        elements = optimizer.region * optimizer.world
        itemsize = torch.empty((), dtype=optimizer.wire_dtype).element_size()
        self.grads = SymmetricBuffer(elements * itemsize, group)
        self.weights = SymmetricBuffer(elements * itemsize, group)
        self.itemsize = itemsize
        grad_flat = self.grads.typed(optimizer.wire_dtype)
        weight_flat = self.weights.typed(optimizer.wire_dtype)
        weight_flat.copy_(optimizer.weight_flat)
        optimizer.grad_flat = grad_flat
        optimizer.weight_flat = weight_flat
        optimizer._bind_shadows()
        torch.cuda.synchronize()
        dist.barrier(group=group)

    @classmethod
    def create(cls, optimizer, group):
        if optimizer.wire_dtype != torch.bfloat16:
            return None
        if optimizer.world > 16:
            return None
        return cls(optimizer, group)

    def reduce_scatter_mean(self, grad_flat: torch.Tensor, out: torch.Tensor) -> None:
        assert grad_flat.data_ptr() == self.grads.local.data_ptr()
        ext().peer_reduce_scatter_mean(
            self.grads.pointers, self.runtime.pads.pointers, out, self.region, self.rank,
            self.runtime.next_epoch(), self.runtime.wait_limit_s,
        )

    def all_gather(self, weight_flat: torch.Tensor) -> None:
        assert weight_flat.data_ptr() == self.weights.local.data_ptr()
        ext().peer_all_gather(
            self.weights.pointers, self.runtime.pads.pointers, self.region * self.itemsize,
            self.rank, self.runtime.next_epoch(), self.runtime.wait_limit_s,
        )
