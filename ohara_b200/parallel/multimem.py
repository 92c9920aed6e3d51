"""One-shot all-reduce with the additions done inside NVSwitch (``multimem.ld_reduce``).

Every rank copies its values into a symmetric buffer that is bound to one multicast object; after
a barrier each rank reads the *multicast* address, where one 16-byte load returns the sum of that
offset over all ranks' buffers, and writes the result to its own output. Compared with the
peer-load kernel of :class:`ohara_b200.parallel.peer.PeerRuntime` (every rank reads ``world - 1``
remote copies) each element crosses this GPU's links once, whatever the number of ranks.

The symmetric buffer and its multicast address come from PyTorch's symmetric-memory allocator
(``torch.distributed._symmetric_memory``: ``cuMulticastCreate`` / ``cuMulticastBindMem`` and the
exchange of handles between the processes). The reduction kernel is this package's
(``csrc/multimem.cu``) and has no waits of its own; it runs between two barriers of the peer
runtime, whose waits are bounded and report through the status word:

    copy into my buffer -> barrier -> multimem.ld_reduce into the output -> barrier

so a lost peer ends in ``CollectiveTimeout`` at the next status check instead of a hang. A group
must not use its multicast buffer after one of its ranks has exited: tear the object down first
(``close()``), which is why fault-tolerance tests run with this path off.

Opt-in (``MulticastAllReduce(group)``; the engine does not create one by default). The reference
has no counterpart (its small all-reduces are ``torch.distributed.all_reduce`` calls:
ohara/runtime/engine.py:398-409).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor

from ohara_b200.ops._ext import ext
from ohara_b200.parallel.peer import PeerRuntime


class MulticastAllReduce:
    """In-place sum (or mean) of small contiguous bf16 / fp32 CUDA tensors over ``group``."""

    def __init__(self, group=None, max_bytes: int = 1 << 20, runtime: PeerRuntime | None = None,
                 wait_limit_s: float = 10.0) -> None:
        import torch.distributed._symmetric_memory as symmetric_memory

        if max_bytes % 16:
            raise ValueError("max_bytes must be a multiple of 16")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.max_bytes = max_bytes
        device = torch.device("cuda", torch.cuda.current_device())
        # two halves used alternately: a rank is at most one call ahead of its slowest peer
        self.buffer = symmetric_memory.empty(2 * max_bytes, dtype=torch.uint8, device=device)
        self.handle = symmetric_memory.rendezvous(self.buffer, self.group)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if self.multicast_ptr == 0:
            raise RuntimeError("these devices (or this driver) offer no NVLink multicast: use "
                               "PeerRuntime.all_reduce_ instead")
        self.runtime = runtime if runtime is not None else PeerRuntime(self.group, wait_limit_s)
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def all_reduce_(self, tensor: Tensor, average: bool = False) -> Tensor:
        nbytes = tensor.numel() * tensor.element_size()
        if (not tensor.is_cuda or not tensor.is_contiguous() or nbytes % 16 or nbytes > self.max_bytes
                or tensor.dtype not in (torch.bfloat16, torch.float32)):
            raise ValueError("multicast all-reduce takes contiguous bf16 / fp32 CUDA tensors of a "
                             f"multiple of 16 bytes, at most {self.max_bytes}")
        if self.buffer is None:
            raise RuntimeError("this multicast buffer was closed")
        self.calls += 1
        half = (self.calls % 2) * self.max_bytes
        staging = self.buffer[half : half + nbytes].view(tensor.dtype)
        staging.copy_(tensor.reshape(-1))
        self.runtime.barrier()  # every rank's copy has landed (bounded wait, status word)
        ext().multimem_sum(self.multicast_ptr + half, tensor,
                           1.0 / self.world if average else 1.0)
        # The other half is written next; this half is reused two calls from now, after the
        # barrier of the call in between, by which time every rank has finished reading it.
        return tensor

    def close(self) -> None:
        """Drop the symmetric buffer (collective: every rank calls it before any rank exits)."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self.buffer = None
        self.handle = None
