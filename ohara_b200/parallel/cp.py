"""Context parallelism: causal attention over a sequence sharded in contiguous chunks.

Rank ``r`` of the group holds queries, keys and values of chunk ``r``. Its queries need the keys
and values of chunks ``0 .. r``. The exchange is overlapped with attention instead of preceding it:

1. every rank copies its ``(K, V)`` chunk into a symmetric staging buffer and publishes a flag;
2. a side stream pulls the earlier chunks with the copy engines (stream-ordered wait on the
   owner's flag, peer-to-peer copy) while
3. the main stream already runs causal flash attention of the local queries against the *local*
   chunk;
4. once the remote chunks have landed, a second, non-causal flash attention pass covers them and
   the two partial results are merged through their log-sum-exp.

The backward pass runs the two flash-attention backward kernels with the merged statistics, then
returns the key/value gradients of remote chunks to their owners with peer-to-peer copies into
per-source slots that the owner sums. Staging and slot buffers are double-buffered and every reuse
is preceded by the bounded flag barrier of :class:`PeerRuntime`.

Staged layout is ``(T_local, B, 2, kv_heads, D)`` so that consecutive chunks form one sequence with
a uniform token stride for any batch size.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import Tensor

from ohara_b200.ops._ext import ext
from ohara_b200.parallel.peer import PeerRuntime, SymmetricBuffer

_KV_SLOT = 0


class CPWorkspace:
    def __init__(self, group, chunk_elements: int, wait_limit_s: float = 10.0) -> None:
        """``chunk_elements``: elements of one staged chunk, ``T_local * B * 2 * kv_heads * D``."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("context parallelism over peer memory supports up to 8 ranks")
        self.chunk_elements = chunk_elements
        self.runtime = PeerRuntime(group, wait_limit_s)
        self.flags = SymmetricBuffer(4096, group)
        self.stage = [SymmetricBuffer(chunk_elements * 2, group) for _ in range(2)]
        self.grad_slots = [SymmetricBuffer(chunk_elements * 2 * self.world, group) for _ in range(2)]
        self.device = self.flags.device
        self.gathered = [torch.empty(self.world * chunk_elements, device=self.device,
                                     dtype=torch.bfloat16) for _ in range(2)]
        self.copy_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.kv_epoch = 0
        self.grad_epoch = 0
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def exchange_kv(self, kv_local: Tensor):
        """Stage this rank's ``(T_local, B, 2, Hk, D)`` chunk and start pulling chunks ``0 .. rank-1``.
        Returns ``(remote, arrived)``: a view ``(rank * T_local, B, 2, Hk, D)`` of the earlier chunks
        in sequence order (valid until two exchanges later) and the event that marks its arrival."""
        if kv_local.numel() > self.chunk_elements:
            raise ValueError("key/value chunk exceeds the workspace")
        self.runtime.barrier()  # every rank has finished pulling from the buffer about to be reused
        self.kv_epoch += 1
        epoch, index = self.kv_epoch, self.kv_epoch % 2
        count = kv_local.numel()
        self.stage[index].typed(torch.bfloat16)[:count].copy_(kv_local.reshape(-1))
        ext().tp_signal(self.flags.pointers, _KV_SLOT, self.rank, epoch)
        main = torch.cuda.current_stream(self.device)
        staged = torch.cuda.Event()
        staged.record(main)
        self.copy_stream.wait_event(staged)
        landing = self.gathered[index]
        arrived = torch.cuda.Event()
        with torch.cuda.stream(self.copy_stream):
            # nearest chunk first: it is the last one the second attention pass reads, but the
            # first whose owner is likely to be ready
            for src in range(self.rank - 1, -1, -1):
                ext().stream_wait_value32(self.flags.pointers[self.rank] + 4 * (_KV_SLOT + src), epoch)
                remote = self.stage[index].typed(torch.bfloat16, rank=src)[:count]
                landing[src * count : (src + 1) * count].copy_(remote)
            arrived.record(self.copy_stream)
        view = landing[: self.rank * count].view(self.rank * kv_local.shape[0], *kv_local.shape[1:])
        return view, arrived

    def return_kv_grads(self, dkv_remote: Tensor | None, dkv_local: Tensor) -> Tensor:
        """Send the gradients of chunks ``0 .. rank-1`` (``(rank * T_local, B, 2, Hk, D)``) to their
        owners and return ``dkv_local`` plus what the later ranks sent for this rank's chunk."""
        count = dkv_local.numel()
        self.runtime.barrier()  # owners have finished summing the previous slots
        self.grad_epoch += 1
        buffer = self.grad_slots[self.grad_epoch % 2]
        if dkv_remote is not None and self.rank > 0:
            flat = dkv_remote.reshape(-1)
            for owner in range(self.rank):
                slot = buffer.typed(torch.bfloat16, rank=owner)[self.rank * count : (self.rank + 1) * count]
                slot.copy_(flat[owner * count : (owner + 1) * count])  # peer-to-peer copy
        self.runtime.barrier()  # all gradients have landed
        total = dkv_local.float()
        mine = buffer.typed(torch.bfloat16)
        for src in range(self.rank + 1, self.world):
            total += mine[src * count : (src + 1) * count].view_as(dkv_local).float()
        return total.to(dkv_local.dtype)


class LazyCPWorkspace:
    """Creates the group's :class:`CPWorkspace` at the first attention call, when the size of a
    key/value chunk is known (all ranks get there together)."""

    def __init__(self, group, wait_limit_s: float = 10.0) -> None:
        self.group, self.wait_limit_s = group, wait_limit_s
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.workspace: CPWorkspace | None = None

    def materialize(self, chunk_elements: int) -> CPWorkspace:
        if self.workspace is None:
            self.workspace = CPWorkspace(self.group, chunk_elements, self.wait_limit_s)
        return self.workspace


def _merge(out_a: Tensor, lse_a: Tensor, out_b: Tensor, lse_b: Tensor):
    """Combine two attention results over disjoint key sets: ``out (B,T,H,D)``, ``lse (B,H,T)``."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).transpose(1, 2).unsqueeze(-1)  # (B, T, H, 1)
    wb = torch.exp(lse_b - lse).transpose(1, 2).unsqueeze(-1)
    out = (out_a.float() * wa + out_b.float() * wb).to(out_a.dtype)
    return out, lse


class _ContextParallelAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, workspace: CPWorkspace, scale: float):
        C = ext()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        kv = torch.stack((k, v), dim=2).transpose(0, 1).contiguous()  # (T_local, B, 2, Hk, D)
        remote, arrived = workspace.exchange_kv(kv)
        out, lse = C.flash_attn_fwd(q, k, v, True, scale)  # overlaps the copies
        k_far = v_far = None
        if workspace.rank > 0:
            torch.cuda.current_stream(q.device).wait_event(arrived)
            saved = remote.clone()  # the landing buffer is recycled; backward needs these chunks
            k_far = saved[:, :, 0].transpose(0, 1)  # (B, rank * T_local, Hk, D), strided view
            v_far = saved[:, :, 1].transpose(0, 1)
            out_far, lse_far = C.flash_attn_fwd(q, k_far, v_far, False, scale)
            out, lse = _merge(out, lse, out_far, lse_far)
            out = out.contiguous()
            lse = lse.contiguous()
        ctx.save_for_backward(q, k, v, out, lse, k_far, v_far)
        ctx.workspace, ctx.scale = workspace, scale
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        C = ext()
        q, k, v, out, lse, k_far, v_far = ctx.saved_tensors
        ws = ctx.workspace
        dout = dout.contiguous()
        dq, dk, dv = C.flash_attn_bwd(dout, q, k, v, out, lse, True, ctx.scale)
        dkv_far = None
        if k_far is not None:
            dq_far, dk_far, dv_far = C.flash_attn_bwd(dout, q, k_far, v_far, out, lse, False, ctx.scale)
            dq = dq + dq_far
            dkv_far = torch.stack((dk_far, dv_far), dim=2).transpose(0, 1).contiguous()
        dkv_local = torch.stack((dk, dv), dim=2).transpose(0, 1).contiguous()
        dkv = ws.return_kv_grads(dkv_far, dkv_local)  # (T_local, B, 2, Hk, D)
        dk_total = dkv[:, :, 0].transpose(0, 1).contiguous()
        dv_total = dkv[:, :, 1].transpose(0, 1).contiguous()
        return dq, dk_total, dv_total, None, None


def context_parallel_attention(q: Tensor, k: Tensor, v: Tensor, workspace: CPWorkspace,
                               scale: float | None = None) -> Tensor:
    """Causal attention for this rank's chunk: ``q (B, T_local, H, D)``, ``k/v (B, T_local, Hk, D)``
    bf16, already rotated with their global positions. Returns ``(B, T_local, H, D)``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if isinstance(workspace, LazyCPWorkspace):
        workspace = workspace.materialize(2 * k.numel())
    return _ContextParallelAttention.apply(q, k, v, workspace, float(scale))
