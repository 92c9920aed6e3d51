"""Context parallelism: causal attention over a sequence sharded in a zig-zag over the ranks.

The sequence is cut into ``2 * world`` blocks of ``h`` tokens; rank ``r`` holds block ``r`` (its
*early* half) followed by block ``2 * world - 1 - r`` (its *late* half). With contiguous chunks
the last rank would attend to ``world`` times as many keys as the first; in the zig-zag every rank
does the same ``2 * world * h^2`` of attention work:

* local pass: the two halves in order are a causal sequence of their own (the early half
  precedes the late half), so one causal flash attention over the local ``2h`` tokens covers them;
* *near* pass: all local queries against the early halves of the ranks before this one;
* *far* pass: the late-half queries against both halves of the ranks after this one.

Both remote passes are non-causal (every key in them precedes every query that sees it) and are
merged into the local result through the log-sum-exp. The exchange is overlapped with attention:

1. every rank copies its ``(K, V)`` tokens into a symmetric staging buffer and publishes a flag;
2. a side stream pulls what this rank needs with the copy engines (stream-ordered wait on the
   owner's flag, peer-to-peer copy: half a buffer from earlier ranks, a whole one from later
   ranks) while
3. the main stream already runs the local pass;
4. once the remote tokens have landed, the near and far passes run and are merged.

The backward pass runs the flash-attention backward kernels with the merged statistics, then
returns the key/value gradients of remote tokens to their owners with peer-to-peer copies into
per-source slots that the owner sums. Staging and slot buffers are double-buffered and every reuse
is preceded by the bounded flag barrier of :class:`PeerRuntime`.

Staged layout is ``(T_local, B, 2, kv_heads, D)``: token-major, so the early half of a rank is the
first half of its buffer and pulled pieces concatenate into one key sequence for any batch size.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import Tensor

from ohara_b200.ops._ext import ext
from ohara_b200.parallel.peer import PeerRuntime, SymmetricBuffer, release_stream_waits
from ohara_b200.utils.profiling import nvtx_annotate

_KV_SLOT = 0


# -- buffer arithmetic of the exchange (pure functions, checked on CPU) ---------------------------------
def landing_layout(rank: int, world: int, count: int):
    """Where the pulled key/value tokens land in this rank's gather buffer. ``count`` = elements of
    one rank's staged tokens. Returns ``(near, far)``: lists of ``(source rank, offset, elements)``;
    a near piece is the first half of the source's buffer, a far piece the whole of it. Near pieces
    are contiguous from 0 in source order, far pieces follow them in source order."""
    half = count // 2
    near = [(src, src * half, half) for src in range(rank)]
    base = rank * half
    far = [(src, base + slot * count, count) for slot, src in enumerate(range(rank + 1, world))]
    return near, far


def gradient_span(owner: int, source: int, count: int) -> int:
    """Elements of key/value gradient that ``source`` returns to ``owner``: a later rank saw only
    the owner's early half, an earlier rank saw both halves."""
    return count // 2 if source > owner else count


# -- zig-zag sharding (host-side helpers, no device needed) -------------------------------------------
def zigzag_blocks(rank: int, world: int) -> tuple[int, int]:
    """Indices of the two sequence blocks (out of ``2 * world``) that ``rank`` holds."""
    return rank, 2 * world - 1 - rank


def shard_sequence(x: Tensor, rank: int, world: int, dim: int = 1) -> Tensor:
    """This rank's tokens of a full sequence along ``dim``: early block, then late block."""
    length = x.shape[dim]
    if length % (2 * world):
        raise ValueError(f"sequence of {length} does not split into {2 * world} zig-zag blocks")
    h = length // (2 * world)
    early, late = zigzag_blocks(rank, world)
    return torch.cat((x.narrow(dim, early * h, h), x.narrow(dim, late * h, h)), dim=dim)


def unshard_sequence(shards: list[Tensor], dim: int = 1) -> Tensor:
    """Inverse of :func:`shard_sequence` given the shards of all ranks in rank order."""
    world = len(shards)
    blocks: list[Tensor | None] = [None] * (2 * world)
    for rank, shard in enumerate(shards):
        h = shard.shape[dim] // 2
        early, late = zigzag_blocks(rank, world)
        blocks[early] = shard.narrow(dim, 0, h)
        blocks[late] = shard.narrow(dim, h, h)
    return torch.cat(blocks, dim=dim)


def local_positions(rank: int, world: int, local_length: int, device=None) -> Tensor:
    """Global positions (int64) of this rank's ``local_length`` tokens."""
    if local_length % 2:
        raise ValueError("a zig-zag shard holds an even number of tokens")
    h = local_length // 2
    early, late = zigzag_blocks(rank, world)
    steps = torch.arange(h, device=device)
    return torch.cat((early * h + steps, late * h + steps))


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
        self.poisoned = False
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def abort(self) -> None:
        """Satisfy every stream-ordered wait the copy stream may be parked in (the awaited "staged"
        flags live in this rank's own flag buffer) and mark the workspace unusable; the way out
        for the copy engines when a peer is lost or a collective timed out."""
        self.poisoned = True
        release_stream_waits([self.flags.pointers[self.rank] + 4 * (_KV_SLOT + r)
                              for r in range(self.world)], self.device)

    @nvtx_annotate("cp.exchange_kv")
    def exchange_kv(self, kv_local: Tensor):
        """Stage this rank's ``(T_local, B, 2, Hk, D)`` tokens and start pulling the early halves of
        the ranks before this one and everything of the ranks after it. Returns ``(near, far,
        arrived)``: views ``(rank * T_local / 2, B, 2, Hk, D)`` and ``((world - 1 - rank) * T_local,
        B, 2, Hk, D)`` (either may be ``None``; valid until two exchanges later) and the event that
        marks their arrival."""
        if self.poisoned:
            raise RuntimeError("this context-parallel workspace was aborted after a lost peer or a "
                               "timed-out collective; rebuild the engine to continue")
        if kv_local.numel() > self.chunk_elements:
            raise ValueError("key/value chunk exceeds the workspace")
        if kv_local.shape[0] % 2:
            raise ValueError("a zig-zag shard holds an even number of tokens")
        self.runtime.barrier()  # every rank has finished pulling from the buffer about to be reused
        self.kv_epoch += 1
        epoch, index = self.kv_epoch, self.kv_epoch % 2
        count = kv_local.numel()
        half = count // 2
        self.stage[index].typed(torch.bfloat16)[:count].copy_(kv_local.reshape(-1))
        ext().tp_signal(self.flags.pointers, _KV_SLOT, self.rank, epoch)
        main = torch.cuda.current_stream(self.device)
        staged = torch.cuda.Event()
        staged.record(main)
        self.copy_stream.wait_event(staged)
        landing = self.gathered[index]
        near_elements = self.rank * half
        near_pieces, far_pieces = landing_layout(self.rank, self.world, count)
        arrived = torch.cuda.Event()
        with torch.cuda.stream(self.copy_stream):
            for src, begin, elements in near_pieces[::-1] + far_pieces:  # nearest earlier owner first
                ext().stream_wait_value32(self.flags.pointers[self.rank] + 4 * (_KV_SLOT + src), epoch)
                remote = self.stage[index].typed(torch.bfloat16, rank=src)[:elements]
                landing[begin : begin + elements].copy_(remote)
            arrived.record(self.copy_stream)
        tokens, tail = kv_local.shape[0], kv_local.shape[1:]
        near = far = None
        if self.rank > 0:
            near = landing[:near_elements].view(self.rank * (tokens // 2), *tail)
        later = self.world - 1 - self.rank
        if later > 0:
            far = landing[near_elements : near_elements + later * count].view(later * tokens, *tail)
        return near, far, arrived

    @nvtx_annotate("cp.return_kv_grads")
    def return_kv_grads(self, dkv_near: Tensor | None, dkv_far: Tensor | None,
                        dkv_local: Tensor) -> Tensor:
        """Send the gradients of the near tokens (early halves of ranks ``0 .. rank-1``) and of the
        far tokens (ranks ``rank+1 ..``) to their owners and return ``dkv_local`` plus what the
        other ranks sent for this rank's tokens."""
        count = dkv_local.numel()
        half = count // 2
        self.runtime.barrier()  # owners have finished summing the previous slots
        self.grad_epoch += 1
        buffer = self.grad_slots[self.grad_epoch % 2]
        mine_at = self.rank * count  # this rank's slot in every owner's buffer
        if dkv_near is not None:
            flat = dkv_near.reshape(-1)
            for owner in range(self.rank):
                slot = buffer.typed(torch.bfloat16, rank=owner)[mine_at : mine_at + half]
                slot.copy_(flat[owner * half : (owner + 1) * half])  # peer-to-peer copy
        if dkv_far is not None:
            flat = dkv_far.reshape(-1)
            for index, owner in enumerate(range(self.rank + 1, self.world)):
                slot = buffer.typed(torch.bfloat16, rank=owner)[mine_at : mine_at + count]
                slot.copy_(flat[index * count : (index + 1) * count])
        self.runtime.barrier()  # all gradients have landed
        total = dkv_local.float().contiguous()
        flat_total = total.view(-1)
        mine = buffer.typed(torch.bfloat16)
        for src in range(self.world):
            if src == self.rank:
                continue
            span = gradient_span(self.rank, src, count)
            flat_total[:span] += mine[src * count : src * count + span].float()
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


def _split_kv(staged: Tensor) -> tuple[Tensor, Tensor]:
    """``(T, B, 2, Hk, D)`` staged tokens -> strided ``(B, T, Hk, D)`` views of keys and values."""
    return staged[:, :, 0].transpose(0, 1), staged[:, :, 1].transpose(0, 1)


def _stack_kv(dk: Tensor, dv: Tensor) -> Tensor:
    return torch.stack((dk, dv), dim=2).transpose(0, 1).contiguous()  # (T, B, 2, Hk, D)


class _ContextParallelAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, workspace: CPWorkspace, scale: float):
        C = ext()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        h = q.shape[1] // 2
        near, far, arrived = workspace.exchange_kv(_stack_kv(k, v))
        out, lse = C.flash_attn_fwd(q, k, v, True, scale)  # overlaps the copies
        k_near = v_near = k_far = v_far = None
        if near is not None or far is not None:
            torch.cuda.current_stream(q.device).wait_event(arrived)
        if near is not None:
            # the landing buffer is recycled; backward needs these tokens
            k_near, v_near = _split_kv(near.clone())
            out_near, lse_near = C.flash_attn_fwd(q, k_near, v_near, False, scale)
            out, lse = _merge(out, lse, out_near, lse_near)
        if far is not None:
            k_far, v_far = _split_kv(far.clone())
            out_far, lse_far = C.flash_attn_fwd(q[:, h:], k_far, v_far, False, scale)
            out_late, lse_late = _merge(out[:, h:], lse[:, :, h:], out_far, lse_far)
            out = torch.cat((out[:, :h], out_late), dim=1)
            lse = torch.cat((lse[:, :, :h], lse_late), dim=2)
        out, lse = out.contiguous(), lse.contiguous()
        ctx.save_for_backward(q, k, v, out, lse, k_near, v_near, k_far, v_far)
        ctx.workspace, ctx.scale = workspace, scale
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        C = ext()
        q, k, v, out, lse, k_near, v_near, k_far, v_far = ctx.saved_tensors
        ws = ctx.workspace
        h = q.shape[1] // 2
        dout = dout.contiguous()
        dq, dk, dv = C.flash_attn_bwd(dout, q, k, v, out, lse, True, ctx.scale)
        dkv_near = dkv_far = None
        if k_near is not None:
            dq_near, dk_near, dv_near = C.flash_attn_bwd(dout, q, k_near, v_near, out, lse, False,
                                                         ctx.scale)
            dq = dq + dq_near
            dkv_near = _stack_kv(dk_near, dv_near)
        if k_far is not None:
            dq_far, dk_far, dv_far = C.flash_attn_bwd(
                dout[:, h:], q[:, h:], k_far, v_far, out[:, h:].contiguous(),
                lse[:, :, h:].contiguous(), False, ctx.scale)
            dq = torch.cat((dq[:, :h], dq[:, h:] + dq_far), dim=1)
            dkv_far = _stack_kv(dk_far, dv_far)
        dkv = ws.return_kv_grads(dkv_near, dkv_far, _stack_kv(dk, dv))  # (T_local, B, 2, Hk, D)
        dk_total = dkv[:, :, 0].transpose(0, 1).contiguous()
        dv_total = dkv[:, :, 1].transpose(0, 1).contiguous()
        return dq, dk_total, dv_total, None, None


def context_parallel_attention(q: Tensor, k: Tensor, v: Tensor, workspace: CPWorkspace,
                               scale: float | None = None) -> Tensor:
    """Causal attention for this rank's zig-zag shard (:func:`shard_sequence`): ``q (B, T_local, H,
    D)``, ``k/v (B, T_local, Hk, D)`` bf16, already rotated with their global positions
    (:func:`local_positions`). Returns ``(B, T_local, H, D)``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if isinstance(workspace, LazyCPWorkspace):
        workspace = workspace.materialize(2 * k.numel())
    return _ContextParallelAttention.apply(q, k, v, workspace, float(scale))
