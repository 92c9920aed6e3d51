"""Sharded data parallelism: master weights and optimizer state are partitioned over the
data-parallel group, gradients are reduce-scattered and updated weights all-gathered.

What ``StrategyType.FSDP`` means in this package. The reference has no sharded strategy at all
(``dp_shard`` is folded into plain DDP: ohara/runtime/topology.py:33-38, engine.py:165-179); this is
new code.

Layout. All trainable parameters map into one flat index space made of ``world`` equal *regions*;
region ``r`` belongs to rank ``r`` and is ``[matrix part | elementwise part]``:

* parameters of whole-matrix algorithms (Muon, MuonH, AdamH) are assigned as whole matrices,
  round-robin, so the owner can orthogonalise them without any gather (expert stacks
  ``(E, in, out)`` are split along ``E`` when it divides);
* parameters of elementwise algorithms (AdamW) are concatenated and cut into ``world`` equal
  ranges, wherever the cut falls.

Gradients and compute-precision weights each live in one flat buffer with this layout, so a step
is ONE reduce-scatter (gradients) and ONE all-gather (weights), whatever the number of tensors:

    pack grads -> reduce-scatter -> [owner: update fp32 master shard] -> all-gather weights -> unpack

On CUDA the wire format is bf16 for both and each parameter's bf16 compute copy is a *view* of the
gathered buffer, so the forward pass needs no further cast. The collectives run on the c10d
backend, or — with ``fused=True`` on NVLink-connected GPUs — as peer-memory kernels from
``ohara_b200.parallel.peer`` that fold the cast / scale / AdamW update into the reduce-scatter.

Only the owner holds full-precision (fp32) values of a parameter between steps; other ranks hold
the gathered (bf16-rounded on CUDA) values. ``sync_master_weights`` all-gathers the fp32 masters
into the module, which is what checkpointing calls.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor
from torch.optim import Optimizer
from ohara_b200.utils.profiling import nvtx_annotate

ALIGN = 128  # elements; keeps every region 256-byte aligned in bf16


@dataclass
class _Piece:
    """A contiguous run of elements of one parameter inside one rank's region."""

    param: torch.nn.Parameter
    begin: int  # first flat element of the parameter covered by this piece
    length: int
    rank: int
    offset: int  # element offset inside the owner's region
    group: int  # index of the user-visible param group
    shape: tuple[int, ...] | None  # logical shape when the piece is a whole matrix / expert slab


def _is_matrix_group(group: dict[str, Any]) -> bool:
    return group.get("kind") == "muon" or bool(group.get("hypersphere", False))


def _round_up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


class ShardedOptimizer(Optimizer):
    """Wraps an optimizer built over full parameters and runs it on this rank's shard only.

    ``param_groups`` stays the wrapped optimizer's list (schedules and metadata keep working);
    hyper-parameters are copied to the internal shard optimizer before every step.
    """

    def __init__(self, optimizer: Optimizer, process_group=None, fused: bool = False,
                 wire_dtype: torch.dtype | None = None, *, replicate_group=None,
                 replicate_world: int = 1, solo: bool = False,
                 norm_groups: dict[str, Any] | None = None) -> None:
        """``process_group``: the ranks the state is sharded over. ``replicate_group`` (with its
        size ``replicate_world``): ranks that hold a copy of the *same* shard (hybrid sharding,
        ``dp_replicate x dp_shard``); their reduced shards are averaged after the reduce-scatter.
        ``solo=True`` shards over nobody (this rank alone owns the parameters, e.g. the experts
        of an expert-parallel rank without data-parallel replicas). ``norm_groups`` maps
        ``"tp"`` / ``"ep"`` to the process group over which the shards of tensor-parallel /
        expert-parallel parameters are distinct and ``"pp"`` to the pipeline group (whose stages
        hold different parameters altogether), for the global gradient norm."""
        self.inner = optimizer
        self.group = process_group
        distributed = dist.is_initialized() and not solo
        self.world = dist.get_world_size(process_group) if distributed else 1
        self.rank = dist.get_rank(process_group) if distributed else 0
        self.replicate_group = replicate_group
        self.replicate_world = int(replicate_world) if dist.is_initialized() else 1
        self.norm_groups = dict(norm_groups or {})
        self.param_groups = optimizer.param_groups
        self.defaults = optimizer.defaults
        self.state = optimizer.state  # kept for API parity; the live state is in self.local
        params = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        if not params:
            raise ValueError("optimizer has no trainable parameters")
        self.device = params[0].device
        on_gpu = self.device.type == "cuda"
        self.wire_dtype = wire_dtype or (torch.bfloat16 if on_gpu else torch.float32)
        self._plan()
        self._allocate()
        self._build_local_optimizer()
        self._reduced = False
        self.fused = False
        self._peer = None
        if fused and on_gpu and self.world > 1:
            self._try_enable_fused()

    # -- planning ----------------------------------------------------------------------------
    def _plan(self) -> None:
        self.pieces, self.matrix_size, self.elementwise_size = self._compute_plan(self.world)
        self.region = self.matrix_size + self.elementwise_size
        self.all_pieces = [piece for per_rank in self.pieces for piece in per_rank]

    def _compute_plan(self, world: int) -> tuple[list[list[_Piece]], int, int]:
        """Layout for ``world`` ranks: ``(pieces per rank, matrix part size, elementwise part
        size)``. A pure function of the parameter groups, so the layout a checkpoint was written
        with can be rebuilt at any other world size."""
        matrix_pieces: list[list[_Piece]] = [[] for _ in range(world)]
        matrix_fill = [0] * world
        counter = 0
        elementwise: list[tuple[torch.nn.Parameter, int]] = []
        for gi, group in enumerate(self.param_groups):
            params = [p for p in group["params"] if p.requires_grad]
            if not _is_matrix_group(group):
                elementwise += [(p, gi) for p in params]
                continue
            for p in params:
                if p.ndim == 3 and p.shape[0] % world == 0 and world > 1:
                    per = p.shape[0] // world
                    slab = per * p.shape[1] * p.shape[2]
                    for r in range(world):
                        matrix_pieces[r].append(_Piece(p, r * slab, slab, r, matrix_fill[r], gi,
                                                       (per, p.shape[1], p.shape[2])))
                        matrix_fill[r] += _round_up(slab, 8)
                else:
                    r = counter % world
                    counter += 1
                    matrix_pieces[r].append(_Piece(p, 0, p.numel(), r, matrix_fill[r], gi,
                                                   tuple(p.shape)))
                    matrix_fill[r] += _round_up(p.numel(), 8)
        matrix_size = _round_up(max(matrix_fill) if matrix_fill else 0, ALIGN)
        total = sum(p.numel() for p, _ in elementwise)
        elementwise_size = _round_up((total + world - 1) // world, ALIGN) if total else 0
        ew_pieces: list[list[_Piece]] = [[] for _ in range(world)]
        cursor = 0
        for p, gi in elementwise:
            done = 0
            while done < p.numel():
                r = cursor // elementwise_size
                room = (r + 1) * elementwise_size - cursor
                take = min(room, p.numel() - done)
                ew_pieces[r].append(_Piece(p, done, take, r,
                                           matrix_size + cursor - r * elementwise_size,
                                           gi, None))
                done += take
                cursor += take
        pieces = [matrix_pieces[r] + ew_pieces[r] for r in range(world)]
        return pieces, matrix_size, elementwise_size

    def _local_layout(self, pieces_of_rank: list[_Piece]) -> list[tuple[int, list[list[_Piece]]]]:
        """Parameters of a rank's shard optimizer, in order: ``[(user group index, [pieces of
        local parameter 0, pieces of local parameter 1, ...])]``. Adjacent elementwise pieces of
        one group form a single 1-D local parameter."""
        layout: list[tuple[int, list[list[_Piece]]]] = []
        for gi, group in enumerate(self.param_groups):
            mine = [piece for piece in pieces_of_rank if piece.group == gi]
            if not mine:
                continue
            contiguous = all(a.offset + a.length == b.offset for a, b in zip(mine, mine[1:]))
            if not _is_matrix_group(group) and len(mine) > 1 and contiguous:
                layout.append((gi, [mine]))
            else:
                layout.append((gi, [[piece] for piece in mine]))
        return layout

    def _allocate(self) -> None:
        n = self.region * self.world
        dev = self.device
        self.grad_flat = torch.zeros(n, device=dev, dtype=self.wire_dtype)
        self.weight_flat = torch.zeros(n, device=dev, dtype=self.wire_dtype)
        self.master = torch.zeros(self.region, device=dev, dtype=torch.float32)
        self.grad_local = torch.zeros(self.region, device=dev, dtype=torch.float32)
        with torch.no_grad():
            for piece in self.pieces[self.rank]:
                src = piece.param.detach().reshape(-1)[piece.begin : piece.begin + piece.length]
                self.master[piece.offset : piece.offset + piece.length].copy_(src)
            for piece in self.all_pieces:
                base = piece.rank * self.region + piece.offset
                src = piece.param.detach().reshape(-1)[piece.begin : piece.begin + piece.length]
                self.weight_flat[base : base + piece.length].copy_(src)
        self._bind_shadows()

    def _bind_shadows(self) -> None:
        """Point each parameter's bf16 compute copy at the gathered weight buffer (CUDA only;
        parameters split across regions keep a private copy)."""
        if self.wire_dtype != torch.bfloat16:
            return
        from ohara_b200.ops import refresh_bf16_weight

        whole: dict[int, _Piece] = {}
        counts: dict[int, int] = {}
        for piece in self.all_pieces:
            counts[id(piece.param)] = counts.get(id(piece.param), 0) + 1
            whole[id(piece.param)] = piece
        for key, piece in whole.items():
            p = piece.param
            if counts[key] != 1 or piece.length != p.numel() or p.dtype != torch.float32:
                continue
            base = piece.rank * self.region + piece.offset
            if (base * 2) % 16:
                continue
            refresh_bf16_weight(p, self.weight_flat[base : base + p.numel()].view(p.shape))

    def _build_local_optimizer(self) -> None:
        """Shard-sized parameters (views of the fp32 master) grouped like the user's groups."""
        local_groups: list[dict[str, Any]] = []
        self._local_of_group: list[int | None] = [None] * len(self.param_groups)
        for gi, entries in self._local_layout(self.pieces[self.rank]):
            shard_params = []
            for entry in entries:
                first, last = entry[0], entry[-1]
                view = self.master[first.offset : last.offset + last.length]
                if len(entry) == 1 and first.shape is not None:
                    view = view.view(first.shape)
                param = torch.nn.Parameter(view, requires_grad=True)
                if len(entry) == 1 and hasattr(first.param, "tensor_parallel_dim"):
                    # whole-matrix algorithms need to know that this is a tensor-parallel shard
                    param.tensor_parallel_dim = first.param.tensor_parallel_dim
                if len(entry) == 1:
                    param._shard_piece = first
                else:
                    # Elementwise pieces of one group are adjacent in the region: they are
                    # updated as one 1-D tensor (identical maths, one kernel).
                    param._shard_span = (first.offset, last.offset + last.length)
                shard_params.append(param)
            clone = {k: v for k, v in self.param_groups[gi].items() if k != "params"}
            clone["params"] = shard_params
            self._local_of_group[gi] = len(local_groups)
            local_groups.append(clone)
        self.local: Optimizer | None = None
        if local_groups:
            cls = getattr(self.inner, "optimizer_class", None) or type(self.inner)
            try:
                self.local = cls(local_groups)
            except TypeError:
                self.local = cls(local_groups, **{k: v for k, v in self.inner.defaults.items()})
            for name in ("tensor_parallel_group", "tensor_parallel_world"):
                if hasattr(self.inner, name):
                    setattr(self.local, name, getattr(self.inner, name))

    # -- fused peer-memory path ----------------------------------------------------------------
    def _try_enable_fused(self) -> None:
        try:
            from ohara_b200.parallel.peer import PeerBuffers

            self._peer = PeerBuffers.create(self, self.group)
            self.fused = self._peer is not None
        except Exception as error:  # noqa: BLE001 - fall back to c10d, but say so
            if self.rank == 0:
                print(f"[ohara_b200] peer-memory collectives unavailable ({error}); using c10d")
            self._peer = None
            self.fused = False

    # -- step ----------------------------------------------------------------------------------
    def _span(self, param) -> tuple[int, int]:
        span = getattr(param, "_shard_span", None)
        if span is not None:
            return span
        piece = param._shard_piece
        return piece.offset, piece.offset + piece.length

    @torch.no_grad()
    def _pack_gradients(self) -> None:
        dst, src = [], []
        for piece in self.all_pieces:
            grad = piece.param.grad
            base = piece.rank * self.region + piece.offset
            target = self.grad_flat[base : base + piece.length]
            if grad is None:
                target.zero_()
                continue
            dst.append(target)
            src.append(grad.reshape(-1)[piece.begin : piece.begin + piece.length])
        if dst:
            torch._foreach_copy_(dst, src)

    @torch.no_grad()
    @nvtx_annotate("zero.reduce_scatter_gradients")
    def reduce_gradients(self) -> None:
        """Pack local gradients, reduce-scatter them and leave the mean in ``grad_local``."""
        if self._reduced:
            return
        self._pack_gradients()
        if self.world == 1:
            self.grad_local.copy_(self.grad_flat[: self.region])
        elif self.fused and self._peer is not None:
            self._peer.reduce_scatter_mean(self.grad_flat, self.grad_local)
        else:
            if dist.get_backend(self.group) == "gloo":  # gloo has no reduce-scatter
                dist.all_reduce(self.grad_flat, group=self.group)
                shard = self.grad_flat[self.rank * self.region : (self.rank + 1) * self.region]
            else:
                shard = torch.empty(self.region, device=self.device, dtype=self.wire_dtype)
                dist.reduce_scatter_tensor(shard, self.grad_flat, op=dist.ReduceOp.SUM,
                                           group=self.group)
            self.grad_local.copy_(shard)
            self.grad_local.div_(self.world)
        if self.replicate_world > 1:
            # hybrid sharding: the same shard exists once per replica group; average them
            dist.all_reduce(self.grad_local, group=self.replicate_group)
            self.grad_local.div_(self.replicate_world)
        self._reduced = True

    def _norm_classes(self) -> dict[str, list[tuple[int, int]]]:
        """Spans of this rank's region by how the parameter is laid out over the *other* parallel
        dimensions: ``"whole"`` (replicated there), ``"tp"`` / ``"ep"`` (every rank of that
        dimension holds a distinct shard, so squared norms add up over it)."""
        cached = getattr(self, "_norm_spans", None)
        if cached is None:
            cached = {"whole": [], "tp": [], "ep": []}
            for piece in self.pieces[self.rank]:
                kind = ("tp" if hasattr(piece.param, "tensor_parallel_dim")
                        else "ep" if getattr(piece.param, "expert_parallel", False) else "whole")
                if kind not in self.norm_groups and kind != "whole":
                    kind = "whole"
                spans = cached[kind]
                if spans and spans[-1][1] == piece.offset:
                    spans[-1] = (spans[-1][0], piece.offset + piece.length)
                else:
                    spans.append((piece.offset, piece.offset + piece.length))
            self._norm_spans = cached
        return cached

    @torch.no_grad()
    def grad_sq_norm(self) -> Tensor:
        """Squared l2 norm of the whole (unsharded, all tensor / expert shards included) mean
        gradient of the parameters this optimizer manages; collective, same value on every rank
        that takes part. Reduces the gradients first if that has not happened yet."""
        self.reduce_gradients()
        parts = []
        for kind in ("whole", "tp", "ep"):
            views = [self.grad_local[lo:hi] for lo, hi in self._norm_classes()[kind]]
            if views:
                norms = torch.stack(torch._foreach_norm(views)).float()
                parts.append(norms.square().sum())
            else:
                parts.append(torch.zeros((), device=self.device, dtype=torch.float32))
        sums = torch.stack(parts)
        if self.world > 1:
            dist.all_reduce(sums, group=self.group)
        total = sums[0]
        for index, kind in ((1, "tp"), (2, "ep")):
            if kind in self.norm_groups:
                part = sums[index].clone()
                dist.all_reduce(part, group=self.norm_groups[kind])
                total = total + part
        if "pp" in self.norm_groups:  # every pipeline stage holds different parameters
            total = total.clone()
            dist.all_reduce(total, group=self.norm_groups["pp"])
        return total

    @torch.no_grad()
    def scale_gradients_(self, scale: Tensor) -> None:
        self.grad_local.mul_(scale)

    @torch.no_grad()
    def clip_grad_norm_(self, model, max_norm: float) -> Tensor:
        """Global gradient-norm clipping on the reduced shards (collective)."""
        norm = self.grad_sq_norm().sqrt()
        scale = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        self.scale_gradients_(scale)
        return norm

    def _sync_hyperparameters(self) -> None:
        if self.local is None:
            return
        for gi, group in enumerate(self.param_groups):
            li = self._local_of_group[gi]
            if li is None:
                continue
            target = self.local.param_groups[li]
            for key, value in group.items():
                if key != "params":
                    target[key] = value

    @torch.no_grad()
    @nvtx_annotate("zero.step")
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.reduce_gradients()
        self._sync_hyperparameters()
        if self.local is not None:
            for group in self.local.param_groups:
                for param in group["params"]:
                    lo, hi = self._span(param)
                    param.grad = self.grad_local[lo:hi].view(param.shape)
            self.local.step()
            for group in self.local.param_groups:
                for param in group["params"]:
                    param.grad = None
        self._publish_weights()
        self._reduced = False
        return loss

    @torch.no_grad()
    def _publish_weights(self) -> None:
        """Write this rank's updated shard in wire precision, all-gather, refresh the module."""
        mine = self.weight_flat[self.rank * self.region : (self.rank + 1) * self.region]
        if self.wire_dtype == torch.bfloat16 and self.device.type == "cuda":
            from ohara_b200.ops._ext import ext

            ext().cast_bf16_into(self.master, mine)
        else:
            mine.copy_(self.master)
        if self.world > 1:
            if self.fused and self._peer is not None:
                self._peer.all_gather(self.weight_flat)
            else:
                self._all_gather_flat(self.weight_flat, mine.clone())
        dst, src = [], []
        for piece in self.all_pieces:
            base = piece.rank * self.region + piece.offset
            dst.append(piece.param.data.reshape(-1)[piece.begin : piece.begin + piece.length])
            src.append(self.weight_flat[base : base + piece.length])
        torch._foreach_copy_(dst, src)
        self._bind_shadows()

    @nvtx_annotate("zero.all_gather_weights")
    def _all_gather_flat(self, out: Tensor, mine: Tensor) -> None:
        if dist.get_backend(self.group) == "gloo":
            parts = [out[r * self.region : (r + 1) * self.region] for r in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
        else:
            dist.all_gather_into_tensor(out, mine, group=self.group)

    @torch.no_grad()
    def sync_master_weights(self) -> None:
        """All-gather the fp32 master shards into the module's parameters (collective)."""
        if self.world > 1:
            full = torch.empty(self.region * self.world, device=self.device, dtype=torch.float32)
            self._all_gather_flat(full, self.master)
        else:
            full = self.master
        for piece in self.all_pieces:
            base = piece.rank * self.region + piece.offset
            piece.param.data.reshape(-1)[piece.begin : piece.begin + piece.length].copy_(
                full[base : base + piece.length]
            )
        self._bind_shadows()

    def zero_grad(self, set_to_none: bool = True) -> None:
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.detach_()
                    p.grad.zero_()

    # -- checkpoints ---------------------------------------------------------------------------
    def _gather_shards(self) -> list[dict[str, Any]]:
        local = self.local.state_dict() if self.local is not None else None
        payload = {"master": self.master.detach().cpu(), "optimizer": _to_cpu(local)}
        if self.world > 1:
            gathered: list[Any] = [None] * self.world
            dist.all_gather_object(gathered, payload, group=self.group)
            return gathered
        return [payload]

    def _group_metadata(self) -> list[dict[str, Any]]:
        return [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]

    def state_dict(self) -> dict[str, Any]:
        """Shard states of every rank, gathered (collective). ``load_state_dict`` accepts it at
        any world size: the layout of the writing job is rebuilt from ``world_size``."""
        return {
            "sharded": True,
            "world_size": self.world,
            "region": self.region,
            "param_groups": self._group_metadata(),
            "shards": self._gather_shards(),
        }

    def full_state_dict(self) -> dict[str, Any]:
        """Unsharded optimizer state in the format of the wrapped optimizer's own ``state_dict()``
        (collective): per-parameter Adam moments, one stacked momentum / second-moment buffer per
        Muon group keyed on the group's first parameter (ohara/optimizer.py:283-371). A
        single-process optimizer of the same class can load it."""
        full, _ = self._assemble_full(self._gather_shards(), self.world)
        return full

    def _param_indices(self) -> dict[int, int]:
        index: dict[int, int] = {}
        for group in self.param_groups:
            for p in group["params"]:
                index.setdefault(id(p), len(index))
        return index

    def _assemble_full(self, shards: list[dict[str, Any]], world: int):
        """``(full optimizer state dict, {param index: flat fp32 master values})`` from the shard
        states of a job of ``world`` ranks."""
        pieces, _, _ = self._compute_plan(world)
        index_of = self._param_indices()
        state: dict[int, dict[str, Any]] = {}
        masters: dict[int, Tensor] = {}
        for rank in range(world):
            master = shards[rank]["master"]
            for piece in pieces[rank]:
                flat = masters.setdefault(index_of[id(piece.param)],
                                          torch.zeros(piece.param.numel(), dtype=torch.float32))
                flat[piece.begin : piece.begin + piece.length] = master[
                    piece.offset : piece.offset + piece.length]
            local = shards[rank]["optimizer"]
            if local is None:
                continue
            for li, (gi, entries) in enumerate(self._local_layout(pieces[rank])):
                group = self.param_groups[gi]
                packed = local["param_groups"][li]["params"]
                if group.get("kind") == "muon":
                    saved = local["state"].get(packed[0])
                    if not saved:
                        continue
                    dest = state.setdefault(index_of[id(group["params"][0])], {})
                    for key, value in saved.items():
                        for i, entry in enumerate(entries):
                            piece, p = entry[0], entry[0].param
                            if p.ndim == 3:  # an expert stack, split along its first dimension
                                batch, per = p.shape[0], piece.shape[0]
                                first = piece.begin // (p.shape[1] * p.shape[2])
                                rows, source = slice(first, first + per), value
                            else:
                                batch = len(group["params"])
                                j = next(n for n, q in enumerate(group["params"]) if q is p)
                                rows, source = slice(j, j + 1), value[i : i + 1]
                            if key not in dest:
                                dest[key] = torch.zeros((batch, *value.shape[1:]), dtype=value.dtype)
                            dest[key][rows] = source
                    continue
                for entry, pid in zip(entries, packed):
                    saved = local["state"].get(pid)
                    if not saved:
                        continue
                    span = sum(piece.length for piece in entry)
                    for piece in entry:
                        p = piece.param
                        dest = state.setdefault(index_of[id(p)], {})
                        for key, value in saved.items():
                            if isinstance(value, Tensor) and value.ndim >= 1 and value.numel() == span:
                                if key not in dest:
                                    dest[key] = torch.zeros(p.numel(), dtype=value.dtype)
                                lo = piece.offset - entry[0].offset
                                dest[key][piece.begin : piece.begin + piece.length] = value.reshape(
                                    -1)[lo : lo + piece.length]
                            else:
                                dest[key] = value.clone() if isinstance(value, Tensor) else value
        shape_of = {index_of[id(p)]: p.shape for g in self.param_groups for p in g["params"]}
        for idx, entry in state.items():
            for key, value in entry.items():
                if isinstance(value, Tensor) and value.ndim == 1 and value.numel() == math.prod(
                        shape_of[idx]) and "momentum_buffer" not in key:
                    entry[key] = value.view(shape_of[idx])
        groups = []
        for meta, group in zip(self._group_metadata(), self.param_groups):
            groups.append({**meta, "params": [index_of[id(p)] for p in group["params"]]})
        return {"state": state, "param_groups": groups}, masters

    def _slice_full(self, full: dict[str, Any]) -> dict[str, Any] | None:
        """This rank's shard-optimizer state dict cut out of an unsharded state dict."""
        if self.local is None:
            return None
        index_of = self._param_indices()
        template = self.local.state_dict()
        state: dict[int, dict[str, Any]] = {}
        saved_state = {int(k): v for k, v in full["state"].items()}
        for li, (gi, entries) in enumerate(self._local_layout(self.pieces[self.rank])):
            group = self.param_groups[gi]
            packed = template["param_groups"][li]["params"]
            if group.get("kind") == "muon":
                saved = saved_state.get(index_of[id(group["params"][0])])
                if not saved:
                    continue
                local: dict[str, Any] = {}
                for key, value in saved.items():
                    parts = []
                    for entry in entries:
                        piece, p = entry[0], entry[0].param
                        if p.ndim == 3:
                            first = piece.begin // (p.shape[1] * p.shape[2])
                            parts.append(value[first : first + piece.shape[0]])
                        else:
                            j = next(n for n, q in enumerate(group["params"]) if q is p)
                            parts.append(value[j : j + 1])
                    local[key] = torch.cat(parts).clone()
                state[packed[0]] = local
                continue
            for entry, pid in zip(entries, packed):
                local = {}
                for piece in entry:
                    saved = saved_state.get(index_of[id(piece.param)])
                    if not saved:
                        continue
                    for key, value in saved.items():
                        if isinstance(value, Tensor) and value.numel() == piece.param.numel() \
                                and value.ndim >= 1:
                            cut = value.reshape(-1)[piece.begin : piece.begin + piece.length]
                            local.setdefault(key, []).append(cut)
                        else:
                            local[key] = value
                if not local:
                    continue
                for key, value in list(local.items()):
                    if isinstance(value, list):
                        joined = torch.cat(value).clone()
                        if len(entry) == 1 and entry[0].shape is not None:
                            joined = joined.view(entry[0].shape)
                        local[key] = joined
                state[pid] = local
        groups = []
        for li, template_group in enumerate(template["param_groups"]):
            gi = self._local_of_group.index(li)
            saved_group = {k: v for k, v in full["param_groups"][gi].items() if k != "params"}
            groups.append({**template_group, **saved_group, "params": template_group["params"]})
        return {"state": state, "param_groups": groups}

    @torch.no_grad()
    def _load_masters(self, masters: dict[int, Tensor] | None) -> None:
        """Refill the fp32 master shard (from ``masters`` when given, else from the module's
        current parameters) and republish the compute-precision weights (collective)."""
        index_of = self._param_indices()
        for piece in self.pieces[self.rank]:
            if masters is not None:
                source = masters[index_of[id(piece.param)]].to(self.device)
            else:
                source = piece.param.detach().reshape(-1).float()
            self.master[piece.offset : piece.offset + piece.length].copy_(
                source[piece.begin : piece.begin + piece.length])
        self._publish_weights()

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Accepts (a) ``state_dict()`` of a sharded job of any world size, (b) an unsharded state
        dict (``full_state_dict()`` or the wrapped optimizer class run on one process); in case
        (b) the master weights are taken from the module, which must be loaded first."""
        if state_dict.get("sharded"):
            same = state_dict["world_size"] == self.world and state_dict["region"] == self.region
            if same:
                shard = state_dict["shards"][self.rank]
                self.master.copy_(shard["master"].to(self.device))
                if self.local is not None and shard["optimizer"] is not None:
                    self.local.load_state_dict(shard["optimizer"])
                for saved, group in zip(state_dict["param_groups"], self.param_groups):
                    group.update(saved)
                self._publish_weights()
                return
            full, masters = self._assemble_full(state_dict["shards"], state_dict["world_size"])
        else:
            full, masters = state_dict, None
        local = self._slice_full(full)
        if self.local is not None and local is not None:
            self.local.load_state_dict(local)
        for saved, group in zip(full["param_groups"], self.param_groups):
            group.update({k: v for k, v in saved.items() if k != "params"})
        self._load_masters(masters)


class _GroupView:
    """What :class:`ShardedOptimizer` needs from "the wrapped optimizer" when it manages only some
    of that optimizer's parameters: the parameter groups (with the subset), the defaults and the
    class to instantiate for the shard."""

    def __init__(self, base: Optimizer, groups: list[dict[str, Any]]) -> None:
        self.param_groups = groups
        self.defaults = base.defaults
        self.state: dict = {}
        self.optimizer_class = getattr(base, "optimizer_class", None) or type(base)


class HybridShardedOptimizer(Optimizer):
    """Several :class:`ShardedOptimizer` parts, each over its own subset of the parameters and its
    own process group, behind one optimizer.

    This is what expert parallelism needs next to sharded data parallelism: the dense parameters
    (attention, shared experts, router, embeddings) are replicated over *all* ranks that see
    different data, expert-parallel peers included, and are sharded over that whole group; the
    routed experts of a rank are replicated only over the ranks that hold the same experts (its
    ``dp`` peers) — possibly over nobody — and are sharded over those alone.

    ``parts`` is a list of dictionaries: ``select`` (a predicate on parameters) plus the keyword
    arguments of :class:`ShardedOptimizer`. ``param_groups`` stays the wrapped optimizer's list, so
    schedules keep working; hyper-parameters are copied to the parts before every step. All ranks
    must build the parts in the same order (the parts run their collectives one after another).
    """

    def __init__(self, optimizer: Optimizer, parts: list[dict[str, Any]]) -> None:
        self.inner = optimizer
        self.param_groups = optimizer.param_groups
        self.defaults = optimizer.defaults
        self.state = optimizer.state
        self.parts: list[ShardedOptimizer] = []
        self._links: list[list[int]] = []  # per part: user group index of each of its groups
        claimed: set[int] = set()
        for spec in parts:
            spec = dict(spec)
            select = spec.pop("select")
            groups, links = [], []
            for gi, group in enumerate(self.param_groups):
                chosen = [p for p in group["params"] if p.requires_grad and select(p)]
                if not chosen:
                    continue
                overlap = claimed.intersection(id(p) for p in chosen)
                if overlap:
                    raise ValueError("a parameter was selected by two parts of a hybrid optimizer")
                claimed.update(id(p) for p in chosen)
                groups.append({**{k: v for k, v in group.items() if k != "params"},
                               "params": chosen})
                links.append(gi)
            if not groups:
                continue
            self.parts.append(ShardedOptimizer(_GroupView(optimizer, groups), **spec))
            self._links.append(links)
        missing = [p for g in self.param_groups for p in g["params"]
                   if p.requires_grad and id(p) not in claimed]
        if missing:
            raise ValueError(f"{len(missing)} trainable parameters belong to no part")
        if not self.parts:
            raise ValueError("optimizer has no trainable parameters")

    @property
    def fused(self) -> bool:
        return any(part.fused for part in self.parts)

    def _sync_hyperparameters(self) -> None:
        for part, links in zip(self.parts, self._links):
            for sub, gi in zip(part.param_groups, links):
                for key, value in self.param_groups[gi].items():
                    if key != "params":
                        sub[key] = value

    def reduce_gradients(self) -> None:
        for part in self.parts:
            part.reduce_gradients()

    @torch.no_grad()
    def clip_grad_norm_(self, model, max_norm: float) -> Tensor:
        total = sum(part.grad_sq_norm() for part in self.parts)
        norm = total.sqrt()
        scale = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        for part in self.parts:
            part.scale_gradients_(scale)
        return norm

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._sync_hyperparameters()
        for part in self.parts:
            part.step()
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        for part in self.parts:
            part.zero_grad(set_to_none)

    def sync_master_weights(self) -> None:
        for part in self.parts:
            part.sync_master_weights()

    def state_dict(self) -> dict[str, Any]:
        return {"hybrid": True, "parts": [part.state_dict() for part in self.parts]}

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if not state_dict.get("hybrid") or len(state_dict["parts"]) != len(self.parts):
            raise ValueError("expected the state of a hybrid sharded optimizer with "
                             f"{len(self.parts)} parts")
        for part, saved in zip(self.parts, state_dict["parts"]):
            part.load_state_dict(saved)
        for part, links in zip(self.parts, self._links):
            for sub, gi in zip(part.param_groups, links):
                self.param_groups[gi].update({k: v for k, v in sub.items() if k != "params"})


def _to_cpu(obj: Any) -> Any:
    if isinstance(obj, Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj
