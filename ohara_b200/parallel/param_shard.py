"""Parameter sharding per transformer block (what FSDP2's ``fully_shard`` does), for models that are
too large to keep a full copy of their weights on every GPU.

:class:`ohara_b200.parallel.zero.ShardedOptimizer` shards the optimizer state and the master
weights but leaves a full copy of the parameters and of the gradients on every rank. Here a rank
keeps, between uses, only ``1 / world`` of every parameter:

* the model is cut into *units* (the embedding, every block, the final norm + output projection);
* each unit's parameters are one flat fp32 vector, padded to ``world`` equal regions; rank ``r``
  owns region ``r`` as its master shard and holds optimizer state for that region only;
* before a unit runs (forward, and again backward) its vector is all-gathered into a transient
  buffer and the unit's ``nn.Parameter`` objects are pointed at views of it; the gather of the next
  unit (the previous one in the backward pass) is issued before the current unit computes, so it
  overlaps; after use the parameters are pointed back at a shape-only placeholder and the buffer
  is released;
* when the last gradient of a unit has been accumulated, the unit's gradients are packed,
  reduce-scattered (mean, asynchronously: the previous block's backward pass runs meanwhile) and
  added to the rank's fp32 gradient shard, and the full gradients are dropped. A unit some of
  whose parameters may stay without a gradient on some ranks (the loop
  MoE: experts no token chose) is reduced at the end of the backward pass instead, by every rank
  in turn.

At most two units are gathered at a time (three around the hand-over), so the parameter memory of a
rank is ``total / world`` plus about two blocks instead of ``total``.

The collectives are the process group's ``all_gather_into_tensor`` / ``reduce_scatter_tensor``
(NCCL on GPUs, gloo on CPUs, where the reduce-scatter is an all-reduce plus a slice). The reference
has nothing of the kind (``dp_shard`` is arithmetic only: ohara/runtime/topology.py:33-38).

Two layouts. ``"even"`` cuts a unit's concatenated parameters into equal ranges wherever the cut
falls (least padding; element-wise optimizers such as AdamW). ``"matrix"`` places every parameter
of a block inside one rank's range, so the owner of a matrix holds all of it and Muon runs
there without any gather (the hyperspherical recipes are not supported: they also treat the
output projection as a whole matrix, and the head is cut evenly), at the price of ranges as large as
the fullest rank's share (up to about 2x padding for a block over 8 ranks); the embedding and the
head, which those recipes update element-wise, are still cut evenly.

Limits: composes with tensor and context parallelism (the units are then this rank's tensor
shards, sharded over its data-parallel and context-parallel peers) and with hybrid sharding, not
with expert or pipeline parallelism; fp32 on the wire. Checkpoints (the model's full state dict
plus the optimizer state stored per unit as whole vectors and per matrix for the whole-matrix
groups) reload at any world size. A resharded parameter keeps its shape, ``numel()`` and ``ndim``
but reads as one repeated element: take state dicts through
:meth:`ParameterSharding.full_state_dict`.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Callable, Iterable

import torch
import torch.distributed as dist
from torch import Tensor, nn
from torch.optim import Optimizer

ALIGN = 64  # elements: every parameter starts 256 bytes into the flat vector at the least


class _Unit:
    """One all-gather / reduce-scatter granule."""

    def __init__(self, name: str, params: list[nn.Parameter], world: int, rank: int,
                 reshard_after_forward: bool, whole_tensors: bool = False) -> None:
        """``whole_tensors``: lay the unit out so that every parameter lies inside ONE rank's
        region (largest first, each to the rank with the least so far) instead of cutting the
        concatenation into equal ranges. Regions are then as large as the fullest rank's share,
        which costs padding (up to about 2x for a transformer block over 8 ranks) and buys
        whole matrices at their owners, as Muon needs."""
        self.name = name
        self.params = params
        self.reshard_after_forward = reshard_after_forward
        self.whole_tensors = whole_tensors and world > 1
        self.shapes = [tuple(p.shape) for p in params]
        self.numels = [p.numel() for p in params]
        aligned = [(n + ALIGN - 1) // ALIGN * ALIGN for n in self.numels]
        if self.whole_tensors:
            load = [0] * world
            placed: list[tuple[int, int]] = [(0, 0)] * len(params)
            for index in sorted(range(len(params)), key=lambda i: (-aligned[i], i)):
                owner = min(range(world), key=lambda r: (load[r], r))
                placed[index] = (owner, load[owner])
                load[owner] += aligned[index]
            self.region = max(max(load), ALIGN)
            self.total = self.region * world
            self.offsets = [owner * self.region + at for owner, at in placed]
        else:
            self.offsets = []
            cursor = 0
            for size in aligned:
                self.offsets.append(cursor)
                cursor += size
            chunk = world * ALIGN
            self.total = max((cursor + chunk - 1) // chunk * chunk, chunk)
            self.region = self.total // world
        device = params[0].device
        flat = torch.zeros(self.total, device=device, dtype=torch.float32)
        for p, off, n in zip(params, self.offsets, self.numels):
            flat[off : off + n].copy_(p.detach().reshape(-1).float())
        self.master = flat[rank * self.region : (rank + 1) * self.region].clone()
        self.grad: Tensor | None = None          # reduced mean gradient of this rank's region
        self.full: Tensor | None = None          # gathered vector while the unit is unsharded
        self.work: Any | None = None             # pending all-gather
        self.bound = False                       # parameters point at ``full``
        # Some parameters may get no gradient on some ranks (experts no token chose): the ranks
        # then cannot agree, from their own gradients, on when the unit is complete, so its
        # reduction waits for the end of the backward pass, where every rank does it in turn.
        self.deferred = False
        self.used = False                        # ran in a forward pass with gradients enabled
        self.trainable = sum(1 for p in params if p.requires_grad)
        self.remaining = self.trainable          # gradients still to come in this backward pass
        self.placeholders = [torch.zeros(1, device=device, dtype=torch.float32).expand(shape)
                             for shape in self.shapes]

    @property
    def gathered(self) -> bool:
        return self.full is not None and self.work is None


def _drop_compute_copies(param: nn.Parameter) -> None:
    """Forget the bf16 / fp32 compute copies that the kernels' front-ends cache on a parameter:
    they belong to the buffer the parameter pointed at before."""
    for name in ("_ohara_bf16", "_ohara_f32"):
        if getattr(param, name, None) is not None:
            setattr(param, name, None)


class _PreBackward(torch.autograd.Function):
    """Identity on a unit's outputs; its backward runs before the unit's own backward and makes
    sure the unit's parameters are gathered by then."""

    @staticmethod
    def forward(ctx, sharding, unit, *tensors):
        ctx.sharding, ctx.unit = sharding, unit
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        ctx.sharding._pre_backward(ctx.unit)
        return (None, None, *grads)


class ParameterSharding:
    """Shards ``units`` (``[(name, [parameters]), ...]`` in execution order) over ``group``.

    The model drives it: ``run_unit(name, fn, *args)`` around every unit that is released after
    its forward pass, ``enter_unit(name)`` before a unit that stays gathered until its gradients
    are complete, and ``finish_backward()`` after ``loss.backward()`` (``OharaEngine.backward``
    does that)."""

    def __init__(self, units: Iterable[tuple[str, list[nn.Parameter]]], group=None, *,
                 keep_gathered: Iterable[str] = (), prefetch: bool = True,
                 solo: bool = False, replicate_group=None, replicate_world: int = 1,
                 whole_tensor_units: Iterable[str] = ()) -> None:
        """``whole_tensor_units``: names of units laid out with every parameter inside one rank's
        region (see :class:`_Unit`). ``solo``: shard over nobody although a process group
        exists (every other rank of the
        job holds different tensors, e.g. the tensor-parallel peers). ``replicate_group`` (of
        ``replicate_world`` ranks): hybrid sharding, the ranks that hold the same shard as this
        one in other replica groups; reduced gradient shards are averaged over it."""
        self.group = group
        self.replicate_group = replicate_group
        self.replicate_world = int(replicate_world) if dist.is_initialized() else 1
        distributed = dist.is_available() and dist.is_initialized() and not solo
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        self.prefetch = prefetch
        keep = set(keep_gathered)
        whole = set(whole_tensor_units)
        seen: set[int] = set()
        self.units: list[_Unit] = []
        self.by_name: dict[str, _Unit] = {}
        self.unit_of_param: dict[int, _Unit] = {}
        for name, params in units:
            fresh = [p for p in params if id(p) not in seen]
            if not fresh:
                continue
            seen.update(id(p) for p in fresh)
            unit = _Unit(name, fresh, self.world, self.rank, name not in keep,
                         whole_tensors=name in whole)
            unit.index = len(self.units)
            self.units.append(unit)
            self.by_name[name] = unit
            for p in fresh:
                self.unit_of_param[id(p)] = unit
                if p.requires_grad:
                    p.register_post_accumulate_grad_hook(self._on_gradient)
        # Set by the engine under sequence-parallel tensor parallelism: the ranks of this group
        # see different tokens, so gradients of parameters that are NOT tensor-parallel shards
        # are partial sums and are added up over it before the data-parallel reduction.
        self.partial_gradient_group = None   # (``None`` is also the default group: see the flag)
        self.partial_gradients = False
        self._reductions: list[tuple[_Unit, Any, Tensor | None, Tensor]] = []   # in flight
        self.unsharded_bytes = sum(sum(u.numels) for u in self.units) * 4
        self.peak_gathered_bytes = 0
        for unit in self.units:
            self._release(unit)

    # -- gather / release ------------------------------------------------------------------------
    def _issue(self, unit: _Unit, asynchronous: bool) -> None:
        if unit.full is not None:
            return
        unit.full = torch.empty(unit.total, device=unit.master.device, dtype=torch.float32)
        if self.world == 1:
            unit.full.copy_(unit.master)
            return
        work = dist.all_gather_into_tensor(unit.full, unit.master, group=self.group,
                                           async_op=asynchronous)
        unit.work = work if asynchronous else None

    def _bind(self, unit: _Unit) -> None:
        if unit.work is not None:
            unit.work.wait()
            unit.work = None
        for p, off, n, shape in zip(unit.params, unit.offsets, unit.numels, unit.shapes):
            view = unit.full[off : off + n].view(shape)
            # Vectors (norm weights) get their own small tensor: kernels keep a reference to the
            # fp32 vector for their backward pass, and a view would keep the whole gathered
            # buffer alive until then.
            p.data = view.clone() if len(shape) <= 1 else view
            _drop_compute_copies(p)
        unit.bound = True
        gathered = sum(u.total for u in self.units if u.full is not None) * 4
        self.peak_gathered_bytes = max(self.peak_gathered_bytes, gathered)

    def unshard(self, unit: _Unit) -> None:
        """Gather ``unit`` now (waits for a prefetch in flight) and point its parameters at it."""
        if unit.gathered and unit.bound:
            return
        self._issue(unit, asynchronous=False)
        self._bind(unit)

    def _release(self, unit: _Unit) -> None:
        if unit.work is not None:
            unit.work.wait()
            unit.work = None
        for p, placeholder in zip(unit.params, unit.placeholders):
            p.data = placeholder
            _drop_compute_copies(p)
        unit.full = None
        unit.bound = False

    def _neighbour(self, unit: _Unit, step: int) -> _Unit | None:
        index = unit.index + step
        return self.units[index] if 0 <= index < len(self.units) else None

    # -- what the model calls --------------------------------------------------------------------
    def enter_unit(self, name: str, prefetch_next: bool = True) -> None:
        """Gather a unit that stays gathered until its gradients are complete (or, without a
        backward pass, until ``release_all``)."""
        unit = self.by_name[name]
        self.unshard(unit)
        following = self._neighbour(unit, +1)
        if self.prefetch and prefetch_next and following is not None:
            self._issue(following, asynchronous=True)

    def run_unit(self, name: str, fn: Callable, *args):
        """``fn(*args)`` with the unit's parameters gathered; released again afterwards."""
        unit = self.by_name[name]
        self.unshard(unit)
        following = self._neighbour(unit, +1)
        if self.prefetch and following is not None:
            self._issue(following, asynchronous=True)
        out = fn(*args)
        if torch.is_grad_enabled():
            unit.used = True
            # backward of the marker runs before the unit's own backward: gather (a unit that
            # stayed gathered is there already) and prefetch the unit before it
            single = isinstance(out, Tensor)
            items = (out,) if single else tuple(out)
            live = [i for i, t in enumerate(items) if isinstance(t, Tensor) and t.requires_grad]
            if live:
                marked = _PreBackward.apply(self, unit, *[items[i] for i in live])
                items = list(items)
                for i, t in zip(live, marked):
                    items[i] = t
                out = items[0] if single else tuple(items)
        if unit.reshard_after_forward or not torch.is_grad_enabled():
            self._release(unit)
        return out

    def _pre_backward(self, unit: _Unit) -> None:
        self.unshard(unit)
        previous = self._neighbour(unit, -1)
        if self.prefetch and previous is not None and previous.trainable:
            self._issue(previous, asynchronous=True)

    # -- gradients -------------------------------------------------------------------------------
    def _on_gradient(self, param: nn.Parameter) -> None:
        unit = self.unit_of_param[id(param)]
        unit.remaining -= 1
        if unit.remaining == 0 and not unit.deferred:
            self._reduce(unit)

    @torch.no_grad()
    def _reduce(self, unit: _Unit, always: bool = False) -> None:
        """Pack the unit's gradients, reduce-scatter the mean into this rank's gradient shard,
        drop the full gradients and release the unit. ``always``: take part in the collective
        even if this rank has no gradient for the unit (its peers may)."""
        unit.used = False
        if unit.trainable and (always or any(p.grad is not None for p in unit.params)):
            flat = torch.zeros(unit.total, device=unit.master.device, dtype=torch.float32)
            for p, off, n in zip(unit.params, unit.offsets, unit.numels):
                if p.grad is not None:
                    flat[off : off + n].copy_(p.grad.reshape(-1))
                    p.grad = None
            if self.partial_gradients:
                for p, off, n in zip(unit.params, unit.offsets, unit.numels):
                    if not hasattr(p, "tensor_parallel_dim"):
                        dist.all_reduce(flat[off : off + n], group=self.partial_gradient_group)
            if self.world == 1:
                self._accumulate(unit, flat)
            else:
                # Asynchronous: the backward pass of the next block runs while this block's
                # gradients are on the wire. At most two reductions are in flight (each holds one
                # block-sized buffer); older ones are completed first.
                while len(self._reductions) >= 2:
                    self._complete(self._reductions.pop(0))
                if dist.get_backend(self.group) == "gloo":  # gloo has no reduce-scatter
                    work = dist.all_reduce(flat, group=self.group, async_op=True)
                    shard = None
                else:
                    shard = torch.empty(unit.region, device=flat.device, dtype=torch.float32)
                    work = dist.reduce_scatter_tensor(shard, flat, group=self.group, async_op=True)
                self._reductions.append((unit, work, shard, flat))
        unit.remaining = unit.trainable
        self._release(unit)

    def _complete(self, reduction) -> None:
        """Wait for a reduce-scatter in flight and add its mean to the unit's gradient shard."""
        unit, work, shard, flat = reduction
        work.wait()
        if shard is None:  # an all-reduce of the whole vector stood in for the reduce-scatter
            shard = flat[self.rank * unit.region : (self.rank + 1) * unit.region].clone()
        shard.div_(self.world)
        self._accumulate(unit, shard)

    def _accumulate(self, unit: _Unit, shard: Tensor) -> None:
        if self.replicate_world > 1:
            dist.all_reduce(shard, group=self.replicate_group)
            shard.div_(self.replicate_world)
        unit.grad = shard if unit.grad is None else unit.grad.add_(shard)

    def _drain_reductions(self) -> None:
        while self._reductions:
            self._complete(self._reductions.pop(0))

    def finish_backward(self) -> None:
        """After ``backward()``: units whose gradients did not all arrive (unused parameters), or
        that were gathered by a prefetch and never used, are reduced and released here."""
        for unit in reversed(self.units):
            if unit.deferred and unit.used:
                self._reduce(unit, always=True)
            elif unit.full is not None or unit.remaining != unit.trainable:
                self._reduce(unit)
        self._drain_reductions()

    def release_all(self) -> None:
        """Release every gathered unit (after an evaluation or generation pass)."""
        for unit in self.units:
            if unit.full is not None:
                self._release(unit)

    # -- whole-model access ------------------------------------------------------------------------
    @contextmanager
    def gathered(self):
        """All parameters readable (and writable: changes are copied back into the master shards
        on exit)."""
        for unit in self.units:
            self.unshard(unit)
        try:
            yield
        finally:
            with torch.no_grad():
                for unit in self.units:
                    for p, off, n, shape in zip(unit.params, unit.offsets, unit.numels,
                                                unit.shapes):
                        if len(shape) <= 1:  # vectors are bound as copies (see _bind)
                            unit.full[off : off + n].copy_(p.detach().reshape(-1))
                    lo = self.rank * unit.region
                    unit.master.copy_(unit.full[lo : lo + unit.region])
                    self._release(unit)

    def full_state_dict(self, module: nn.Module) -> dict[str, Tensor]:
        """``module.state_dict()`` with every parameter whole (collective; clones)."""
        with self.gathered():
            return {k: v.detach().clone() for k, v in module.state_dict().items()}

    def load_full_state_dict(self, module: nn.Module, state: dict[str, Tensor], strict: bool = True):
        with self.gathered():
            return module.load_state_dict(state, strict=strict)

    def memory_report(self) -> dict[str, int]:
        """Bytes of parameter storage: what a rank keeps between uses, the most it held gathered
        at one time so far, and what an unsharded copy takes."""
        persistent = sum(u.region for u in self.units) * 4
        return {"persistent_bytes_per_rank": persistent,
                "peak_gathered_bytes": self.peak_gathered_bytes,
                "unsharded_bytes": self.unsharded_bytes}


def shard_llama(model: nn.Module, group=None, prefetch: bool = True, solo: bool = False,
                replicate_group=None, replicate_world: int = 1,
                layout: str = "even") -> ParameterSharding:
    """Cut a Llama into units (embedding, blocks, final norm + output projection), shard them over
    ``group`` and attach the result as ``model._param_sharding``; the model's forward pass then
    gathers and releases the units as it goes."""
    if not all(hasattr(model, name) for name in ("token_emb", "layers", "norm", "vocab_proj")):
        raise ValueError("parameter sharding needs a Llama-style model")
    if getattr(model, "_param_sharding", None) is not None:
        raise RuntimeError("this model's parameters are sharded already")
    tied = model.vocab_proj.weight is model.token_emb.weight
    units: list[tuple[str, list[nn.Parameter]]] = []
    keep = ["head"]
    if tied:
        # one unit for the shared matrix: it is used first and last, so it stays gathered
        units.append(("embed", [model.token_emb.weight, *model.norm.parameters()]))
        keep.append("embed")
    else:
        units.append(("embed", list(model.token_emb.parameters())))
    from ohara_b200.modules.moe import MoE

    deferred: list[str] = []
    for index, layer in enumerate(model.layers):
        units.append((f"layers.{index}", list(layer.parameters())))
        if any(isinstance(m, MoE) for m in layer.modules()):
            # an expert no token of this rank chose gets no gradient: reduce at the end of the
            # backward pass, when every rank knows the unit is as complete as it will get
            deferred.append(f"layers.{index}")
    if len(model.layers) > 0:
        # the last block's backward starts right after its forward: keep it gathered
        keep.append(f"layers.{len(model.layers) - 1}")
    if not tied:
        units.append(("head", [*model.norm.parameters(), *model.vocab_proj.parameters()]))
    covered = {id(p) for _, params in units for p in params}
    missing = [name for name, p in model.named_parameters() if id(p) not in covered]
    if missing:
        raise ValueError(f"parameters outside every unit: {missing[:4]}")
    if layout not in ("even", "matrix"):
        raise ValueError(f"unknown parameter-sharding layout {layout!r} (even or matrix)")
    # "matrix": the blocks keep every matrix whole at one owner (what Muon needs); the embedding
    # and the head, which element-wise algorithms update, are still cut evenly
    whole = [name for name, _ in units if name.startswith("layers.")] if layout == "matrix" else []
    sharding = ParameterSharding(units, group, keep_gathered=keep, prefetch=prefetch, solo=solo,
                                 replicate_group=replicate_group, replicate_world=replicate_world,
                                 whole_tensor_units=whole)
    for name in deferred:
        sharding.by_name[name].deferred = True
    sharding.tied = tied
    model._param_sharding = sharding
    return sharding


class ParameterShardedOptimizer(Optimizer):
    """Runs ``optimizer``'s algorithm on this rank's master shards of a :class:`ParameterSharding`.

    ``optimizer`` was built on the model's parameters; its groups (learning rate, weight decay
    ...) are kept as the user-visible ``param_groups`` and mirrored onto a local optimizer of the
    same class over views of the master shards: 1-D ranges for element-wise groups, whole
    matrices at their owners for whole-matrix groups (which need the ``"matrix"`` layout)."""

    def __init__(self, optimizer: Optimizer, sharding: ParameterSharding,
                 norm_groups: dict[str, Any] | None = None) -> None:
        """``norm_groups["tp"]``: the tensor-parallel group, over which the squared norms of
        tensor-parallel shards add up for the global gradient norm (replicated parameters are
        counted once)."""
        self.inner = optimizer
        self.sharding = sharding
        self.norm_groups = dict(norm_groups or {})
        self._tp_spans: dict[str, list[tuple[int, int]]] = {}
        for unit in sharding.units:
            lo, hi = sharding.rank * unit.region, (sharding.rank + 1) * unit.region
            spans = []
            for p, off, n in zip(unit.params, unit.offsets, unit.numels):
                a, b = max(off, lo), min(off + n, hi)
                if a < b and hasattr(p, "tensor_parallel_dim"):
                    spans.append((a - lo, b - lo))
            self._tp_spans[unit.name] = spans
        self.param_groups = optimizer.param_groups
        self.defaults = optimizer.defaults
        self.state = optimizer.state
        local_groups = []
        self._spans: list[list[tuple[_Unit, int, int, nn.Parameter]]] = []
        self._whole_matrix_group: list[bool] = []
        for group in self.param_groups:
            whole_matrices = group.get("kind") == "muon" or bool(group.get("hypersphere", False))
            self._whole_matrix_group.append(whole_matrices)
            wanted = {id(p) for p in group["params"]}
            spans: list[tuple[_Unit, int, int, nn.Parameter]] = []
            for unit in sharding.units:
                lo, hi = sharding.rank * unit.region, (sharding.rank + 1) * unit.region
                if whole_matrices:
                    # the owner of a matrix updates all of it: every matrix of the group must lie
                    # inside one rank's region (the "matrix" layout of the blocks)
                    for p, off, n, shape in zip(unit.params, unit.offsets, unit.numels,
                                                unit.shapes):
                        if id(p) not in wanted:
                            continue
                        if off // unit.region != (off + n - 1) // unit.region:
                            if unit.whole_tensors:
                                raise RuntimeError(f"{unit.name}: a parameter straddles regions")
                            raise NotImplementedError(
                                f"a whole-matrix algorithm needs every matrix of its groups at "
                                f"one owner, but unit '{unit.name}' is cut evenly. Muon on the "
                                f"blocks' matrices works with the 'matrix' layout "
                                f"(EngineConfig(shard_parameters_layout='matrix')); the "
                                f"hyperspherical recipes (AdamH / MuonH) also put the output "
                                f"projection on a sphere, which the evenly cut head unit does "
                                f"not support")
                        if lo <= off < hi:
                            shard = nn.Parameter(unit.master[off - lo : off - lo + n].view(shape),
                                                 requires_grad=True)
                            if hasattr(p, "tensor_parallel_dim"):  # tensor-parallel Muon needs it
                                shard.tensor_parallel_dim = p.tensor_parallel_dim
                            shard._matrix_id = (unit.name, unit.offsets.index(off))
                            spans.append((unit, off - lo, off - lo + n, shard))
                    continue
                pieces: list[list[int]] = []
                for p, off, n in zip(unit.params, unit.offsets, unit.numels):
                    if id(p) not in wanted:
                        continue
                    a, b = max(off, lo), min(off + n, hi)
                    if a >= b:
                        continue
                    if pieces and pieces[-1][1] == a - lo:
                        pieces[-1][1] = b - lo
                    else:
                        pieces.append([a - lo, b - lo])
                for a, b in pieces:
                    shard = nn.Parameter(unit.master[a:b], requires_grad=True)
                    spans.append((unit, a, b, shard))
            self._spans.append(spans)
            if spans:
                clone = {k: v for k, v in group.items() if k != "params"}
                clone["params"] = [s[3] for s in spans]
                local_groups.append(clone)
        self._local_of_group = []
        index = 0
        for spans in self._spans:
            self._local_of_group.append(index if spans else None)
            index += 1 if spans else 0
        self.local: Optimizer | None = None
        if local_groups:
            cls = getattr(optimizer, "optimizer_class", None) or type(optimizer)
            try:
                self.local = cls(local_groups)
            except TypeError:
                self.local = cls(local_groups, **dict(optimizer.defaults))
            for name in ("tensor_parallel_group", "tensor_parallel_world"):
                if hasattr(optimizer, name):
                    setattr(self.local, name, getattr(optimizer, name))

    # -- step ------------------------------------------------------------------------------------
    def _sync_hyperparameters(self) -> None:
        if self.local is None:
            return
        for group, local_index in zip(self.param_groups, self._local_of_group):
            if local_index is None:
                continue
            target = self.local.param_groups[local_index]
            for key, value in group.items():
                if key != "params":
                    target[key] = value

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.sharding.finish_backward()
        self._sync_hyperparameters()
        if self.local is not None:
            for spans in self._spans:
                for unit, a, b, shard in spans:
                    shard.grad = (unit.grad[a:b].view_as(shard) if unit.grad is not None
                                  else torch.zeros_like(shard))
            self.local.step()
            for spans in self._spans:
                for _, _, _, shard in spans:
                    shard.grad = None
        return loss

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.sharding._drain_reductions()
        for unit in self.sharding.units:
            unit.grad = None
            for p in unit.params:
                p.grad = None

    @torch.no_grad()
    def grad_sq_norm(self) -> Tensor:
        self.sharding.finish_backward()
        device = self.sharding.units[0].master.device
        sums = torch.zeros(2, device=device, dtype=torch.float32)   # everything, tensor shards
        for unit in self.sharding.units:
            if unit.grad is None:
                continue
            sums[0] += unit.grad.square().sum()
            for a, b in self._tp_spans[unit.name]:
                sums[1] += unit.grad[a:b].square().sum()
        if self.sharding.world > 1:
            dist.all_reduce(sums, group=self.sharding.group)
        if "tp" not in self.norm_groups:
            return sums[0]
        shards = sums[1].clone()
        dist.all_reduce(shards, group=self.norm_groups["tp"])   # distinct on every tp rank
        return sums[0] - sums[1] + shards

    @torch.no_grad()
    def clip_grad_norm_(self, model, max_norm: float) -> Tensor:
        norm = self.grad_sq_norm().sqrt()
        scale = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        for unit in self.sharding.units:
            if unit.grad is not None:
                unit.grad.mul_(scale)
        return norm

    def sync_master_weights(self) -> None:
        """Nothing to do: the master shards are the only copy (state dicts go through
        ``ParameterSharding.full_state_dict``)."""

    # -- checkpoints -----------------------------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        """The optimizer state laid out per unit as whole flat vectors (collective; identical on
        all ranks, so the rank that writes the checkpoint has all of it). The layout does not
        depend on the number of ranks: a checkpoint reloads at any world size. The weights
        themselves travel in the model's full state dict."""
        sharding = self.sharding
        mine = []
        matrices: dict[tuple[str, int], dict[str, Tensor]] = {}
        for index, spans in enumerate(self._spans):
            if self._whole_matrix_group[index]:
                # one stacked buffer per state entry, keyed on the group's first matrix, one row
                # per owned matrix in group order: store the rows per matrix
                if spans and self.local is not None:
                    stacked = self.local.state.get(spans[0][3], {})
                    for row, (_, _, _, shard) in enumerate(spans):
                        matrices[shard._matrix_id] = {
                            k: v[row].detach().cpu() for k, v in stacked.items()
                            if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == len(spans)}
                continue
            for unit, a, b, shard in spans:
                state = self.local.state.get(shard, {}) if self.local is not None else {}
                vectors = {k: v.detach().reshape(-1).cpu() for k, v in state.items()
                           if torch.is_tensor(v) and v.dim() > 0 and v.numel() == b - a}
                scalars = {k: (v.detach().cpu() if torch.is_tensor(v) else v)
                           for k, v in state.items() if k not in vectors}
                mine.append((index, unit.name, sharding.rank * unit.region + a, vectors, scalars))
        everyone: list[Any] = [mine]
        if sharding.world > 1:
            everyone = [None] * sharding.world
            dist.all_gather_object(everyone, mine, group=sharding.group)
            parts: list[Any] = [None] * sharding.world
            dist.all_gather_object(parts, matrices, group=sharding.group)
            matrices = {key: value for part in parts for key, value in part.items()}
        units: dict[str, dict[str, Tensor]] = {}
        scalars_of_group: dict[int, dict[str, Any]] = {}
        for pieces in everyone:
            for index, name, begin, vectors, scalars in pieces:
                total = sharding.by_name[name].total
                for key, vector in vectors.items():
                    full = units.setdefault(name, {}).setdefault(
                        key, torch.zeros(total, dtype=vector.dtype))
                    full[begin : begin + vector.numel()] = vector
                if scalars:
                    scalars_of_group.setdefault(index, scalars)
        return {
            "param_sharded": True,
            "units": units,
            "matrices": matrices,
            "group_scalars": scalars_of_group,
            "param_groups": [{k: v for k, v in g.items() if k != "params"}
                             for g in self.param_groups],
        }

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        if not state_dict.get("param_sharded"):
            raise ValueError("not a parameter-sharded optimizer state")
        sharding = self.sharding
        for index, spans in enumerate(self._spans):
            if self._whole_matrix_group[index]:
                saved_rows = [state_dict.get("matrices", {}).get(shard._matrix_id)
                              for _, _, _, shard in spans]
                if spans and all(saved_rows) and self.local is not None:
                    first = spans[0][3]
                    for key in saved_rows[0]:
                        self.local.state[first][key] = torch.stack(
                            [rows[key] for rows in saved_rows]).to(first.device)
                continue
            scalars = state_dict["group_scalars"].get(index, {})
            for unit, a, b, shard in spans:
                saved = state_dict["units"].get(unit.name)
                if not saved:
                    continue
                begin = sharding.rank * unit.region + a
                state = self.local.state[shard]
                for key, full in saved.items():
                    # the tail padding of a unit depends on the world size it was saved at
                    piece = torch.zeros(b - a, dtype=full.dtype)
                    available = max(0, min(b - a, full.numel() - begin))
                    piece[:available] = full[begin : begin + available]
                    state[key] = piece.to(shard.device).view_as(shard)
                for key, value in scalars.items():
                    state[key] = value.clone() if torch.is_tensor(value) else value
        for group, saved in zip(self.param_groups, state_dict["param_groups"]):
            group.update(saved)
        self._sync_hyperparameters()
