"""Fine-grained mixture of experts with shared experts and stacked expert weights.

Parameters: ``w_gate, w_up (E, dim, hidden)``, ``w_down (E, hidden, dim)`` (``x @ W`` layout),
dense shared experts ``shared_{gate,up,down}``, ``router`` and the ``router_bias`` buffer — the
reference layout (ohara/modules/moe_grouped.py:95-117), so checkpoints interchange.

On CUDA the router runs as a split-bf16 tensor-core GEMM plus one top-k kernel (indices, gate
weights, balancing threshold and expert counts in a single launch); (token, expert) pairs are
placed into a buffer whose per-expert row groups are padded to the GEMM tile height; three
*grouped* tcgen05 GEMMs (a per-tile expert table selects the weight matrix) compute the experts, the
SwiGLU kernel fuses the activation, and a gather kernel combines with the gate weights. On CPU a
readable per-expert loop is used, which is also the oracle.

Extensions over the reference (used by the expert-parallel configuration): an optional Switch-style
auxiliary load-balancing loss (``aux_loss_coef``) and a capacity factor with drop policy
(``capacity_factor``; ``None`` keeps the reference's dropless behaviour).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ohara_b200 import ops
from ohara_b200.ops import moe as moe_ops
from ohara_b200.ops.grouped import grouped_swiglu_experts
from ohara_b200.modules.mlp import Linear
from ohara_b200.modules.routing import (
    QuantileBalancedRouter,
    is_recomputing,
    load_balance_aux_loss,
    route_tokens,
    router_logits,
)


class GroupedMoE(QuantileBalancedRouter):
    def __init__(self, dim: int, hidden_dim: int, num_experts: int = 256,
                 num_experts_per_tok: int = 8, num_shared_experts: int = 1,
                 gate_fn: str = "sigmoid", normalize_weights: bool = True,
                 quantile_balancing: bool = True, aux_loss_coef: float = 0.0,
                 capacity_factor: float | None = None) -> None:
        super().__init__()
        if not 1 <= num_experts_per_tok <= num_experts:
            raise ValueError("num_experts_per_tok must be in [1, num_experts]")
        if num_shared_experts < 0:
            raise ValueError("num_shared_experts cannot be negative")
        if gate_fn not in ("softmax", "sigmoid"):
            raise ValueError("gate_fn must be 'softmax' or 'sigmoid'")
        if quantile_balancing and num_experts_per_tok >= num_experts:
            raise ValueError(
                "quantile balancing reads the (k+1)-th logit as a threshold, so it needs "
                "num_experts_per_tok < num_experts"
            )
        if capacity_factor is not None and capacity_factor <= 0:
            raise ValueError("capacity_factor must be positive")
        self.dim = dim
        self.hidden_dim = hidden_dim
        self.num_experts = num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.num_shared_experts = num_shared_experts
        self.gate_fn = gate_fn
        self.normalize_weights = normalize_weights
        self.quantile_balancing = quantile_balancing
        self.aux_loss_coef = float(aux_loss_coef)
        self.capacity_factor = capacity_factor
        self.aux_loss: Tensor | None = None
        self.dropped_pairs: Tensor | None = None
        # Set by ``shard_experts``: the NVLink workspace of the expert-parallel group. The stacked
        # expert weights then hold only this rank's ``num_experts / world`` experts.
        self.ep_workspace = None
        self.ep_slot: int | None = None  # this layer's buffers inside the shared workspace

        self.w_gate = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.w_up = nn.Parameter(torch.empty(num_experts, dim, hidden_dim))
        self.w_down = nn.Parameter(torch.empty(num_experts, hidden_dim, dim))
        if num_shared_experts > 0:
            shared_hidden = hidden_dim * num_shared_experts
            self.shared_gate = Linear(dim, shared_hidden, bias=False)
            self.shared_up = Linear(dim, shared_hidden, bias=False)
            self.shared_down = Linear(shared_hidden, dim, bias=False)
        self.router = Linear(dim, num_experts, bias=False)
        self._register_balancing_buffers()
        self.reset_parameters()

    # -- routing -----------------------------------------------------------------------------
    def _route(self, flat_x: Tensor):
        logits = router_logits(flat_x, self.router.weight)
        indices, weights, alpha = route_tokens(
            logits, self.router_bias, self.num_experts_per_tok, self.gate_fn,
            self.quantile_balancing, normalize_sigmoid=self.normalize_weights,
        )
        return indices, weights, logits, alpha

    def _apply_capacity(self, indices: Tensor, weights: Tensor) -> Tensor:
        """Zero the weights of pairs beyond each expert's capacity (token order priority)."""
        tokens = indices.shape[0]
        capacity = int(self.capacity_factor * tokens * self.num_experts_per_tok / self.num_experts)
        capacity = max(capacity, 1)
        flat = indices.reshape(-1)
        # Position of every pair within its expert, in token order: a stable sort groups the pairs
        # by expert without disturbing their order (a cumulative sum over a pairs x experts
        # one-hot matrix does the same thing two orders of magnitude slower).
        sorted_experts, order = torch.sort(flat, stable=True)
        counts = torch.bincount(flat, minlength=self.num_experts)
        starts = counts.cumsum(0) - counts
        within = torch.arange(flat.numel(), device=flat.device) - starts[sorted_experts]
        rank = torch.empty_like(within)
        rank[order] = within
        keep = (rank < capacity).view_as(weights)
        self.dropped_pairs = (~keep).sum()
        return weights * keep.to(weights.dtype)

    # -- dispatch ----------------------------------------------------------------------------
    def _dispatch_reference(self, flat_x: Tensor, indices: Tensor, weights: Tensor) -> Tensor:
        out = torch.zeros_like(flat_x)
        k = self.num_experts_per_tok
        pair_expert = indices.reshape(-1)
        pair_weight = weights.reshape(-1)
        pair_token = torch.arange(pair_expert.numel(), device=flat_x.device) // k
        for expert in range(self.num_experts):
            chosen = pair_expert == expert
            if not bool(chosen.any()):
                continue
            rows = pair_token[chosen]
            xe = flat_x[rows]
            wg, wu, wd = (w[expert].to(xe.dtype) for w in (self.w_gate, self.w_up, self.w_down))
            ye = (F.silu(xe @ wg) * (xe @ wu)) @ wd
            out.index_add_(0, rows, (ye * pair_weight[chosen].unsqueeze(-1).to(ye.dtype)).to(out.dtype))
        return out

    def _shared(self, x: Tensor) -> Tensor:
        if (type(self.shared_gate) is Linear and type(self.shared_up) is Linear
                and ops.fused_projections(x)):
            fused = ops.linear_cat(x, (self.shared_gate.weight, self.shared_up.weight))
            return self.shared_down(ops.swiglu_cat(fused))
        return self.shared_down(ops.swiglu(self.shared_gate(x), self.shared_up(x)))

    def forward(self, x: Tensor) -> Tensor:
        batch, seq, dim = x.shape
        flat_x = x.reshape(batch * seq, dim)
        kernels = (ops.fast_path(flat_x) and dim % 8 == 0 and self.hidden_dim % 8 == 0
                   and self.num_experts <= 256 and self.num_experts_per_tok <= 16)
        counts = None
        if kernels and moe_ops.router_logits_supported(flat_x, self.router.weight):
            flat16 = flat_x if flat_x.dtype == torch.bfloat16 else flat_x.to(torch.bfloat16)
            logits = moe_ops.router_logits(flat16, self.router.weight)
            indices, weights, alpha, counts = moe_ops.route(
                logits, self.router_bias if self.quantile_balancing else None,
                self.num_experts_per_tok, self.gate_fn, self.normalize_weights,
                self.quantile_balancing,
            )
        else:
            indices, weights, logits, alpha = self._route(flat_x)
        if self.capacity_factor is not None:
            weights = self._apply_capacity(indices.long(), weights)
        if getattr(self.ep_workspace, "uses_process_group", False):
            # process-group all-to-all (ranks without peer memory, e.g. CPU ranks)
            from ohara_b200.parallel.ep_c10d import expert_parallel_swiglu_c10d

            out = expert_parallel_swiglu_c10d(flat_x, indices, weights.to(flat_x.dtype), self.w_gate,
                                              self.w_up, self.w_down, self.ep_workspace)
        elif self.ep_workspace is not None:
            if counts is None:
                raise RuntimeError("expert parallelism needs the CUDA bf16 path (router kernels)")
            from ohara_b200.parallel.ep import expert_parallel_swiglu

            out = expert_parallel_swiglu(flat_x, indices, weights, counts, self.w_gate, self.w_up,
                                         self.w_down, self.ep_workspace,
                                         self.ep_slot if torch.is_grad_enabled() else None)
        elif kernels:
            out = grouped_swiglu_experts(flat_x, indices, weights, self.w_gate, self.w_up,
                                         self.w_down, counts)
        else:
            out = self._dispatch_reference(flat_x, indices, weights.to(flat_x.dtype))
        if self.num_shared_experts > 0:
            out = out + self._shared(flat_x).to(out.dtype)
        if self.training:
            # The recomputation pass of an activation-checkpointed block repeats the operations of
            # the first pass (autograd matches the tensors they save one by one) but leaves the
            # layer's state alone: the tokens were counted the first time.
            first_pass = not is_recomputing()
            if self.aux_loss_coef > 0.0:
                aux_loss = self.aux_loss_coef * load_balance_aux_loss(
                    logits, indices.long(), self.num_experts
                )
                if first_pass:
                    self.aux_loss = aux_loss
            if first_pass:
                if self.quantile_balancing:
                    self._accumulate_qb(logits.detach(), alpha.detach())
                if counts is not None:
                    self.expert_counts += counts
                else:
                    self._record_load(indices.detach())
        return out.view(batch, seq, dim)

    # -- expert parallelism ----------------------------------------------------------------
    @torch.no_grad()
    def shard_experts(self, workspace, slot: int | None = None) -> None:
        """Keep only this rank's slice of the stacked expert weights and route the dispatch /
        combine through ``workspace`` (:class:`ohara_b200.parallel.ep.EPWorkspace`). The router,
        its bias and the shared experts stay replicated. Gradients of the expert weights already
        sum the contributions of every rank's tokens, so they are scaled by ``1 / world`` to match
        a loss averaged over the ranks, and the parameters are tagged ``expert_parallel`` so that a
        data-parallel wrapper leaves them alone."""
        world, rank = workspace.world, workspace.rank
        if self.num_experts % world or workspace.num_experts != self.num_experts:
            raise ValueError("the workspace does not match this layer's expert count")
        local = self.num_experts // world
        for name in ("w_gate", "w_up", "w_down"):
            full = getattr(self, name)
            shard = nn.Parameter(full[rank * local : (rank + 1) * local].detach().clone(),
                                 requires_grad=full.requires_grad)
            shard.expert_parallel = True
            shard.register_hook(lambda grad, scale=1.0 / world: grad * scale)
            setattr(self, name, shard)
        self.ep_workspace = workspace
        self.ep_slot = slot

    # -- init --------------------------------------------------------------------------------
    @torch.no_grad()
    def reset_parameters(self, init_std: float | None = None) -> None:
        bound = (3.0**0.5) * (init_std if init_std else self.dim**-0.5)
        nn.init.uniform_(self.w_gate, -0.4 * bound, 0.4 * bound)
        nn.init.uniform_(self.w_up, -0.4 * bound, 0.4 * bound)
        nn.init.zeros_(self.w_down)
        if self.num_shared_experts > 0:
            nn.init.uniform_(self.shared_gate.weight, -0.4 * bound, 0.4 * bound)
            nn.init.uniform_(self.shared_up.weight, -0.4 * bound, 0.4 * bound)
            nn.init.zeros_(self.shared_down.weight)
        nn.init.normal_(self.router.weight, mean=0.0, std=self.dim**-0.5)
        self.router_bias.zero_()
