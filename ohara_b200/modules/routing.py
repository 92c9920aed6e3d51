"""Top-k routing and quantile balancing shared by the loop and grouped mixture-of-experts layers.

Routing rule (reference: ohara/modules/moe.py:65-154, ohara/modules/moe_grouped.py:122-147,
232-257): router logits are fp32; experts are *selected* by ``logits + router_bias`` but *weighted*
by the unbiased logits; with quantile balancing the (k+1)-th biased logit of each token is its
threshold ``alpha``. After each optimizer step the bias is re-solved in closed form from the
per-expert quantile of ``logit - alpha`` (no auxiliary loss).
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor


def router_logits(flat: Tensor, weight: Tensor) -> Tensor:
    """fp32 router scores ``flat @ weight.T`` regardless of any surrounding autocast region."""
    with torch.autocast(device_type=flat.device.type, enabled=False):
        return torch.nn.functional.linear(flat.float(), weight.float())


_RECOMPUTING = False


class recomputing:
    """Context manager for the second forward pass of an activation-checkpointed block: routers
    inside it do not count the tokens again (load, balancing statistics)."""

    def __enter__(self):
        global _RECOMPUTING
        self._previous = _RECOMPUTING
        _RECOMPUTING = True
        return self

    def __exit__(self, *exc):
        global _RECOMPUTING
        _RECOMPUTING = self._previous
        return False


def is_recomputing() -> bool:
    return _RECOMPUTING


def route_tokens(logits: Tensor, router_bias: Tensor, k: int, gate_fn: str,
                 quantile_balancing: bool, normalize_sigmoid: bool = False):
    """Return ``(expert_indices (N,k), expert_weights (N,k) fp32, alpha (N,1) | None)``."""
    alpha = None
    if quantile_balancing:
        top = torch.topk(logits + router_bias, k + 1, dim=-1)
        alpha = top.values[:, -1:]
        indices = top.indices[:, :k]
    else:
        indices = torch.topk(logits, k, dim=-1).indices
    chosen = logits.gather(-1, indices)
    if gate_fn == "softmax":
        weights = chosen.softmax(dim=-1)
    else:
        weights = torch.sigmoid(chosen)
        if normalize_sigmoid:
            weights = weights / weights.sum(dim=-1, keepdim=True).clamp_min(1e-9)
    return indices, weights, alpha


def load_balance_aux_loss(logits: Tensor, indices: Tensor, num_experts: int) -> Tensor:
    """Switch-style auxiliary loss ``E * sum_e f_e * p_e`` (f = routed fraction, p = mean softmax
    probability). An extension over the reference's ``ohara`` package, which balances only through
    the router bias; the same loss appears in experiments/deepseek_moe/dsmoe.py:211-225."""
    probs = logits.softmax(dim=-1).mean(dim=0)
    counts = torch.bincount(indices.reshape(-1), minlength=num_experts).to(probs.dtype)
    fraction = counts / max(indices.numel(), 1)
    return num_experts * torch.sum(fraction * probs)


def global_kth_largest(values: Tensor, k: int | Tensor, group=None) -> Tensor:
    """Per column of ``values (N, E)`` fp32, the ``k``-th largest entry over the rows of *every*
    rank of ``group`` (each rank passes its own rows; ``k`` counts over all of them).

    Exact radix select on an order-preserving integer image of the floats: four passes, most
    significant byte first; each pass builds a per-column histogram of the current byte among the
    entries that still match the prefix found so far, sums the histograms over the group (the
    only communication: ``E x 256`` counters) and descends into the byte that contains the
    ``k``-th entry. No sort, no host synchronisation, identical result on every rank.

    The reference averages per-rank quantiles instead (ohara/modules/moe_grouped.py:249-251),
    which is not the quantile of the union when ranks see differently distributed tokens."""
    n, e = values.shape
    bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    negative = bits >= 0x80000000
    keys = torch.where(negative, bits ^ 0xFFFFFFFF, bits | 0x80000000)  # larger float, larger key
    column = torch.arange(e, device=values.device).expand(n, e)
    remaining = torch.as_tensor(k, device=values.device, dtype=torch.int64).expand(e).clone()
    prefix = torch.zeros(e, device=values.device, dtype=torch.int64)
    distributed = dist.is_available() and dist.is_initialized()
    for shift in (24, 16, 8, 0):
        alive = (keys >> (shift + 8)) == prefix if shift < 24 else torch.ones_like(keys, dtype=torch.bool)
        byte = (keys >> shift) & 0xFF
        hist = torch.zeros(e * 256, device=values.device, dtype=torch.int64)
        hist.scatter_add_(0, (column * 256 + byte).reshape(-1), alive.reshape(-1).to(torch.int64))
        if distributed:
            dist.all_reduce(hist, group=group)
        from_top = hist.view(e, 256).flip(1).cumsum(1)            # entries with byte >= 255 - j
        position = (from_top >= remaining[:, None]).to(torch.int64).argmax(1)
        above = torch.where(position > 0,
                            from_top.gather(1, (position - 1).clamp_min(0)[:, None]).squeeze(1),
                            torch.zeros_like(remaining))
        remaining = remaining - above
        prefix = (prefix << 8) | (255 - position)
    back = torch.where(prefix >= 0x80000000, prefix ^ 0x80000000, prefix ^ 0xFFFFFFFF)
    back = torch.where(back >= 0x80000000, back - (1 << 32), back)  # as signed 32-bit
    return back.to(torch.int32).view(torch.float32)


class QuantileBalancedRouter(nn.Module):
    """Mixin holding the router bias and the balancing statistics buffers."""

    num_experts: int
    num_experts_per_tok: int
    quantile_balancing: bool

    def _register_balancing_buffers(self) -> None:
        e = self.num_experts
        self.register_buffer("router_bias", torch.zeros(e))
        self.register_buffer("qb_beta_sum", torch.zeros(e), persistent=False)
        self.register_buffer("qb_beta_count", torch.zeros(()), persistent=False)
        self.register_buffer("expert_counts", torch.zeros(e, dtype=torch.long), persistent=False)

    # Set by the engine under expert parallelism: the balancing statistic then is the quantile over
    # the tokens of every rank of this group (all of which route through the same experts), not
    # an average of per-rank quantiles.
    qb_global_group = None
    qb_global = False
    qb_global_world = 1

    @torch.no_grad()
    def _accumulate_qb(self, logits: Tensor, alpha: Tensor) -> None:
        tokens = logits.size(0)
        if self.qb_global:
            total = tokens * self.qb_global_world
            fair_share = min(max(1, total * self.num_experts_per_tok // self.num_experts), total)
            margin = logits.float() - alpha.float().view(-1, 1)
            self.qb_beta_sum += global_kth_largest(margin, fair_share, self.qb_global_group)
            self.qb_beta_count += 1
            return
        fair_share = max(1, tokens * self.num_experts_per_tok // self.num_experts)
        fair_share = min(fair_share, tokens)
        if logits.is_cuda and logits.dtype == torch.float32:
            from ohara_b200.ops.moe import accumulate_quantile

            # exact radix select per expert instead of a sort over (experts, tokens)
            accumulate_quantile(logits, alpha.float(), self.qb_beta_sum, fair_share)
        else:
            margin = logits - alpha.view(-1, 1)  # expert e wins a token when its margin is positive
            self.qb_beta_sum += torch.topk(margin.t(), fair_share, dim=-1).values[:, -1]
        self.qb_beta_count += 1

    @torch.no_grad()
    def _record_load(self, indices: Tensor) -> None:
        self.expert_counts += torch.bincount(indices.reshape(-1), minlength=self.num_experts)

    @torch.no_grad()
    def apply_qb_update(self, group=None) -> None:
        """Fold the statistics of this optimizer step into ``router_bias`` (mean-zero)."""
        # "nothing accumulated" is decided on the device (a host read here would stall the launch
        # queue once per layer and step): with a zero count the old bias is kept.
        seen = self.qb_beta_count > 0
        beta = self.qb_beta_sum / self.qb_beta_count.clamp_min(1)
        if dist.is_available() and dist.is_initialized() and not self.qb_global:
            dist.all_reduce(beta, op=dist.ReduceOp.SUM, group=group)
            beta /= dist.get_world_size(group=group)
        bias = -beta
        self.router_bias.copy_(torch.where(seen, bias - bias.mean(), self.router_bias))
        self.qb_beta_sum.zero_()
        self.qb_beta_count.zero_()

    @torch.no_grad()
    def expert_load(self, reset: bool = True) -> Tensor:
        counts = self.expert_counts.clone()
        if reset:
            self.expert_counts.zero_()
        return counts


def apply_qb_update(module: nn.Module) -> None:
    """Run ``apply_qb_update`` on every balancing MoE layer of ``module``."""
    for layer in module.modules():
        if isinstance(layer, QuantileBalancedRouter) and layer.quantile_balancing:
            layer.apply_qb_update()


def expert_load(module: nn.Module, reset: bool = True) -> Tensor | None:
    """Tokens routed to each expert since the last reset for every MoE layer of ``module``,
    stacked ``(num_moe_layers, num_experts)``; ``None`` without MoE layers (reference:
    ohara/modules/moe.py:194-203)."""
    counts = [
        layer.expert_load(reset=reset)
        for layer in module.modules()
        if isinstance(layer, QuantileBalancedRouter)
    ]
    return torch.stack(counts) if counts else None


def maximal_violation(counts: Tensor) -> Tensor:
    """MaxVio = max_e load_e / mean load − 1 along the last dimension (one value per layer for a
    stacked count table); zero means perfectly balanced. Rows without any token give zero."""
    counts = counts.float()
    mean = counts.mean(dim=-1, keepdim=True)
    violation = (counts.max(dim=-1, keepdim=True).values - mean) / mean.clamp_min(1e-12)
    return torch.where(mean > 0, violation, torch.zeros_like(violation)).squeeze(-1)
