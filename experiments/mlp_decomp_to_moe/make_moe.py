"""Cut a trained dense feed-forward layer into a mixture of experts (reference:
experiments/mlp_decomp_to_moe/make_moe.py:29-39, which clusters the rows and stops at
"TODO: create router").

The hidden units of a gated MLP are independent: ``down(act(gate x) * up x)`` is a sum over hidden
units, so any partition of the units into ``E`` groups gives ``E`` experts whose outputs add up to
the dense layer exactly. Here the units are grouped by balanced k-means on their normalised
``gate`` rows (units that react to similar inputs share an expert; equal sizes keep the experts one
stacked tensor), and the router the reference leaves open scores expert ``e`` by how strongly its
units' gates fire: ``score_e(x) = mean over units of e of |act(gate_row . x)|`` approximated
linearly by the expert's mean gate direction. With ``top_k = E`` the result equals the dense layer;
smaller ``top_k`` trades accuracy for compute.

``balanced_kmeans`` is self-contained (the reference needs ``k_means_constrained`` and
scikit-learn): Lloyd iterations whose assignment step fills clusters greedily in order of the
margin between a point's best and second-best centre, with every cluster capped at ``n / k``."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


def _balanced_assign(distance: Tensor, capacity: int) -> Tensor:
    points, clusters = distance.shape
    order = torch.argsort(distance, dim=1)
    best2 = distance.gather(1, order[:, :2]) if clusters > 1 else distance.repeat(1, 2)
    # points that lose most by not getting their first choice choose first
    priority = torch.argsort(best2[:, 1] - best2[:, 0], descending=True)
    room = [capacity] * clusters
    labels = torch.empty(points, dtype=torch.long)
    for p in priority.tolist():
        for c in order[p].tolist():
            if room[c] > 0:
                room[c] -= 1
                labels[p] = c
                break
    return labels


def balanced_kmeans(points: Tensor, clusters: int, iterations: int = 20, seed: int = 0) -> Tensor:
    """Labels in ``[0, clusters)`` with exactly ``len(points) / clusters`` points each."""
    count = points.shape[0]
    if count % clusters:
        raise ValueError("the number of points must divide into the clusters")
    generator = torch.Generator().manual_seed(seed)
    centres = points[torch.randperm(count, generator=generator)[:clusters]].clone()
    labels = None
    for _ in range(iterations):
        new = _balanced_assign(torch.cdist(points, centres), count // clusters)
        if labels is not None and torch.equal(new, labels):
            break
        labels = new
        for c in range(clusters):
            centres[c] = points[labels == c].mean(0)
    return labels


def split_weights_into_experts(ffn_weight: Tensor, split_num: int) -> list[Tensor]:
    """Rows of a ``(hidden, dim)`` matrix grouped into ``split_num`` equally sized experts."""
    labels = balanced_kmeans(F.normalize(ffn_weight.float(), dim=1), split_num)
    return [ffn_weight[labels == e] for e in range(split_num)]


class DecomposedMoE(nn.Module):
    """``E`` experts cut out of one gated MLP, stacked, with a top-k router."""

    def __init__(self, gate: Tensor, up: Tensor, down: Tensor, labels: Tensor, num_experts: int,
                 top_k: int, activation=F.silu) -> None:
        super().__init__()
        order = torch.argsort(labels, stable=True)
        per = gate.shape[0] // num_experts
        self.num_experts, self.top_k, self.activation = num_experts, top_k, activation
        self.w_gate = nn.Parameter(gate[order].reshape(num_experts, per, -1).clone())   # (E, h, d)
        self.w_up = nn.Parameter(up[order].reshape(num_experts, per, -1).clone())
        self.w_down = nn.Parameter(down[:, order].reshape(down.shape[0], num_experts, per)
                                   .permute(1, 0, 2).clone())                            # (E, d, h)
        self.router = nn.Linear(gate.shape[1], num_experts, bias=False)
        with torch.no_grad():  # an expert is chosen when the input points along its gate rows
            self.router.weight.copy_(F.normalize(self.w_gate, dim=-1).mean(1))

    def forward(self, x: Tensor) -> Tensor:
        flat = x.reshape(-1, x.shape[-1])
        chosen = self.router(flat).topk(self.top_k, dim=-1).indices                 # (N, k)
        keep = torch.zeros(flat.shape[0], self.num_experts, dtype=flat.dtype, device=flat.device)
        keep.scatter_(1, chosen, 1.0)
        hidden = self.activation(torch.einsum("nd,ehd->neh", flat, self.w_gate)) \
            * torch.einsum("nd,ehd->neh", flat, self.w_up)
        out = torch.einsum("neh,edh->ned", hidden, self.w_down)
        return (out * keep[..., None]).sum(1).view_as(x)


def decompose_gated_mlp(mlp: nn.Module, num_experts: int, top_k: int) -> DecomposedMoE:
    """``mlp`` has ``gate``, ``up`` (``dim -> hidden``) and ``down`` (``hidden -> dim``) linears
    without biases (the package's SwiGLU / GLU layers)."""
    gate, up, down = mlp.gate.weight.detach(), mlp.up.weight.detach(), mlp.down.weight.detach()
    labels = balanced_kmeans(F.normalize(gate.float(), dim=1), num_experts)
    return DecomposedMoE(gate, up, down, labels, num_experts, top_k)
