"""Optimizers: AdamW, Muon (Polar-Express Newton-Schulz), and their hyperspherical variants.

Recipes and group metadata follow the reference (ohara/optimizer.py:15-795) so schedules, resume
and checkpoints interchange: ``build_adamw``, ``build_muon_adamw``, ``build_adamh``,
``build_muonh_adamh`` and the ``MuonAdamW`` class with per-group ``kind`` / ``hypersphere`` /
``name`` / ``initial_lr`` / ``lr_scale``.

On CUDA devices the heavy parts run on this package's kernels: AdamW is one fused pass per tensor
that also refreshes the bf16 compute copy of the weight, and each Newton-Schulz iteration is three
batched tcgen05 GEMMs with the ``b·G + c·G²`` and ``a·X + X·C`` combinations fused into the GEMM
epilogues. CPU tensors take the fp32 PyTorch path, which is the oracle for the kernels.
"""

from __future__ import annotations

import math
from collections import defaultdict
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor, optim

# Five-step Polar Express coefficients (a, b, c): X <- a X + (b A + c A^2) X with A = X X^T.
POLAR_EXPRESS_COEFFICIENTS = (
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
)


# --------------------------------------------------------------------------------------------------
# AdamW builders
# --------------------------------------------------------------------------------------------------
class FusedAdamW(optim.AdamW):
    """``torch.optim.AdamW`` whose step runs the fused sm_100a kernel for fp32 CUDA parameters
    (identical update rule; other tensors fall back to the stock implementation)."""

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        leftovers = []
        for group in self.param_groups:
            if group.get("amsgrad") or group.get("maximize"):
                leftovers.append(group)
                continue
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not _fused_adamw_ok(p):
                    _adamw_reference_step(p, group, state, tensor_step=True)
                    continue
                if not state:
                    state["step"] = torch.zeros((), dtype=torch.float32)
                    state["exp_avg"] = torch.zeros_like(p)
                    state["exp_avg_sq"] = torch.zeros_like(p)
                state["step"] += 1
                _fused_adamw(p, state, float(group["lr"]), beta1, beta2, float(group["eps"]),
                             float(group["weight_decay"]), int(state["step"]))
        for group in leftovers:
            raise RuntimeError("FusedAdamW does not support amsgrad / maximize")
        return loss


def _fused_adamw_ok(p: Tensor) -> bool:
    return (
        p.is_cuda
        and p.dtype == torch.float32
        and p.is_contiguous()
        and p.grad is not None
        and p.grad.is_contiguous()
        and p.grad.dtype in (torch.float32, torch.bfloat16)
    )


def _fused_adamw(p: Tensor, state: dict, lr: float, beta1: float, beta2: float, eps: float,
                 weight_decay: float, step: int) -> None:
    from ohara_b200.ops import refresh_bf16_weight
    from ohara_b200.ops._ext import ext

    shadow = None
    cached = getattr(p, "_ohara_bf16", None)
    if cached is not None and cached[1].shape == p.shape and cached[1].device == p.device:
        shadow = cached[1]
    ext().adamw_step(p, p.grad, state["exp_avg"], state["exp_avg_sq"], shadow, lr, beta1, beta2,
                     eps, weight_decay, step, 1.0)
    if shadow is not None:
        refresh_bf16_weight(p, shadow)


def _adamw_reference_step(p: Tensor, group: dict, state: dict, tensor_step: bool = False) -> None:
    """Decoupled-decay Adam with bias correction and eps added after the square root."""
    grad = p.grad
    if grad.is_sparse:
        raise RuntimeError("MuonAdamW does not support sparse gradients")
    if not state:
        state["step"] = torch.zeros((), dtype=torch.float32) if tensor_step else 0
        state["exp_avg"] = torch.zeros_like(p)
        state["exp_avg_sq"] = torch.zeros_like(p)
    state["step"] += 1
    step = int(state["step"])
    beta1, beta2 = group["betas"]
    lr = float(group["lr"])
    p.mul_(1.0 - lr * float(group["weight_decay"]))
    state["exp_avg"].lerp_(grad.to(p.dtype), 1.0 - beta1)
    state["exp_avg_sq"].lerp_(grad.to(p.dtype).square(), 1.0 - beta2)
    denom = (state["exp_avg_sq"] / (1.0 - beta2**step)).sqrt().add_(group["eps"])
    p.addcdiv_(state["exp_avg"], denom, value=-lr / (1.0 - beta1**step))


def build_adamw(model: torch.nn.Module, *, learning_rate: float, weight_decay: float,
                betas: tuple[float, float] = (0.9, 0.95)) -> optim.AdamW:
    """AdamW with decay on matrices (``ndim >= 2``) and none on norm gains / biases."""
    if learning_rate <= 0:
        raise ValueError("learning_rate must be positive")
    if weight_decay < 0:
        raise ValueError("weight_decay cannot be negative")
    decay, no_decay = [], []
    for p in model.parameters():
        if p.requires_grad:
            (decay if p.ndim >= 2 else no_decay).append(p)
    if not decay:
        raise ValueError("model has no trainable matrix parameters")
    return FusedAdamW(
        [{"params": decay, "weight_decay": weight_decay},
         {"params": no_decay, "weight_decay": 0.0}],
        lr=learning_rate, betas=betas,
    )


# --------------------------------------------------------------------------------------------------
# Hyperspherical (constant-norm) updates
# --------------------------------------------------------------------------------------------------
def _whole_norms(tensors: list[Tensor], sharded: list[bool] | None, group) -> list[Tensor]:
    """Frobenius norms of ``tensors``; where ``sharded[i]`` the tensor is one shard of a matrix
    spread over ``group`` and the norm is that of the whole matrix (squared norms summed over the
    group, one all-reduce for all of them)."""
    norms = list(torch._foreach_norm(tensors))
    if not sharded or not any(sharded):  # (``group=None`` is the default process group)
        return norms
    import torch.distributed as dist

    picked = [i for i, flag in enumerate(sharded) if flag]
    squares = torch.stack([norms[i].float().square() for i in picked])
    dist.all_reduce(squares, group=group)
    for slot, i in enumerate(picked):
        norms[i] = squares[slot].sqrt().to(norms[i].dtype)
    return norms


def _hypersphere_update_(params: list[Tensor], directions: list[Tensor], learning_rate: float, *,
                         eps: float = 1e-10, sharded: list[bool] | None = None,
                         group=None) -> None:
    """``p <- p - lr·u·‖p‖/‖u‖`` then rescale back to the original Frobenius norm, per tensor.
    With ``group`` and ``sharded`` the flagged tensors are tensor-parallel shards and every norm
    is taken over the whole matrix."""
    if not params:
        return
    p_norms = _whole_norms(params, sharded, group)
    u_norms = torch._foreach_clamp_min(_whole_norms(directions, sharded, group), eps)
    steps = torch._foreach_div(p_norms, u_norms)
    torch._foreach_mul_(steps, learning_rate)
    torch._foreach_add_(params, torch._foreach_mul(directions, steps), alpha=-1)
    new_norms = torch._foreach_clamp_min(_whole_norms(params, sharded, group), eps)
    torch._foreach_mul_(params, torch._foreach_div(p_norms, new_norms))


def _stacked_norms(stacked: Tensor, group) -> Tensor:
    """Norms of whole matrices from a stack of their shards (sum of squares over ``group``)."""
    import torch.distributed as dist

    squares = stacked.float().square().sum(dim=(-2, -1), keepdim=True)
    dist.all_reduce(squares, group=group)
    return squares.sqrt().to(stacked.dtype)


def _hypersphere_update_stacked_(stacked: Tensor, updates: Tensor, learning_rate: float, *,
                                 eps: float = 1e-10, sharded: bool = False, group=None) -> None:
    """Same rule for a ``(batch, rows, cols)`` stack, one norm per matrix; with ``sharded`` the
    stack holds tensor-parallel shards and the norms are those of the whole matrices, summed
    over ``group`` (``None``: the default process group)."""
    if sharded:
        p_norms = _stacked_norms(stacked, group)
        u_norms = _stacked_norms(updates, group).clamp_min(eps)
    else:
        p_norms = torch.linalg.matrix_norm(stacked, keepdim=True)
        u_norms = torch.linalg.matrix_norm(updates, keepdim=True).clamp_min(eps)
    stacked.sub_(updates * (p_norms * learning_rate / u_norms))
    if sharded:
        new_norms = _stacked_norms(stacked, group).clamp_min(eps)
    else:
        new_norms = torch.linalg.matrix_norm(stacked, keepdim=True).clamp_min(eps)
    stacked.mul_(p_norms / new_norms)


# --------------------------------------------------------------------------------------------------
# Newton-Schulz (Polar Express)
# --------------------------------------------------------------------------------------------------
def _fused_muon_ok(params: list[Tensor], rows: int, cols: int) -> bool:
    """Fused Muon stages: fp32 CUDA parameters and gradients, contiguous and 16-byte aligned,
    tile-friendly sizes, at most 128 tensors in the group."""
    if not params or len(params) > 128 or rows % 8 or cols % 8:
        return False
    for p in params:
        g = p.grad
        if not (p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and g is not None
                and g.dtype == torch.float32 and g.is_contiguous() and g.shape == p.shape
                and p.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0):
            return False
    return True


def _polar_express_kernels(x: Tensor, steps: int) -> Tensor:
    """bf16 iteration on the tcgen05 GEMM. ``x`` is a contiguous (B, r, c) bf16 stack, already
    normalised. Gram on the short side; the symmetric products need no explicit transposes."""
    from ohara_b200.ops._ext import ext

    C = ext()
    b, r, c = x.shape
    tall = r > c
    side = c if tall else r
    gram = torch.empty(b, side, side, device=x.device, dtype=torch.bfloat16)
    corr = torch.empty_like(gram)
    nxt = torch.empty_like(x)
    for ca, cb, cc in POLAR_EXPRESS_COEFFICIENTS[:steps]:
        if tall:
            # A = X^T X: both operands stored (K=r rows, c contiguous) -> MN-major.
            C.gemm(x, x, gram, side, side, r, True, True)
        else:
            # A = X X^T: both operands K-major.
            C.gemm(x, x, gram, side, side, c, False, False)
        # corr = cb*A + cc*A@A  (A symmetric, so A @ A^T = A^2 with K-major operands)
        C.gemm(gram, gram, corr, side, side, side, False, False, alpha=cc, residual=gram, beta=cb)
        if tall:
            # X <- ca*X + X @ corr : B = corr stored (K, N) -> MN-major
            C.gemm(x, corr, nxt, r, c, c, False, True, residual=x, beta=ca)
        else:
            # X <- ca*X + corr @ X : B = X stored (K=r, N=c) -> MN-major
            C.gemm(corr, x, nxt, r, c, r, False, True, residual=x, beta=ca)
        x, nxt = nxt, x
    return x


def _polar_express(matrix: Tensor, steps: int) -> Tensor:
    """Approximate polar factor (orthogonalisation) of every matrix in a ``(B, r, c)`` stack."""
    if matrix.ndim != 3:
        raise ValueError("Muon expects a stack of two-dimensional gradients")
    if not 1 <= steps <= len(POLAR_EXPRESS_COEFFICIENTS):
        raise ValueError("ns_steps must be between 1 and 5")
    on_gpu = matrix.device.type == "cuda" and matrix.dtype != torch.float64
    x = matrix.to(torch.bfloat16) if on_gpu else matrix.float()
    norm = x.float().norm(dim=(-2, -1), keepdim=True)
    x = x / (norm.to(x.dtype) * 1.01 + 1e-6)
    r, c = matrix.shape[-2:]
    if on_gpu and r % 8 == 0 and c % 8 == 0:
        return _polar_express_kernels(x.contiguous(), steps)
    if r > c:
        for ca, cb, cc in POLAR_EXPRESS_COEFFICIENTS[:steps]:
            gram = x.mT @ x
            x = ca * x + x @ (cb * gram + cc * (gram @ gram))
    else:
        for ca, cb, cc in POLAR_EXPRESS_COEFFICIENTS[:steps]:
            gram = x @ x.mT
            x = ca * x + (cb * gram + cc * (gram @ gram)) @ x
    return x


# --------------------------------------------------------------------------------------------------
# The hybrid optimizer
# --------------------------------------------------------------------------------------------------
class MuonAdamW(optim.Optimizer):
    """One optimizer, per-group algorithm: ``kind="adamw"`` or ``kind="muon"``, each optionally
    ``hypersphere=True`` (AdamH / MuonH: constant-norm steps, ``lr`` is a relative step size and
    ``weight_decay`` must be 0). Muon groups hold same-shaped 2-D parameters or one pre-stacked
    3-D (experts, rows, cols) parameter."""

    def __init__(self, param_groups: list[dict[str, Any]]):
        if not param_groups:
            raise ValueError("param_groups cannot be empty")
        for group in param_groups:
            self._validate_group(group)
        super().__init__(param_groups, defaults={})

    @staticmethod
    def _validate_group(group: dict[str, Any]) -> None:
        kind = group.get("kind")
        if kind not in {"adamw", "muon"}:
            raise ValueError(f"unknown optimizer kind: {kind!r}")
        if float(group.get("lr", 0.0)) <= 0:
            raise ValueError("every optimizer group needs a positive lr")
        if float(group.get("weight_decay", 0.0)) < 0:
            raise ValueError("weight_decay cannot be negative")
        params = list(group.get("params", ()))
        if group.get("hypersphere", False):
            if float(group.get("weight_decay", 0.0)) != 0.0:
                raise ValueError(
                    "hyperspherical groups must use weight_decay=0: renormalizing the parameter "
                    "cancels decay to first order. Fold it into the learning rate instead "
                    "(lr = sqrt(lr * weight_decay) of the additive recipe)."
                )
            if any(p.ndim < 2 for p in params):
                raise ValueError(
                    "hyperspherical groups hold matrix parameters only; keep vectors such as "
                    "norm gains and biases in a plain AdamW group"
                )
        if kind == "muon":
            if not params:
                raise ValueError("Muon groups must contain matrix parameters")
            pre_stacked = len(params) == 1 and params[0].ndim == 3
            if not pre_stacked:
                if any(p.ndim != 2 for p in params):
                    raise ValueError(
                        "Muon groups must contain two-dimensional parameters, or a single "
                        "pre-stacked three-dimensional parameter"
                    )
                if any(p.shape != params[0].shape for p in params):
                    raise ValueError("parameters in a Muon group must have identical shapes")
            momentum = float(group.get("momentum", 0.95))
            beta2 = float(group.get("beta2", 0.9))
            if not 0 <= momentum < 1 or not 0 <= beta2 < 1:
                raise ValueError("Muon momentum and beta2 must be in [0, 1)")
            if not 1 <= int(group.get("ns_steps", 5)) <= len(POLAR_EXPRESS_COEFFICIENTS):
                raise ValueError("ns_steps must be between 1 and 5")

    # -- AdamW / AdamH -----------------------------------------------------------------------
    @staticmethod
    def _adamw_step(parameter: Tensor, group: dict[str, Any], state: dict[str, Any]) -> None:
        if parameter.grad is None:
            return
        if parameter.grad.is_sparse:
            raise RuntimeError("MuonAdamW does not support sparse gradients")
        if _fused_adamw_ok(parameter):
            if not state:
                state["step"] = 0
                state["exp_avg"] = torch.zeros_like(parameter)
                state["exp_avg_sq"] = torch.zeros_like(parameter)
            state["step"] += 1
            beta1, beta2 = group["betas"]
            _fused_adamw(parameter, state, float(group["lr"]), beta1, beta2, float(group["eps"]),
                         float(group["weight_decay"]), int(state["step"]))
            return
        _adamw_reference_step(parameter, group, state)

    def _adamh_step(self, group: dict[str, Any]) -> None:
        params = [p for p in group["params"] if p.grad is not None]
        if not params:
            return
        grads = [p.grad for p in params]
        if any(g.is_sparse for g in grads):
            raise RuntimeError("MuonAdamW does not support sparse gradients")
        states = [self.state[p] for p in params]
        for p, state in zip(params, states, strict=True):
            if not state:
                state["step"] = 0
                state["exp_avg"] = torch.zeros_like(p)
                state["exp_avg_sq"] = torch.zeros_like(p)
            state["step"] += 1
        beta1, beta2 = group["betas"]
        eps = float(group["eps"])
        step = states[0]["step"]
        exp_avgs = [s["exp_avg"] for s in states]
        exp_avg_sqs = [s["exp_avg_sq"] for s in states]
        torch._foreach_lerp_(exp_avgs, grads, 1.0 - beta1)
        torch._foreach_lerp_(exp_avg_sqs, torch._foreach_mul(grads, grads), 1.0 - beta2)
        denoms = torch._foreach_sqrt(torch._foreach_div(exp_avg_sqs, 1.0 - beta2**step))
        torch._foreach_add_(denoms, eps)
        directions = torch._foreach_div(torch._foreach_div(exp_avgs, 1.0 - beta1**step), denoms)
        # tensor-parallel shards: the sphere is that of the whole matrix
        distributed = self._tensor_parallel_world() > 1
        sharded = [distributed and hasattr(p, "tensor_parallel_dim") for p in params]
        if len(params) == 1 and params[0].ndim == 3:
            _hypersphere_update_stacked_(params[0], directions[0], float(group["lr"]),
                                         sharded=sharded[0], group=self.tensor_parallel_group)
        else:
            _hypersphere_update_(params, directions, float(group["lr"]), sharded=sharded,
                                 group=self.tensor_parallel_group)

    # -- Muon / MuonH ------------------------------------------------------------------------
    def _muon_step(self, group: dict[str, Any]) -> None:
        params: list[Tensor] = group["params"]
        active = [p for p in params if p.grad is not None]
        if not active:
            return
        if len(active) != len(params):
            raise RuntimeError(
                "a Muon group has missing gradients; all same-shaped matrix parameters "
                "must participate in each optimization step"
            )
        if any(p.grad.is_sparse for p in active):
            raise RuntimeError("MuonAdamW does not support sparse gradients")
        first = params[0]
        pre_stacked = len(params) == 1 and first.ndim == 3
        rows, cols = first.shape[-2:]
        batch = first.size(0) if pre_stacked else len(params)
        state = self.state[first]
        if "momentum_buffer" not in state:
            state["momentum_buffer"] = torch.zeros(batch, rows, cols, dtype=first.dtype,
                                                   device=first.device)
        hyperspherical = bool(group.get("hypersphere", False))
        reduce_dim = -1 if rows >= cols else -2
        if not hyperspherical and "second_momentum_buffer" not in state:
            shape = (batch, rows, 1) if reduce_dim == -1 else (batch, 1, cols)
            state["second_momentum_buffer"] = torch.zeros(shape, dtype=first.dtype,
                                                          device=first.device)
        tp_dim = getattr(first, "tensor_parallel_dim", None)
        if tp_dim is not None and self._tensor_parallel_world() > 1:
            self._muon_step_tensor_parallel(group, state, params, int(tp_dim))
            return
        if not hyperspherical and _fused_muon_ok(params, rows, cols):
            self._muon_step_fused(group, state, params, batch, rows, cols)
            return
        if pre_stacked:
            grads = first.grad
            stacked = first.detach()
        else:
            grads = torch.stack([p.grad for p in params])
            stacked = torch.stack([p.detach() for p in params])
        grads = grads.to(first.dtype)

        momentum = float(group["momentum"])
        buf = state["momentum_buffer"]
        buf.lerp_(grads, 1.0 - momentum)
        update = _polar_express(grads.lerp(buf, momentum), int(group["ns_steps"]))

        if hyperspherical:
            _hypersphere_update_stacked_(stacked, update.to(stacked.dtype), float(group["lr"]))
        else:
            second = state["second_momentum_buffer"]
            beta2 = float(group["beta2"])
            variance = update.float().square().mean(dim=reduce_dim, keepdim=True)
            size = update.size(reduce_dim)
            norm_before = (variance.sum(dim=(-2, -1), keepdim=True) * size).sqrt()
            second.lerp_(variance.to(second.dtype), 1.0 - beta2)
            inv_rms = second.clamp_min(1e-10).rsqrt()
            norm_after = ((variance * size) * inv_rms.float().square()).sum(
                dim=(-2, -1), keepdim=True).sqrt()
            update = update * (inv_rms * (norm_before / norm_after.clamp_min(1e-10))).to(update.dtype)
            lr = float(group["lr"]) * math.sqrt(max(1.0, rows / cols))
            wd = float(group["weight_decay"])
            update = update.to(stacked.dtype)
            aligned = (update * stacked) >= 0  # cautious decay: only where the step agrees
            stacked.sub_(lr * update + lr * wd * stacked * aligned)
        if not pre_stacked:
            torch._foreach_copy_(params, list(stacked.unbind(0)))

    # -- Muon on tensor-parallel shards ------------------------------------------------------------
    # Set by the engine (``OharaEngine.prepare_optimizers``): the process group over which the
    # matrices of this optimizer are sharded. Kept off the param groups so that state dicts stay
    # plain data.
    tensor_parallel_group = None
    tensor_parallel_world = 1

    def _tensor_parallel_world(self) -> int:
        return int(getattr(self, "tensor_parallel_world", 1) or 1)

    def _muon_step_tensor_parallel(self, group: dict[str, Any], state: dict[str, Any],
                                   params: list[Tensor], tp_dim: int) -> None:
        """The Muon step when every matrix of the group is a shard (rows for ``tp_dim`` 0, columns
        for 1) of a matrix spread over a tensor-parallel group. The orthogonalisation of a shard
        is not the shard of the orthogonalised matrix, so the momentum-corrected gradients are
        gathered over the group, the Newton-Schulz iteration and the row / column statistics run
        on the whole matrices (redundantly on every rank of the group: a few small GEMMs), and
        each rank applies its own slice. Momentum stays sharded; the factored second moment is a
        vector over whole rows or columns and is kept in full on every rank. Identical, up to
        summation order, to the step on the unsharded matrices. (The reference rejects this
        combination: examples/train_llama_engine.py:280-281.)"""
        import torch.distributed as dist

        hyperspherical = bool(group.get("hypersphere", False))
        world, pg = self._tensor_parallel_world(), self.tensor_parallel_group
        rank = dist.get_rank(pg)
        first = params[0]
        pre_stacked = len(params) == 1 and first.ndim == 3
        grads = first.grad if pre_stacked else torch.stack([p.grad for p in params])
        stacked = first.detach() if pre_stacked else torch.stack([p.detach() for p in params])
        grads = grads.to(first.dtype)
        momentum = float(group["momentum"])
        buf = state["momentum_buffer"]
        buf.lerp_(grads, 1.0 - momentum)
        local = grads.lerp(buf, momentum).contiguous()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local, group=pg)
        whole = torch.cat(parts, dim=1 + tp_dim)
        update = _polar_express(whole, int(group["ns_steps"]))
        if hyperspherical:
            # MuonH: a constant-norm step along the orthogonalised direction; every norm is that
            # of the whole matrix, so the shards stay on the whole matrix's sphere
            mine = update.chunk(world, dim=1 + tp_dim)[rank].to(stacked.dtype).contiguous()
            _hypersphere_update_stacked_(stacked, mine, float(group["lr"]), sharded=True, group=pg)
            if not pre_stacked:
                torch._foreach_copy_(params, list(stacked.unbind(0)))
            for p in params:
                if getattr(p, "_ohara_bf16", None) is not None:
                    p._ohara_bf16 = None
            return
        rows, cols = whole.shape[-2:]
        reduce_dim = -1 if rows >= cols else -2
        shape = (whole.shape[0], rows, 1) if reduce_dim == -1 else (whole.shape[0], 1, cols)
        second = state.get("second_momentum_buffer")
        if second is None or tuple(second.shape) != shape:
            second = state["second_momentum_buffer"] = torch.zeros(shape, dtype=first.dtype,
                                                                   device=first.device)
        beta2 = float(group["beta2"])
        variance = update.float().square().mean(dim=reduce_dim, keepdim=True)
        size = update.size(reduce_dim)
        norm_before = (variance.sum(dim=(-2, -1), keepdim=True) * size).sqrt()
        second.lerp_(variance.to(second.dtype), 1.0 - beta2)
        inv_rms = second.clamp_min(1e-10).rsqrt()
        norm_after = ((variance * size) * inv_rms.float().square()).sum(
            dim=(-2, -1), keepdim=True).sqrt()
        update = update * (inv_rms * (norm_before / norm_after.clamp_min(1e-10))).to(update.dtype)
        lr = float(group["lr"]) * math.sqrt(max(1.0, rows / cols))
        wd = float(group["weight_decay"])
        mine = update.chunk(world, dim=1 + tp_dim)[rank].to(stacked.dtype)
        aligned = (mine * stacked) >= 0
        stacked.sub_(lr * mine + lr * wd * stacked * aligned)
        if not pre_stacked:
            torch._foreach_copy_(params, list(stacked.unbind(0)))
        for p in params:  # written without a version bump on the compute copies
            if getattr(p, "_ohara_bf16", None) is not None:
                p._ohara_bf16 = None

    @staticmethod
    def _muon_step_fused(group: dict[str, Any], state: dict[str, Any], params: list[Tensor],
                         batch: int, rows: int, cols: int) -> None:
        """The same step on the kernels of ``csrc/muon.cu``: gradients and parameters are read
        and written in place through pointer tables (no stacking, no copy back), the element-wise
        work is three passes instead of about twenty."""
        from ohara_b200.ops import refresh_bf16_weight
        from ohara_b200.ops._ext import ext

        C = ext()
        device = params[0].device
        momentum = float(group["momentum"])
        u = torch.empty(batch, rows, cols, device=device, dtype=torch.bfloat16)
        norm2 = torch.empty(batch, device=device, dtype=torch.float32)
        C.muon_prepare([p.grad for p in params], state["momentum_buffer"], u, norm2, momentum)
        update = _polar_express_kernels(u, int(group["ns_steps"]))
        by_row = rows >= cols
        variance = C.muon_variance(update, by_row)  # (B, r, 1) or (B, 1, c), fp32
        size = cols if by_row else rows
        second = state["second_momentum_buffer"]
        norm_before = (variance.sum(dim=(-2, -1), keepdim=True) * size).sqrt()
        second.lerp_(variance, 1.0 - float(group["beta2"]))
        inv_rms = second.clamp_min(1e-10).rsqrt()
        norm_after = ((variance * size) * inv_rms.square()).sum(dim=(-2, -1), keepdim=True).sqrt()
        factor = (inv_rms * (norm_before / norm_after.clamp_min(1e-10))).to(torch.bfloat16).float()
        lr = float(group["lr"]) * math.sqrt(max(1.0, rows / cols))
        shadows = []
        for p in params:
            cached = getattr(p, "_ohara_bf16", None)
            if cached is None or cached[1].shape != p.shape or cached[1].device != p.device \
                    or not cached[1].is_contiguous():
                shadows = []
                break
            shadows.append(cached[1])
        C.muon_apply([p.detach() for p in params], shadows, update, factor.contiguous(), lr,
                     float(group["weight_decay"]), by_row)
        if shadows:
            for p, shadow in zip(params, shadows):
                refresh_bf16_weight(p, shadow)
        else:
            # The kernel wrote through raw pointers (no version bump): drop any compute copy.
            for p in params:
                if getattr(p, "_ohara_bf16", None) is not None:
                    p._ohara_bf16 = None

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            if group["kind"] == "adamw":
                if group.get("hypersphere", False):
                    self._adamh_step(group)
                else:
                    for p in group["params"]:
                        self._adamw_step(p, group, self.state[p])
            elif group["kind"] == "muon":
                self._muon_step(group)
            else:
                raise ValueError(f"unknown optimizer kind: {group['kind']!r}")
        return loss


# --------------------------------------------------------------------------------------------------
# Parameter partition and recipes
# --------------------------------------------------------------------------------------------------
def _unwrap_model(model: torch.nn.Module) -> torch.nn.Module:
    while hasattr(model, "module") and isinstance(model.module, torch.nn.Module):
        model = model.module
    return model


@dataclass(frozen=True)
class _LlamaParameterGroups:
    embedding: list[torch.nn.Parameter]
    unembedding: list[torch.nn.Parameter]  # empty when tied to the embedding
    matrix: list[torch.nn.Parameter]  # 2-D hidden weights
    stacked_matrix: list[torch.nn.Parameter]  # 3-D (experts, in, out) tensors
    scalar: list[torch.nn.Parameter]  # norm gains, biases, anything else
    hidden_size: int


def _partition_llama_parameters(model: torch.nn.Module, caller: str) -> _LlamaParameterGroups:
    """Split a Llama-shaped model (``token_emb``, ``vocab_proj``, ``layers``, ``config``) by role.
    The partition is checked to be disjoint and complete. A pipeline stage of such a model
    (``pipeline_stage = True``) may lack the embedding or the output projection (``None``)."""
    root = _unwrap_model(model)
    if any(not hasattr(root, name) for name in ("token_emb", "vocab_proj", "layers", "config")):
        raise TypeError(f"{caller} expects an ohara Llama-compatible model")
    is_stage = bool(getattr(root, "pipeline_stage", False))

    def params_of(module):
        return [] if module is None else [p for p in module.parameters() if p.requires_grad]

    trainable = [p for p in root.parameters() if p.requires_grad]
    embedding = params_of(root.token_emb)
    taken = {id(p) for p in embedding}
    unembedding = [p for p in params_of(root.vocab_proj) if id(p) not in taken]
    taken |= {id(p) for p in unembedding}
    layer_params = [p for p in root.layers.parameters() if p.requires_grad and id(p) not in taken]
    matrix = [p for p in layer_params if p.ndim == 2]
    stacked = [p for p in layer_params if p.ndim == 3]
    matrix_ids = {id(p) for p in matrix} | {id(p) for p in stacked}
    scalar = [p for p in trainable if id(p) not in taken and id(p) not in matrix_ids]
    assigned = embedding + unembedding + matrix + stacked + scalar
    if len({id(p) for p in assigned}) != len(assigned):
        raise RuntimeError("optimizer parameter groups overlap")
    if {id(p) for p in assigned} != {id(p) for p in trainable}:
        raise RuntimeError("optimizer parameter partition is incomplete")
    if (not embedding and not is_stage) or not matrix:
        raise ValueError("model must have token embeddings and transformer matrices")
    return _LlamaParameterGroups(embedding, unembedding, matrix, stacked, scalar,
                                 int(root.config.hidden_size))


def _group_matrices_by_shape(params):
    buckets: defaultdict[torch.Size, list] = defaultdict(list)
    for p in params:
        buckets[p.shape].append(p)
    return [(shape, buckets[shape]) for shape in sorted(buckets, key=tuple)]


def _shape_tag(shape) -> str:
    return "x".join(str(s) for s in shape)


def build_muon_adamw(model: torch.nn.Module, *, matrix_learning_rate: float = 0.02,
                     embedding_learning_rate: float = 0.3,
                     unembedding_learning_rate: float = 0.008, scalar_learning_rate: float = 0.5,
                     weight_decay: float = 0.28, reference_hidden_size: int = 768,
                     momentum: float = 0.95, beta2: float = 0.9, ns_steps: int = 5) -> MuonAdamW:
    """nanochat-style hybrid: Muon on hidden matrices (one group per shape, one per expert stack),
    AdamW on lm_head / embedding / scalars with ``1/sqrt(d_model)`` width transfer on the AdamW
    rates."""
    rates = (matrix_learning_rate, embedding_learning_rate, unembedding_learning_rate,
             scalar_learning_rate)
    if any(v <= 0 for v in rates):
        raise ValueError("all learning rates must be positive")
    if weight_decay < 0:
        raise ValueError("weight_decay cannot be negative")
    if reference_hidden_size < 1:
        raise ValueError("reference_hidden_size must be positive")
    part = _partition_llama_parameters(model, "build_muon_adamw")
    width = math.sqrt(reference_hidden_size / part.hidden_size)
    groups: list[dict[str, Any]] = []

    def adamw(name, params, lr, betas, decay):
        if params:
            groups.append({"name": name, "kind": "adamw", "params": params, "lr": lr,
                           "initial_lr": lr, "lr_scale": lr / matrix_learning_rate,
                           "betas": betas, "eps": 1e-10, "weight_decay": decay})

    adamw("unembedding", part.unembedding, unembedding_learning_rate * width, (0.8, 0.96), 0.01)
    adamw("embedding", part.embedding, embedding_learning_rate * width, (0.8, 0.995), 0.001)
    adamw("norms_and_scalars", part.scalar, scalar_learning_rate * 0.01, (0.8, 0.95), 0.0)

    def muon(name, params):
        groups.append({"name": name, "kind": "muon", "params": params,
                       "lr": matrix_learning_rate, "initial_lr": matrix_learning_rate,
                       "lr_scale": 1.0, "weight_decay": weight_decay, "momentum": momentum,
                       "beta2": beta2, "ns_steps": ns_steps})

    for p in part.stacked_matrix:
        muon(f"expert_{_shape_tag(p.shape)}", [p])
    for shape, params in _group_matrices_by_shape(part.matrix):
        muon(f"matrix_{_shape_tag(shape)}", params)
    return MuonAdamW(groups)


def _hyper_group(name, kind, params, lr, **extra) -> dict[str, Any]:
    return {"name": name, "kind": kind, "hypersphere": True, "params": params, "lr": lr,
            "initial_lr": lr, "lr_scale": 1.0, "weight_decay": 0.0, **extra}


def _plain_adam_group(params, lr, base_lr, betas, eps) -> dict[str, Any]:
    return {"name": "embedding_and_scalars", "kind": "adamw", "params": params, "lr": lr,
            "initial_lr": lr, "lr_scale": lr / base_lr, "betas": betas, "eps": eps,
            "weight_decay": 0.0}


def build_adamh(model: torch.nn.Module, *, learning_rate: float = 0.007,
                adam_learning_rate: float = 6e-4, betas: tuple[float, float] = (0.9, 0.95),
                eps: float = 1e-8) -> MuonAdamW:
    """AdamH (https://arxiv.org/abs/2603.28743): constant-norm Adam on every matrix incl. the
    lm_head, plain AdamW (no decay) on embeddings and vectors. ``learning_rate`` is the relative
    step ``‖dW‖/‖W‖``; port an AdamW recipe with ``sqrt(lr * weight_decay)``."""
    if learning_rate <= 0 or adam_learning_rate <= 0:
        raise ValueError("all learning rates must be positive")
    part = _partition_llama_parameters(model, "build_adamh")
    groups = [
        _hyper_group(f"adamh_{_shape_tag(shape)}", "adamw", params, learning_rate, betas=betas, eps=eps)
        for shape, params in _group_matrices_by_shape(part.matrix + part.unembedding)
    ]
    groups += [
        _hyper_group(f"adamh_expert_{_shape_tag(p.shape)}", "adamw", [p], learning_rate,
                     betas=betas, eps=eps)
        for p in part.stacked_matrix
    ]
    rest = part.embedding + part.scalar
    if rest:
        groups.append(_plain_adam_group(rest, adam_learning_rate, learning_rate, betas, eps))
    return MuonAdamW(groups)


def build_muonh_adamh(model: torch.nn.Module, *, learning_rate: float = 0.075,
                      adam_learning_rate: float = 6e-4, momentum: float = 0.95, ns_steps: int = 5,
                      betas: tuple[float, float] = (0.9, 0.95), eps: float = 1e-8) -> MuonAdamW:
    """MuonH on hidden matrices, AdamH on the lm_head (same relative rate), AdamW on the rest."""
    if learning_rate <= 0 or adam_learning_rate <= 0:
        raise ValueError("all learning rates must be positive")
    part = _partition_llama_parameters(model, "build_muonh_adamh")
    muon_extra = {"momentum": momentum, "ns_steps": ns_steps, "beta2": 0.9}
    groups = [
        _hyper_group(f"muonh_{_shape_tag(shape)}", "muon", params, learning_rate, **muon_extra)
        for shape, params in _group_matrices_by_shape(part.matrix)
    ]
    groups += [
        _hyper_group(f"muonh_expert_{_shape_tag(p.shape)}", "muon", [p], learning_rate, **muon_extra)
        for p in part.stacked_matrix
    ]
    groups += [
        _hyper_group(f"adamh_unembedding_{_shape_tag(shape)}", "adamw", params, learning_rate,
                     betas=betas, eps=eps)
        for shape, params in _group_matrices_by_shape(part.unembedding)
    ]
    rest = part.embedding + part.scalar
    if rest:
        groups.append(_plain_adam_group(rest, adam_learning_rate, learning_rate, betas, eps))
    return MuonAdamW(groups)
