"""``SoapTP``: a ``torch.optim.Optimizer`` around :func:`soap_tp_b200.soap_step`.

The reference stops at the per-parameter kernel and leaves the integration to the caller; its
README sketches the loop (``README.md:43-60``): call ``soap_step`` for every tensor-parallel 2-D
weight in the same order on every rank, then apply learning rate and weight decay yourself
(``src/soap_tp/soap.py:149-151``).  This class is that loop:

* 2-D parameters carrying ``tp_shard_dim`` (0: row shards, e.g. a column-parallel ``nn.Linear``
  weight ``[out/W, in]``; 1: column shards, e.g. a row-parallel weight ``[out, in/W]``) and
  ``tp_global_shape`` run SOAP-TP; ``state[p]`` IS the mapping handed to ``soap_step``, so it holds
  exactly the reference's keys (``left_preconditioner`` ... ``variance``, ``step``);
* replicated 2-D parameters are sharded on the fly (each rank preconditions a slice of the
  gradient, the update shards are all-gathered);
* a tensor-parallel matrix whose SHARDED side exceeds ``max_precond_dim`` (vocabulary-sized embeddings and
  heads) is preconditioned on its other side only, with the identity as the long side's basis, as original SOAP
  does (``tests/reference/soap.py:363-367`` of the reference); on CUDA that one-sided update is local to a rank
  apart from one all-reduce (``engine/one_sided.py``);
* everything else (1-D parameters, other matrices with a side above ``max_precond_dim`` or with no side
  divisible by the world size) gets AdamW;
* decoupled weight decay and the learning rate are applied here.

``state_dict()`` adds a layout header per SOAP parameter (global shape, shard dimension, block
size, grid) because packed block-cyclic buffers are only meaningful for the grid they were written
on; ``load_state_dict()`` checks it and restores fp32 column-major buffers bit-exactly.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from .layout import allocate_2d_block_cyclic, most_square_grid
from .step import soap_step, state_shapes


class SoapTP(torch.optim.Optimizer):
    def __init__(
        self,
        params: Iterable,
        lr: float = 3e-3,
        betas: Tuple[float, float] = (0.95, 0.95),
        shampoo_beta: float = 0.95,
        eps: float = 1e-8,
        weight_decay: float = 0.01,
        precondition_frequency: int = 10,
        block_size: int = 128,
        process_grid_shape: Optional[Tuple[int, int]] = None,
        basis_implementation: str = "householder",
        max_precond_dim: int = 16384,
        adamw_betas: Tuple[float, float] = (0.9, 0.95),
    ) -> None:
        if lr < 0.0:
            raise ValueError(f"invalid learning rate {lr}")
        if precondition_frequency <= 0:
            raise ValueError("precondition_frequency must be positive.")
        defaults = dict(lr=lr, betas=betas, shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                        precondition_frequency=precondition_frequency, block_size=block_size,
                        basis_implementation=basis_implementation, max_precond_dim=max_precond_dim,
                        adamw_betas=adamw_betas)
        super().__init__(params, defaults)
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.grid = tuple(process_grid_shape) if process_grid_shape is not None else most_square_grid(world)
        if self.grid[0] * self.grid[1] != world:
            raise ValueError(f"process_grid_shape={self.grid} does not match world_size={world}.")

    # ---- classification -------------------------------------------------------------------------
    def _plan(self, p: Tensor, group: dict) -> Optional[dict]:
        """How ``p`` is preconditioned: ``None`` (AdamW) or the ``soap_step`` layout arguments."""
        if p.ndim != 2:
            return None
        world = dist.get_world_size() if dist.is_initialized() else 1
        shard_dim = getattr(p, "tp_shard_dim", None)
        if shard_dim is not None:
            global_shape = tuple(getattr(p, "tp_global_shape"))
            plan = dict(global_shape=global_shape, shard_dim=int(shard_dim), replicated=False)
        else:
            rows, cols = p.shape
            if rows % world == 0:
                plan = dict(global_shape=(rows, cols), shard_dim=0, replicated=True)
            elif cols % world == 0:
                plan = dict(global_shape=(rows, cols), shard_dim=1, replicated=True)
            else:
                return None
        limit = group["max_precond_dim"]
        if max(plan["global_shape"]) > limit:
            long_side = 0 if plan["global_shape"][0] > limit else 1
            short_fits = plan["global_shape"][1 - long_side] <= limit
            if (p.is_cuda and not plan["replicated"] and long_side == plan["shard_dim"] and short_fits):
                plan["one_sided"] = True       # the sharded side keeps the identity basis
                return plan
            return None
        return plan

    # ---- the step ---------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialized first.")
        world, rank = dist.get_world_size(), dist.get_rank()
        for group in self.param_groups:
            lr, wd = group["lr"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                plan = self._plan(p, group)
                if plan is None:
                    self._adamw(p, group)
                    continue
                state = self.state[p]
                gradient = p.grad
                if plan.get("one_sided"):
                    from .engine import one_sided

                    # the engine works on row shards; a column-sharded long side is the same problem transposed
                    rows_sharded = plan["shard_dim"] == 0
                    update = one_sided.step(
                        gradient if rows_sharded else gradient.T, state, beta=group["shampoo_beta"],
                        beta1=group["betas"][0], beta2=group["betas"][1], eps=group["eps"],
                        interval=group["precondition_frequency"], implementation=group["basis_implementation"])
                    if not rows_sharded:
                        update = update.T
                    if wd != 0.0:
                        p.mul_(1.0 - lr * wd)
                    p.add_(update.to(p.dtype), alpha=-lr)
                    continue
                if plan["replicated"] and world > 1:
                    gradient = gradient.chunk(world, dim=plan["shard_dim"])[rank].contiguous()
                update = soap_step(
                    gradient, state, global_shape=plan["global_shape"], shard_dim=plan["shard_dim"],
                    block_size=group["block_size"], process_grid_shape=self.grid,
                    preconditioner_beta=group["shampoo_beta"], beta1=group["betas"][0], beta2=group["betas"][1],
                    eps=group["eps"], basis_refresh_interval=group["precondition_frequency"],
                    basis_implementation=group["basis_implementation"],
                )
                if plan["replicated"] and world > 1:
                    parts = [torch.empty_like(update) for _ in range(world)]
                    dist.all_gather(parts, update.contiguous())
                    update = torch.cat(parts, dim=plan["shard_dim"])
                if wd != 0.0:
                    p.mul_(1.0 - lr * wd)
                p.add_(update.to(p.dtype), alpha=-lr)
        return loss

    def _adamw(self, p: Tensor, group: dict) -> None:
        state = self.state[p]
        if "exp_avg" not in state:
            state["step"] = 0
            state["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        state["step"] += 1
        beta1, beta2 = group["adamw_betas"]
        grad = p.grad.float()
        state["exp_avg"].lerp_(grad, 1.0 - beta1)
        state["exp_avg_sq"].mul_(beta2).addcmul_(grad, grad, value=1.0 - beta2)
        bias1 = 1.0 - beta1 ** state["step"]
        bias2 = 1.0 - beta2 ** state["step"]
        denominator = (state["exp_avg_sq"] / bias2).sqrt_().add_(group["eps"])
        if group["weight_decay"] != 0.0:
            p.mul_(1.0 - group["lr"] * group["weight_decay"])
        p.add_((state["exp_avg"] / bias1 / denominator).to(p.dtype), alpha=-group["lr"])

    # ---- checkpointing ------------------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        result = super().state_dict()
        layouts = {}
        index = 0
        for group in self.param_groups:
            for p in group["params"]:
                plan = self._plan(p, group)
                if plan is not None and not plan.get("one_sided") and "left_basis" in self.state.get(p, {}):
                    layouts[index] = dict(global_shape=list(plan["global_shape"]), shard_dim=plan["shard_dim"],
                                          block_size=group["block_size"], grid=list(self.grid))
                index += 1
        result["soap_tp_layout"] = layouts
        return result

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        state_dict = dict(state_dict)
        layouts = state_dict.pop("soap_tp_layout", {})
        params = [p for group in self.param_groups for p in group["params"]]
        groups = [group for group in self.param_groups for _ in group["params"]]
        saved_state = state_dict["state"]
        # AdamW-style entries go through the stock loader; packed SOAP buffers are restored by hand
        # because the stock loader would cast them to the parameter dtype and drop their strides.
        stock = {k: v for k, v in saved_state.items() if "right_basis" not in v}
        super().load_state_dict({"state": stock, "param_groups": state_dict["param_groups"]})
        for index, entry in saved_state.items():
            if "right_basis" not in entry:
                continue
            if "left_basis" not in entry:
                # one-sided state: fp32 buffers of this rank, restored with their strides
                p = params[int(index)]
                self.state[p] = {name: (value.to(device=p.device, dtype=torch.float32).clone(memory_format=torch.preserve_format)
                                        if torch.is_tensor(value) else value) for name, value in entry.items()}
                continue
            p, group = params[int(index)], groups[int(index)]
            plan = self._plan(p, group)
            layout = layouts.get(int(index), layouts.get(str(index)))
            if plan is None:
                raise ValueError(f"parameter {index} has SOAP state in the checkpoint but is not preconditioned here.")
            if layout is not None:
                expected = dict(global_shape=list(plan["global_shape"]), shard_dim=plan["shard_dim"],
                                block_size=group["block_size"], grid=list(self.grid))
                if {k: list(v) if isinstance(v, (list, tuple)) else v for k, v in layout.items()} != expected:
                    raise ValueError(f"checkpoint layout {layout} does not match the current layout {expected}; "
                                     "packed block-cyclic state is only valid for the grid it was written on.")
            restored: Dict[str, Any] = {}
            for name, shape in state_shapes(plan["global_shape"]).items():
                buffer = allocate_2d_block_cyclic(shape, group["block_size"], self.grid, device=p.device)
                source = entry[name]
                if tuple(source.shape) != tuple(buffer.shape):
                    raise ValueError(f"{name}: checkpoint shape {tuple(source.shape)} != {tuple(buffer.shape)}.")
                buffer.copy_(source.to(torch.float32))
                restored[name] = buffer
            restored["step"] = int(entry["step"])
            self.state[p] = restored
        self._drop_device_caches()

    @staticmethod
    def _drop_device_caches() -> None:
        """Operand planes of the bases are cached per buffer address and tensor version.  Freshly restored
        buffers can reuse the addresses (and version numbers) of the ones they replace, so the caches are
        emptied whenever state is loaded."""
        import sys

        local = sys.modules.get("soap_tp_b200.engine.local")
        if local is not None:
            local._CONTEXTS.clear()
        one_sided = sys.modules.get("soap_tp_b200.engine.one_sided")
        if one_sided is not None:
            one_sided._PLANES.clear()
        distributed = sys.modules.get("soap_tp_b200.engine.distributed")
        if distributed is not None:
            for engine in distributed._ENGINES.values():
                engine._basis_cache.clear()


__all__ = ["SoapTP"]
