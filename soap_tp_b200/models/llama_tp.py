"""Llama-3-shaped decoder with Megatron-style tensor parallelism, for training with ``SoapTP``.

The reference contains no model (its README points at an external framework for the layers,
``README.md:68-69``); the benchmark configuration "TP=8 training of a Llama-3-8B-shaped decoder
with SOAP-TP on every 2-D weight" needs one, so this module provides it:

* ``ColumnParallelLinear`` stores ``weight[out / W, in]`` -> contiguous ROW shards of the logical
  matrix -> ``tp_shard_dim = 0``; ``RowParallelLinear`` stores ``weight[out, in / W]`` -> COLUMN
  shards -> ``tp_shard_dim = 1`` (the convention of ``README.md:82-83`` of the reference);
* attention heads are split over ranks (32 query / 8 key-value heads -> 4 / 1 per rank at W = 8),
  RoPE, causal ``scaled_dot_product_attention``;
* SwiGLU MLP (gate/up column-parallel, down row-parallel), RMSNorm, vocab-parallel embedding and
  vocab-parallel cross entropy (no rank ever holds full logits).

Every 2-D weight carries ``tp_shard_dim`` and ``tp_global_shape`` so the optimizer can hand it to
``soap_step`` unchanged.  Works on CPU (gloo) for tests and on CUDA (NCCL) for training.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.utils.checkpoint
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5
    max_seq_len: int = 4096

    @staticmethod
    def llama3_8b(**overrides) -> "LlamaConfig":
        return LlamaConfig(**overrides)

    @staticmethod
    def tiny(**overrides) -> "LlamaConfig":
        base = dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_layers=2, num_heads=4, num_kv_heads=2,
                    max_seq_len=16)
        base.update(overrides)
        return LlamaConfig(**base)


def _world() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


class _CopyToTensorParallel(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, grad):
        if _world() > 1:
            grad = grad.contiguous()
            dist.all_reduce(grad)
        return grad


class _ReduceFromTensorParallel(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, x):
        if _world() > 1:
            x = x.contiguous()
            dist.all_reduce(x)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad


def _tag(weight: nn.Parameter, shard_dim: int, global_shape) -> nn.Parameter:
    weight.tp_shard_dim = shard_dim
    weight.tp_global_shape = tuple(global_shape)
    return weight


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, *, dtype, device, std: float) -> None:
        super().__init__()
        world = _world()
        if out_features % world:
            raise ValueError(f"out_features={out_features} is not divisible by the world size {world}.")
        self.weight = nn.Parameter(torch.empty(out_features // world, in_features, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=std)
        _tag(self.weight, 0, (out_features, in_features))

    def forward(self, x: Tensor) -> Tensor:
        return F.linear(_CopyToTensorParallel.apply(x), self.weight)


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, *, dtype, device, std: float) -> None:
        super().__init__()
        world = _world()
        if in_features % world:
            raise ValueError(f"in_features={in_features} is not divisible by the world size {world}.")
        self.weight = nn.Parameter(torch.empty(out_features, in_features // world, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=std)
        _tag(self.weight, 1, (out_features, in_features))

    def forward(self, x: Tensor) -> Tensor:
        return _ReduceFromTensorParallel.apply(F.linear(x, self.weight))


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, *, dtype, device, std: float) -> None:
        super().__init__()
        world = _world()
        if vocab_size % world:
            raise ValueError(f"vocab_size={vocab_size} is not divisible by the world size {world}.")
        self.per_rank = vocab_size // world
        self.start = _rank() * self.per_rank
        self.weight = nn.Parameter(torch.empty(self.per_rank, hidden_size, dtype=dtype, device=device))
        nn.init.normal_(self.weight, std=std)
        _tag(self.weight, 0, (vocab_size, hidden_size))

    def forward(self, tokens: Tensor) -> Tensor:
        local = tokens - self.start
        mine = (local >= 0) & (local < self.per_rank)
        embedded = F.embedding(local.clamp(0, self.per_rank - 1), self.weight)
        embedded = embedded * mine.unsqueeze(-1).to(embedded.dtype)
        return _ReduceFromTensorParallel.apply(embedded)


class _VocabParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits: Tensor, targets: Tensor, start: int):
        logits = logits.float()
        local_max = logits.max(dim=-1).values
        if _world() > 1:
            dist.all_reduce(local_max, op=dist.ReduceOp.MAX)
        shifted = logits - local_max.unsqueeze(-1)
        exp = shifted.exp()
        denominator = exp.sum(dim=-1)
        per_rank = logits.shape[-1]
        local_target = targets - start
        mine = (local_target >= 0) & (local_target < per_rank)
        picked = shifted.gather(-1, local_target.clamp(0, per_rank - 1).unsqueeze(-1)).squeeze(-1) * mine
        if _world() > 1:
            dist.all_reduce(denominator)
            dist.all_reduce(picked)
        loss = denominator.log() - picked
        ctx.save_for_backward(exp / denominator.unsqueeze(-1), local_target.clamp(0, per_rank - 1), mine)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        softmax, local_target, mine = ctx.saved_tensors
        grad = softmax.clone()
        grad.scatter_add_(-1, local_target.unsqueeze(-1), -mine.unsqueeze(-1).to(grad.dtype))
        return grad * grad_loss.unsqueeze(-1), None, None


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float, *, dtype, device) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        normed = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        return (normed * self.weight.float()).to(x.dtype)


def rope_tables(head_dim: int, seq_len: int, theta: float, device) -> tuple[Tensor, Tensor]:
    frequencies = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    angles = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), frequencies)
    return angles.cos(), angles.sin()


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    # x: [batch, heads, seq, head_dim]
    x1, x2 = x.float().chunk(2, dim=-1)
    cos, sin = cos[None, None], sin[None, None]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig, *, dtype, device, std: float, out_std: float) -> None:
        super().__init__()
        world = _world()
        if cfg.num_heads % world or cfg.num_kv_heads % world:
            raise ValueError("attention heads and key-value heads must be divisible by the world size.")
        self.head_dim = cfg.hidden_size // cfg.num_heads
        self.local_heads = cfg.num_heads // world
        self.local_kv_heads = cfg.num_kv_heads // world
        kv_features = cfg.num_kv_heads * self.head_dim
        self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.hidden_size, dtype=dtype, device=device, std=std)
        self.k_proj = ColumnParallelLinear(cfg.hidden_size, kv_features, dtype=dtype, device=device, std=std)
        self.v_proj = ColumnParallelLinear(cfg.hidden_size, kv_features, dtype=dtype, device=device, std=std)
        self.o_proj = RowParallelLinear(cfg.hidden_size, cfg.hidden_size, dtype=dtype, device=device, std=out_std)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        batch, seq, _ = x.shape
        q = self.q_proj(x).view(batch, seq, self.local_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(batch, seq, self.local_kv_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(batch, seq, self.local_kv_heads, self.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        repeat = self.local_heads // self.local_kv_heads
        if repeat > 1:
            k = k.repeat_interleave(repeat, dim=1)
            v = v.repeat_interleave(repeat, dim=1)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(out.transpose(1, 2).reshape(batch, seq, self.local_heads * self.head_dim))


class MLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, *, dtype, device, std: float, out_std: float) -> None:
        super().__init__()
        self.gate_proj = ColumnParallelLinear(cfg.hidden_size, cfg.intermediate_size, dtype=dtype, device=device, std=std)
        self.up_proj = ColumnParallelLinear(cfg.hidden_size, cfg.intermediate_size, dtype=dtype, device=device, std=std)
        self.down_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, dtype=dtype, device=device, std=out_std)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig, *, dtype, device, std: float, out_std: float) -> None:
        super().__init__()
        self.input_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps, dtype=dtype, device=device)
        self.attention = Attention(cfg, dtype=dtype, device=device, std=std, out_std=out_std)
        self.post_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps, dtype=dtype, device=device)
        self.mlp = MLP(cfg, dtype=dtype, device=device, std=std, out_std=out_std)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        x = x + self.attention(self.input_norm(x), cos, sin)
        return x + self.mlp(self.post_norm(x))


class LlamaTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, *, dtype: torch.dtype = torch.bfloat16, device=None, seed: int = 0) -> None:
        super().__init__()
        self.cfg = cfg
        # identical seeds on every rank would give identical shards; offset by rank for random init
        torch.manual_seed(seed * 1000 + _rank())
        std = 0.02
        out_std = 0.02 / math.sqrt(2 * cfg.num_layers)
        self.embed = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device, std=std)
        self.blocks = nn.ModuleList(
            Block(cfg, dtype=dtype, device=device, std=std, out_std=out_std) for _ in range(cfg.num_layers))
        self.final_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps, dtype=dtype, device=device)
        self.lm_head = ColumnParallelLinear(cfg.hidden_size, cfg.vocab_size, dtype=dtype, device=device, std=std)
        self.vocab_start = _rank() * (cfg.vocab_size // _world())
        # recompute every block in the backward pass instead of keeping its activations (32 layers at sequence
        # length 4096 and batch 8 would otherwise hold over 100 GB of activations per rank)
        self.checkpoint_activations = False

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None) -> Tensor:
        """Mean next-token loss if ``targets`` is given, else this rank's slice of the logits."""
        _, seq = tokens.shape
        cos, sin = rope_tables(self.cfg.hidden_size // self.cfg.num_heads, seq, self.cfg.rope_theta, tokens.device)
        x = self.embed(tokens)
        for block in self.blocks:
            if self.checkpoint_activations and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(block, x, cos, sin, use_reentrant=False)
            else:
                x = block(x, cos, sin)
        logits = self.lm_head(self.final_norm(x))
        if targets is None:
            return logits
        return _VocabParallelCrossEntropy.apply(logits, targets, self.vocab_start).mean()

    def soap_parameters(self):
        """2-D tensor-parallel weights (SOAP-TP) and the rest (AdamW), in a fixed order."""
        matrices = [p for p in self.parameters() if p.ndim == 2]
        others = [p for p in self.parameters() if p.ndim != 2]
        return matrices, others


__all__ = ["LlamaConfig", "LlamaTP", "ColumnParallelLinear", "RowParallelLinear", "VocabParallelEmbedding", "RMSNorm"]
