"""Tensor-parallel training loop: Llama-shaped decoder + ``SoapTP`` on synthetic tokens.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m soap_tp_b200.train \
        --preset llama3-8b --seq-len 4096 --global-batch 8 --steps 5

One process per GPU (NCCL); ``--device cpu`` runs the same code on gloo ranks with the tiny preset.
SOAP-TP runs on every 2-D tensor-parallel weight: two-sided where both sides are at most ``--max-precond-dim``,
one-sided (identity basis on the sharded, vocabulary-sized side, as original SOAP does above its
``max_precond_dim``) for the embedding and the head; AdamW on 1-D parameters.  Token ids are uniform
random (there is no dataset here); weights are random-initialised in bf16, optimizer state is fp32.
Rank 0 prints one ``SOAP_TIMING``-style JSON line per step and a summary.
"""
from __future__ import annotations

import argparse
import os
import time

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")    # no lazy kernel loading in the middle of a training step

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from .models.llama_tp import LlamaConfig, LlamaTP
from .optim import SoapTP
from .profiling import emit_timing


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--preset", choices=("llama3-8b", "tiny"), default="tiny")
    parser.add_argument("--layers", type=int, default=None, help="override the number of decoder layers")
    parser.add_argument("--seq-len", type=int, default=None)
    parser.add_argument("--global-batch", type=int, default=8)
    parser.add_argument("--steps", type=int, default=3)
    parser.add_argument("--lr", type=float, default=3e-3)
    parser.add_argument("--block-size", type=int, default=128)
    parser.add_argument("--precondition-frequency", type=int, default=10)
    parser.add_argument("--max-precond-dim", type=int, default=16384)
    parser.add_argument("--basis-implementation", default="householder")
    parser.add_argument("--device", choices=("cuda", "cpu"), default="cuda")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--checkpoint-activations", action="store_true",
                        help="recompute each decoder block in the backward pass (needed for all 32 layers of the 8B preset)")
    return parser.parse_args(argv)


def train(args: argparse.Namespace) -> dict:
    created = False
    if not dist.is_initialized():
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        if args.device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo", rank=rank, world_size=world)
        created = True
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device()) if args.device == "cuda" else torch.device("cpu")
    cfg = LlamaConfig.llama3_8b() if args.preset == "llama3-8b" else LlamaConfig.tiny()
    if args.layers is not None:
        cfg.num_layers = args.layers
    seq_len = args.seq_len or cfg.max_seq_len
    dtype = torch.bfloat16 if args.device == "cuda" else torch.float32
    model = LlamaTP(cfg, dtype=dtype, device=device, seed=args.seed)
    model.checkpoint_activations = bool(args.checkpoint_activations)
    matrices, others = model.soap_parameters()
    optimizer = SoapTP(
        [{"params": matrices}, {"params": others, "weight_decay": 0.0}],
        lr=args.lr, block_size=args.block_size, precondition_frequency=args.precondition_frequency,
        max_precond_dim=args.max_precond_dim, basis_implementation=args.basis_implementation,
    )
    generator = torch.Generator(device=device).manual_seed(args.seed + 17)  # same tokens on every TP rank
    losses, seconds = [], []
    emit_timing("configuration", preset=args.preset, layers=cfg.num_layers, hidden=cfg.hidden_size,
                ranks=world, seq_len=seq_len, global_batch=args.global_batch, measured_steps=args.steps,
                parameters_per_rank=sum(p.numel() for p in model.parameters()))
    for step in range(args.steps):
        tokens = torch.randint(0, cfg.vocab_size, (args.global_batch, seq_len + 1), generator=generator, device=device)
        dist.barrier()
        if device.type == "cuda":
            torch.cuda.synchronize()
        start = time.perf_counter()
        loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        if device.type == "cuda":
            torch.cuda.synchronize()
        elapsed = torch.tensor([time.perf_counter() - start], dtype=torch.float64, device=device)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        losses.append(float(loss.detach()))
        seconds.append(float(elapsed))
        emit_timing("step", step=step, seconds=seconds[-1], loss=losses[-1],
                    tokens_per_second=args.global_batch * seq_len / seconds[-1])
    summary = dict(losses=losses, seconds=seconds)
    peak = torch.cuda.max_memory_allocated(device) / 2**30 if device.type == "cuda" else None
    emit_timing("summary", ranks=world, measured_steps=args.steps, seconds_per_step=sum(seconds) / max(1, len(seconds)),
                final_loss=losses[-1] if losses else None, peak_allocated_gib=peak,
                one_sided_parameters=sum(1 for g in optimizer.param_groups for p in g["params"]
                                         if (optimizer._plan(p, g) or {}).get("one_sided")))
    if created:
        dist.destroy_process_group()
    return summary


if __name__ == "__main__":
    train(parse_args())
