#!/usr/bin/env bash
# Strong-scaling run of soap_step on one 8 x B200 node: N = 8192, 1/2/4/8 ranks, one GPU per rank.
# Counterpart of the reference's scripts/slurm/frontier/submit_soap_tp_scaling.sh (ranks 1..8,
# block = min(N / max grid axis, cap), manifest with the git commit) for torchrun instead of srun/MPI.
# Usage: scaling_8xb200.sh [output_dir]
set -euo pipefail
SIZE="${SOAP_SCALING_SIZE:-8192}"
STEPS="${SOAP_SCALING_STEPS:-100}"
BLOCK_CAP="${SOAP_SCALING_BLOCK_CAP:-128}"
RANKS="${SOAP_SCALING_RANKS:-1 2 4 8}"
OUT="${1:-soap_scaling_$(date +%Y%m%d_%H%M%S)}"
mkdir -p "$OUT"
REPO_ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../../.." && pwd)"
printf 'ranks\tblock\tlog\tcommit\n' > "$OUT/manifest.tsv"
COMMIT="$(git -C "$REPO_ROOT" rev-parse --short HEAD 2>/dev/null || echo unknown)"
for N in $RANKS; do
  LOG="$OUT/soap_step_${SIZE}_r${N}.log"
  ( cd "$REPO_ROOT" && SOAP_PROFILE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" \
      --master-addr 127.0.0.1 --master-port $((29600 + N)) -m soap_tp_b200.bench.timing \
      --size "$SIZE" --world-size "$N" --steps "$STEPS" --block-size "$BLOCK_CAP" --shard-dim 1 ) | tee "$LOG"
  printf '%s\t%s\t%s\t%s\n' "$N" "$BLOCK_CAP" "$LOG" "$COMMIT" >> "$OUT/manifest.tsv"
done
grep -h '"event": "summary"' "$OUT"/*.log || true
