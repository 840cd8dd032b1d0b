#!/usr/bin/env bash
#SBATCH --job-name=soap-tp-b200-accuracy
#SBATCH --nodes=1
#SBATCH --gpus-per-node=8
#SBATCH --time=01:00:00
# Accuracy sweep 8^2 ... 8192^2 on 8 ranks (counterpart of scripts/slurm/frontier/soap_accuracy.slurm:62-68
# of the reference), followed by the log summary.
set -euo pipefail
cd "${SLURM_SUBMIT_DIR:-.}"
OUT="soap_accuracy_${SLURM_JOB_ID:-local}.log"
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m soap_tp_b200.bench.accuracy \
  --sizes 8 16 32 64 128 256 512 1024 2048 4096 8192 --rtol 1e-5 | tee "$OUT"
python -m soap_tp_b200.utils.plot_accuracy "$OUT" --csv "${OUT%.log}.csv" --png "${OUT%.log}.png"
