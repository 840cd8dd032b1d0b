#!/usr/bin/env bash
#SBATCH --job-name=soap-tp-b200-scaling
#SBATCH --nodes=1
#SBATCH --gpus-per-node=8
#SBATCH --time=00:30:00
# Single-node strong-scaling job (the reference's Frontier worker is also one node:
# scripts/slurm/frontier/soap_tp_scaling.slurm:5).  One torchrun per rank count; no GPU or clock
# setting is touched.
set -euo pipefail
cd "${SLURM_SUBMIT_DIR:-.}"
export SOAP_PROFILE=0
exec bash soap_tp_b200/bench/launch/scaling_8xb200.sh "soap_scaling_${SLURM_JOB_ID:-local}"
