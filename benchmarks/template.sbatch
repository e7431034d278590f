#!/bin/bash
# Single-node job template: one task per GPU, launched through torchrun.
# (The reference ships slurms/template.slurm for its multi-node JAX runs; peer memory here is CUDA IPC,
# so a decomposition group lives on one node.)
#SBATCH --job-name=jaxdecomp_b200
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:8
#SBATCH --cpus-per-task=32
#SBATCH --time=00:30:00
#SBATCH --output=%x-%j.out

set -euo pipefail
NGPU=${NGPU:-8}
cd "${SLURM_SUBMIT_DIR:-$(dirname "$0")/..}"
python -m jaxdecomp_b200.native            # build the native core once (no-op when current)
LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NGPU} --master-addr 127.0.0.1 --master-port 29500"
$LAUNCH bench.py --gpus "${NGPU}" --steps 10 --warmup 3
$LAUNCH benchmarks/bench_ops.py --pdims 2x4 --size 1024 --ops fft,transpose,halo --halo 16
