#!/usr/bin/env bash
# Single-node sweeps over GPU counts, process grids and sizes: the analogue of the reference's
# Slurm drivers (benchmarks/slurm.sh weak scaling, benchmarks/slurm_strong_scaling.sh), for one
# NVSwitch box launched with torchrun.  Writes one JSON line per measurement to $OUT.
#   OUT=results.jsonl GPUS="1 2 4 8" SIZES="256 512 1024" bash benchmarks/sweep.sh
set -euo pipefail
cd "$(dirname "$0")/.."
OUT=${OUT:-bench_results.jsonl}
GPUS=${GPUS:-"1 2 4 8"}
SIZES=${SIZES:-"256 512 1024"}
OPS=${OPS:-"fft,transpose,halo"}
PORT=${PORT:-29520}
: > "$OUT"
for n in $GPUS; do
  grids="1x$n"
  if [ "$n" -ge 4 ]; then grids="$grids 2x$((n / 2)) $((n / 2))x2 ${n}x1"; fi
  for pd in $grids; do
    for s in $SIZES; do
      if [ "$n" -eq 1 ]; then
        python benchmarks/bench_ops.py --size "$s" --pdims "$pd" --ops "$OPS" >> "$OUT"
      else
        python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 \
          --master-port "$PORT" benchmarks/bench_ops.py --size "$s" --pdims "$pd" --ops "$OPS" >> "$OUT"
      fi
    done
  done
  # weak scaling point of the reference: 64 x 128 x 128 elements per GPU
  if [ "$n" -eq 1 ]; then
    python benchmarks/bench_ops.py --local-shape 64 128 128 --pdims "1x1" --ops fft >> "$OUT"
  else
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 \
      --master-port "$PORT" benchmarks/bench_ops.py --local-shape 64 128 128 --pdims "1x$n" --ops fft >> "$OUT"
  fi
done
echo "wrote $OUT"
