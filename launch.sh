#!/bin/bash
# One process per GPU on this node, rendezvous on 127.0.0.1 (the role of scripts/launch.sh in the reference).
#
#   bash launch.sh [--nproc N] [--port P] script.py [script args]       e.g.  bash launch.sh --nproc 8 bench.py --gpus 8
#   bash launch.sh --nproc 2 -m triton_distributed_b200.benchmark.bench_comm_gemm
#
# N defaults to the number of visible GPUs. Environment passed through unchanged: the B200DIST_* toggles and NCCL_*.
set -euo pipefail
nproc=""
port="${MASTER_PORT:-29500}"
while [[ $# -gt 0 ]]; do
  case "$1" in
    --nproc) nproc="$2"; shift 2 ;;
    --port) port="$2"; shift 2 ;;
    *) break ;;
  esac
done
if [[ $# -lt 1 ]]; then
  sed -n '2,8p' "$0"; exit 2
fi
if [[ -z "$nproc" ]]; then
  nproc=$(python -c 'import torch; print(max(torch.cuda.device_count(), 1))')
fi
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-4}"
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export PYTHONPATH="$here${PYTHONPATH:+:$PYTHONPATH}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$nproc" --master-addr 127.0.0.1 --master-port "$port" "$@"
