#!/usr/bin/env bash
# TinyStories ablation arms A / E(=F2) / B / C / D, one after another on NGPU GPUs.
#   DATA_DIR=data/tinystories NGPU=2 bash run_ablation.sh
# Reference parity: tinystories/run_ablation.sh.
set -euo pipefail
NGPU=${NGPU:-2}
DATA_DIR=${DATA_DIR:-data/tinystories}
OUT=${OUT:-out/tinystories}
for P in ${PRESETS:-A F2 B C D}; do
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port 29500 \
    -m dual_mod_public_b200.tinystories.train --preset "$P" --data_dir "$DATA_DIR" --out_dir "$OUT" "$@"
done
