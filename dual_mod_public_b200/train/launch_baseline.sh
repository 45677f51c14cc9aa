#!/usr/bin/env bash
# Baseline arms of the 340M comparison under torch DDP (micro-batch accumulation with no_sync): the vanilla
# Transformer++ of the same shape (tpp), the parameter-matched wider Transformer (ematch), the gated delta net
# (gdn), and the sequential / looped controls.
#   ARM=tpp DATA_BIN=/data/slimpj_train.bin OUT=out/tpp340 NGPU=8 bash launch_baseline.sh
#   SMOKE=1 ARM=gdn NGPU=2 bash launch_baseline.sh
# Reference parity: lm/train_340m/scripts/launch_tpp.sh, launch_gdn.sh (same recipe as the Dual-Mod arm:
# 256 x 2048 tokens per step, 30k steps, lr 3e-4 -> 3e-5, seed shared with the Dual-Mod run).
set -euo pipefail
ARM=${ARM:-tpp}
NGPU=${NGPU:-8}
OUT=${OUT:-out/${ARM}340}
STEPS=${STEPS:-30000}
WARMUP=${WARMUP:-1000}
PORT=${PORT:-29501}
DATA_BIN=${DATA_BIN:-}
if [ "${SMOKE:-0}" = 1 ]; then STEPS=20; WARMUP=5; OUT=${OUT}_smoke; DATA_BIN=; fi
case $ARM in
  tpp)    ARCH=vanilla; SHAPE=${SHAPE:-1024,24,16,2816} ;;
  ematch) ARCH=ematch;  SHAPE=${SHAPE:-1024,24,16,2816} ;;
  gdn)    ARCH=gdn;     SHAPE=${SHAPE:-1024,24,16,2816} ;;
  fbt|looped|rdepth|lstm) ARCH=$ARM; SHAPE=${SHAPE:-1024,24,16,2816} ;;
  *) echo "unknown arm $ARM" >&2; exit 1 ;;
esac
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
DATA_ARGS=(--synthetic)
[ -n "$DATA_BIN" ] && DATA_ARGS=(--data_bin "$DATA_BIN")
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "$PORT" \
  -m dual_mod_public_b200.train.train_baseline --arch "$ARCH" --shape "$SHAPE" --out_dir "$OUT" --total_steps "$STEPS" \
  --warmup_steps "$WARMUP" --ckpt_every 500 "${DATA_ARGS[@]}" "$@"
