#!/usr/bin/env bash
# 340M Dual-Mod run on one node (cell engine, c=64, K-ladder 8/16/32 with K=64 probes).
#   DATA_BIN=/data/slimpj_train.bin VAL_BIN=/data/slimpj_val.bin OUT=out/dm340 NGPU=8 bash launch_340m.sh
#   SMOKE=1 NGPU=2 bash launch_340m.sh          # 20 steps on synthetic tokens
#   add --protocol pdn for the batch-256 / 30k-step / lr 4e-4 protocol, --model_overrides for another shape
# Every knob is an environment variable with a default; extra flags are passed through ("$@").
# Reference parity: lm/train_340m/scripts/launch_dm_d960.sh, scripts/launch_torchrun.sh.
set -euo pipefail
NGPU=${NGPU:-8}
# RECIPE=340m: the benchmark shape (24 x d1024, dense linear write law).  RECIPE=d960: the reference's own 340M run
# (26 x d960, rank-120 mult_res write law) under its protocol: batch 256, 30k steps, lr 4e-4 trunk / 3e-4 Dual-Mod
# parameters, calibrated clip at 2x, skip factor 20 (lm/train_340m/scripts/launch_dm_d960.sh).
RECIPE=${RECIPE:-340m}
RECIPE_ARGS=()
[ "$RECIPE" = d960 ] && RECIPE_ARGS=(--protocol pdn --dm_lr 3e-4 --clip_mult 2.0 --skip_factor 20 --seed 42)
OUT=${OUT:-out/dm340}
DATA_BIN=${DATA_BIN:-}
VAL_BIN=${VAL_BIN:-}
STEPS=${STEPS:-30000}
WARMUP=${WARMUP:-1000}
# SMOKE=1: a 20-step end-to-end run on synthetic tokens (graphs captured, one checkpoint written) before a long run
if [ "${SMOKE:-0}" = 1 ]; then STEPS=20; WARMUP=5; OUT=${OUT}_smoke; DATA_BIN=; VAL_BIN=; set -- --ckpt_every 10 --log_every 1 "$@"; fi
PORT=${PORT:-29500}
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
DATA_ARGS=(--synthetic)
[ -n "$DATA_BIN" ] && DATA_ARGS=(--data_bin "$DATA_BIN")
[ -n "$VAL_BIN" ] && DATA_ARGS+=(--val_bin "$VAL_BIN" --val_every 500)
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "$PORT" \
  -m dual_mod_public_b200.train.train_lm --recipe "$RECIPE" "${RECIPE_ARGS[@]}" --out_dir "$OUT" --total_steps "$STEPS" \
  --warmup_steps "$WARMUP" --weight_decay 0.01 --ckpt_every 500 --async_ckpt --resume auto --auto_rewind \
  "${DATA_ARGS[@]}" "$@"
