#!/usr/bin/env bash
# 1.3B Dual-Mod run (wavefront engine, c=64, K-ladder) on one node, or several with NNODES / NODE_RANK / MASTER.
#   DATA_BIN=/data/train.bin OUT=out/hero NGPU=8 RECIPE=1p3b bash launch_1p3b.sh
#   RECIPE=hero selects the 18-layer d=2304 rank-144 recipe with the 8/16/24 ladder.
# Reference parity: lm/train_1p3b/launch_hero_wave3d.sh (c10d rendezvous, async error handling, expandable
# segments, per-rank outlier rejection, resume).
set -euo pipefail
NGPU=${NGPU:-8}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER=${MASTER:-127.0.0.1}
PORT=${PORT:-29500}
RECIPE=${RECIPE:-1p3b}
OUT=${OUT:-out/dm1p3b}
DATA_BIN=${DATA_BIN:-}
STEPS=${STEPS:-190650}
WARMUP=${WARMUP:-2000}
# SMOKE=1: a 20-step end-to-end run on synthetic tokens before a long run
if [ "${SMOKE:-0}" = 1 ]; then STEPS=20; WARMUP=5; OUT=${OUT}_smoke; DATA_BIN=; set -- --log_every 1 "$@"; fi
# WINDOW=2048: sliding-window attention of that many tokens (the operator then travels with the checkpoints)
WINDOW_ARGS=()
[ -n "${WINDOW:-}" ] && WINDOW_ARGS=(--model_overrides "{\"local_window\": ${WINDOW}}")
export TORCH_NCCL_ASYNC_ERROR_HANDLING=1
export PYTORCH_CUDA_ALLOC_CONF=${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}
DATA_ARGS=(--synthetic)
[ -n "$DATA_BIN" ] && DATA_ARGS=(--data_bin "$DATA_BIN")
exec python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node "$NGPU" \
  --master-addr "$MASTER" --master-port "$PORT" \
  -m dual_mod_public_b200.train.train_lm --recipe "$RECIPE" --out_dir "$OUT" --total_steps "$STEPS" \
  --warmup_steps "$WARMUP" --clip_mult 2.0 --gn_hard 50 --rank_outlier_factor 4 --ckpt_every 250 --async_ckpt \
  --persist_every 5000 --resume auto --auto_rewind "${WINDOW_ARGS[@]}" "${DATA_ARGS[@]}" "$@"
