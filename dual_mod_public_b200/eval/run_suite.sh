#!/usr/bin/env bash
# The post-training evaluation battery of one checkpoint, one job per GPU in round-robin.
#   bash run_suite.sh <ckpt> <gpu list, e.g. 0,1,2,3> [tag]
# Environment: TOK (tokenizer folder), VAL_BIN / TEST_BIN (held-out token files), RULER_ROOT (needle jsonl
# tree), ENGINE_K (> 0: likelihood and generation through the wavefront engine at that K), OUT (default
# analysis).  Jobs write OUT/suite_<tag>_<name>.log; result files are collated with
#   python -m dual_mod_public_b200.eval.collate table $OUT <run>
# Reference parity: lm/eval/run_posttrain_suite.sh, lm/eval/gdn2_evals_dist.sh (battery and job split).
set -euo pipefail
CKPT=$(realpath "$1")
IFS=',' read -ra GPUS <<< "$2"
TAG=${3:-$(basename "$(dirname "$CKPT")")}
OUT=${OUT:-analysis}
TOK=${TOK:-bytes}
K_ARGS=()
[ "${ENGINE_K:-0}" -gt 0 ] && K_ARGS=(--engine_K "$ENGINE_K" --T_eval "${T_EVAL:-2048}")
mkdir -p "$OUT"
i=0
launch() {  # launch <name> <command...>
  local name=$1; shift
  local gpu=${GPUS[$((i % ${#GPUS[@]}))]}; i=$((i + 1))
  CUDA_VISIBLE_DEVICES=$gpu nohup "$@" > "$OUT/suite_${TAG}_${name}.log" 2>&1 &
  echo "[$name] gpu $gpu pid $!"
}
EVAL=(python -m dual_mod_public_b200.eval.run_lm_eval --ckpt "$CKPT" --tokenizer "$TOK" --out_dir "$OUT" --tag "$TAG")
[ -n "${VAL_BIN:-}" ] && launch heldout_val python -m dual_mod_public_b200.eval.heldout_loss --ckpt "$CKPT" --val "$VAL_BIN" --n_batches 21
[ -n "${TEST_BIN:-}" ] && launch heldout_test python -m dual_mod_public_b200.eval.heldout_loss --ckpt "$CKPT" --val "$TEST_BIN" --n_batches 21
launch wikitext "${EVAL[@]}" "${K_ARGS[@]}" --tasks wikitext --batch_rows 32
launch likeli1 "${EVAL[@]}" "${K_ARGS[@]}" --tasks lambada_openai,piqa,hellaswag --batch_rows 64
launch likeli2 "${EVAL[@]}" "${K_ARGS[@]}" --tasks winogrande,arc_easy,arc_challenge --batch_rows 64
launch boolq_sciq "${EVAL[@]}" "${K_ARGS[@]}" --tasks boolq,sciq --batch_rows 64
launch recall env EVAL_LEN_QUANT=1 "${EVAL[@]}" "${K_ARGS[@]}" --tasks jrt_swde,jrt_fda,jrt_squad,jrt_triviaqa,jrt_nq,jrt_drop
launch mqar_zs python -m dual_mod_public_b200.eval.mqar --ckpt "$CKPT" --pairs 8,16,32,64 --n_seq 64
if [ -n "${RULER_ROOT:-}" ]; then
  launch needles "${EVAL[@]}" "${K_ARGS[@]}" --tasks niah_single_1,niah_single_2,niah_single_3,niah_multikey_1,niah_multikey_2 \
    --ruler_root "$RULER_ROOT" --ruler_lengths 2048,4096,8192 --ctx_len 8448 --limit 100
fi
echo "launched $i jobs for $TAG over GPUs $2; logs $OUT/suite_${TAG}_*.log"
