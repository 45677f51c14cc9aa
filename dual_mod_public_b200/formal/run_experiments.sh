#!/usr/bin/env bash
# One driver for the formal-language experiment families.  Every run prints a FINAL line and writes
# analysis/statetrack_<tag>_<arch>.json under $OUT; --eval_dump also saves the checkpoint that the next
# link of a warm chain starts from.
#
#   GPU=0 bash run_experiments.sh a5_minlayers  <arm> <T> <layers>      # shallowest depth that solves A5 at T in 5..20
#   GPU=0 bash run_experiments.sh a5_depthgrid                          # accuracy over T x depth, Dual-Mod (3 seeds) and vanilla
#   GPU=0 bash run_experiments.sh keyed         <arm> <K>               # K interleaved A5 registers, 8 ops each, cold start
#   GPU=0 bash run_experiments.sh keyed_chain   <arm> <ckpt> <K_from> <K_to>   # register ramp K -> 2K, warm
#   GPU=0 bash run_experiments.sh cvp           <arm> <n> [layers]      # circuit value problem with n gates, cold start
#   GPU=0 bash run_experiments.sh cvp_chain     <arm> <ckpt> <n>        # n -> 2n gates, warm
#   GPU=0 bash run_experiments.sh lengthgen     <arm> <language> [seed] # train on lengths 2..50, test to 10x (GF=... for 32x)
#   GPU=0 bash run_experiments.sh parity        <arm>                   # positive control for the looped arms
#   GPU=0 bash run_experiments.sh fixed_points  <ckpt> [K]              # per-iterate change / accuracy of a looped checkpoint
#
# Arms: dm (Dual-Mod, mult_res write law; on the cell engine where sequences are long), dm_nope, dm_logn, tpp
# (vanilla), lstm, gdn, fbt (1 layer), fbt9, ag / kt (looped, random / size-tied iteration counts), hug1 / hug2
# (recurrent depth).  Environment: OUT (default .), SEED, STEPS, GF (length factors), PY.
# Reference parity: formal_language/{a5,keyed_a5,cvp,length_gen,loop_fixed_point}/*.sh.
set -euo pipefail
PY=${PY:-python}
OUT=${OUT:-.}
export CUDA_VISIBLE_DEVICES=${GPU:-0}
H=(-m dual_mod_public_b200.formal.train_statetrack --out_root "$OUT")
SEED=${SEED:-1337}

# flags of an arm: arm_flags <arm> <loop budget> <lr of the looped arms>
arm_flags() {
  local arm=$1 lk=${2:-64} llr=${3:-1e-4}
  case $arm in
    dm)      echo "--arch dualmod --ctx_mod mult_res --lr 4e-4" ;;
    dm_ws)   echo "--arch dualmod --ctx_mod mult_res --lr 4e-4 --engine wavescan --loss_guard" ;;
    dm_nope) echo "--arch dualmod --ctx_mod mult_res --lr 4e-4 --nope" ;;
    dm_logn) echo "--arch dualmod --ctx_mod mult_res --lr 4e-4 --attn_logn_ref 50" ;;
    tpp)     echo "--arch vanilla --lr ${TPP_LR:-1e-4}" ;;
    tpp_nope) echo "--arch vanilla --lr ${TPP_LR:-1e-4} --nope" ;;
    lstm)    echo "--arch lstm --lr 4e-4" ;;
    gdn)     echo "--arch gdn --lr 4e-4" ;;
    fbt)     echo "--arch fbt --n_layers 1 --lr 2e-4" ;;
    fbt9)    echo "--arch fbt --lr 2e-4" ;;
    ag)      echo "--arch looped --loop_layers 2 --loop_k $lk --loop_k_min $((lk / 4)) --eval_loop_ks $((lk / 2)),$lk,$((lk * 2)) --lr $llr" ;;
    kt)      echo "--arch looped --loop_layers 2 --loop_k $((lk * 2)) --loop_k_per_ops ${PER_OPS:-1} --lr $llr" ;;
    hug1|hug2) echo "--arch looped --loop_layers ${arm#hug} --loop_k 128 --loop_huginn --loop_emb_scale --eval_loop_ks 16,32,64,128 --lr $llr" ;;
    *) echo "unknown arm $arm" >&2; return 1 ;;
  esac
}
kmax() { local k=$1 m=64; while [ "$m" -lt "$k" ]; do m=$((m * 2)); done; echo "$m"; }     # vocabulary ladder 64 / 128 / ...
rows_for() { local k=$1; if [ "$k" -ge 1024 ]; then echo 2; elif [ "$k" -ge 512 ]; then echo 4; elif [ "$k" -ge 256 ]; then echo 8; else echo 64; fi; }

fam=${1:?family}; shift
case $fam in
  a5_minlayers)
    arm=${1:?arm}; T=${2:?T}; L=${3:?layers}
    # shellcheck disable=SC2046
    $PY "${H[@]}" --task group --group a5 --format tagged --scale 63m --steps "${STEPS:-12000}" --seed "$SEED" --n_ops "$T" \
      --gen_factors 1 $(arm_flags "$arm" 16) --n_layers "$L" ;;
  a5_depthgrid)
    for T in 16 32 48 64; do for L in 1 2 3 4 6 9; do
      for s in 1337 1338 1339; do
        $PY "${H[@]}" --task group --group a5 --format tagged --n_ops $T --gen_factors 1,2,4 --scale 63m --steps "${STEPS:-12000}" \
          --bsz 64 $(arm_flags dm) --n_layers $L --seed $s
      done
      $PY "${H[@]}" --task group --group a5 --format tagged --n_ops $T --gen_factors 1,2,4 --scale 63m --steps "${STEPS:-12000}" \
        --bsz 64 $(arm_flags tpp) --n_layers $L
    done; done ;;
  keyed)
    arm=${1:?arm}; K=${2:?K}
    common="--task keyed --group a5 --D 8 --K $K --K_max $(kmax "$K") --steps ${STEPS:-12000} --seed $SEED --eval_dump"
    if [ "$arm" = dm ]; then      # one-layer Dual-Mod on the cell engine (the eager scan runs out of memory past a few k tokens)
      $PY "${H[@]}" $common --scale 63m --n_layers 1 --bsz 64 $(arm_flags dm_ws)
    else
      $PY "${H[@]}" $common --scale w1280 --curriculum --bsz "$(rows_for "$K")" $(arm_flags "$arm" 64)
    fi ;;
  keyed_chain)
    arm=${1:?arm}; ck=${2:?ckpt}; K=${3:?K_from}; K2=${4:?K_to}
    common="--task keyed --group a5 --D 8 --K $K2 --K_max $(kmax "$K2") --steps ${STEPS:-12000} --key_shuffle --newkey_init mean --K_curriculum $K --init_from $ck --eval_dump --seed $SEED"
    if [ "$arm" = dm ]; then
      $PY "${H[@]}" $common --scale 63m --n_layers 1 --bsz 64 $(arm_flags dm_ws)
    else
      $PY "${H[@]}" $common --scale w1280 --bsz "$(rows_for "$K2")" --early_stop 0.995 $(arm_flags "$arm" 64)
    fi ;;
  cvp)
    arm=${1:?arm}; n=${2:?n}; L=${3:-0}
    common="--task cvp --cvp_format tagged --cvp_inputs 12 --gen_factors 1,2 --scale 63m --steps ${STEPS:-30000} --bsz 64 --curriculum --n_ops $n --seed $SEED --eval_dump"
    [ "$L" -gt 0 ] && common="$common --n_layers $L"
    if [ "$arm" = dm ] && [ "$n" -ge 32 ]; then a=dm_ws; else a=$arm; fi
    $PY "${H[@]}" $common $(arm_flags "$a" $((n * 2))) ;;
  cvp_chain)
    arm=${1:?arm}; ck=${2:?ckpt}; n=${3:?n}; B=64; [ "$n" -ge 512 ] && B=16; [ "$n" -ge 1024 ] && B=4
    common="--task cvp --cvp_format tagged --cvp_inputs 12 --gen_factors 1,2 --scale 63m --steps ${STEPS:-30000} --bsz $B --curriculum --curriculum_end 2000 --n_ops $n --init_from $ck --eval_dump --early_stop 0.995 --seed $SEED"
    if [ "$arm" = dm ]; then a=dm_ws; else a=$arm; fi
    $PY "${H[@]}" $common $(arm_flags "$a" $((n * 2))) ;;
  lengthgen)
    arm=${1:?arm}; lang=${2:?language}; s=${3:-1337}
    extra=""; [ "$lang" = flipflop ] && extra="--dfa_sep"
    TPP_LR=4e-4 $PY "${H[@]}" --task dfa --dfa "$lang" $extra --n_ops 50 --len_min 2 --gen_factors "${GF:-1,2,4,6,8,10}" --scale 63m \
      --steps "${STEPS:-12000}" --bsz 64 --seed "$s" --eval_dump $(TPP_LR=4e-4 arm_flags "$arm" 16) ;;
  parity)
    arm=${1:-tpp}
    TPP_LR=4e-4 $PY "${H[@]}" --task parity --n_ops 32 --gen_factors 1,2,4 --scale 63m --steps "${STEPS:-12000}" --bsz 64 --seed "$SEED" \
      $(TPP_LR=4e-4 arm_flags "$arm" 64) ;;
  fixed_points)
    $PY -m dual_mod_public_b200.formal.loop_fixed_point "${1:?ckpt}" --K "${2:-64}" ;;
  *) echo "unknown family $fam" >&2; exit 1 ;;
esac
