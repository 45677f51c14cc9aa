#!/usr/bin/env bash
# A5 state tracking (word problem of the alternating group on 5 points), one-layer Dual-Mod on the exact cell
# engine (c=16, K=16), against the vanilla Transformer of the same shape.
#   T=64 STEPS=20000 bash run_a5.sh
# Reference parity: formal_language/a5/run_a5_T64.sh.
set -euo pipefail
T=${T:-64}
STEPS=${STEPS:-20000}
OUT=${OUT:-out/a5}
for ARCH in ${ARCHS:-dualmod vanilla}; do
  ENGINE_ARGS=()
  [ "$ARCH" = dualmod ] && ENGINE_ARGS=(--engine wavescan)
  python -m dual_mod_public_b200.formal.train_statetrack --task group --group a5 --arch "$ARCH" --n_ops "$T" \
    --steps "$STEPS" --out_root "$OUT" "${ENGINE_ARGS[@]}" "$@"
done
