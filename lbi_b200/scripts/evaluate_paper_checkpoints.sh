#!/usr/bin/env bash
# Post-hoc evaluation of one run family.  The family is FAMILY_DIR, or OUTPUT_ROOT/FAMILY_NAME, or the name the training
# launchers derive from BACKBONE, MODEL_SCALE, TARGET_STEPS, TOKENIZER_TYPE, VOCAB_SIZE, TIE_EMBEDDINGS and FAMILY_SEQ_LEN.
# CHECKPOINT=best|latest, EVAL_BATCHES, EVAL_SEED, DEVICE, BATCH_SIZE, SEQ_LEN, TOKENIZER_PATH; extra arguments are passed on
# (e.g. --run-dir <dir>).
set -euo pipefail
PY="${PYTHON_BIN:-python}"
FAMILY_NAME="${FAMILY_NAME:-$(LBI_LAUNCH_QUIET=1 "$PY" -m lbi_b200.scripts.paper_presets family-name)}"
FAMILY="${FAMILY_DIR:-${OUTPUT_ROOT:-out/region_interface}/${FAMILY_NAME}}"
OUT="${EVAL_OUTPUT_DIR:-${EVAL_OUTPUT_ROOT:-out/evals/region_interface}/${FAMILY_NAME}}"
exec "$PY" -m lbi_b200.scripts.evaluate_paper_checkpoints --family "$FAMILY" --output-dir "$OUT" \
  --checkpoint "${CHECKPOINT:-best}" --eval-batches "${EVAL_BATCHES:-512}" --eval-seed "${EVAL_SEED:-12345}" \
  --device "${DEVICE:-auto}" ${BATCH_SIZE:+--batch-size "$BATCH_SIZE"} ${SEQ_LEN:+--seq-len "$SEQ_LEN"} \
  ${TOKENIZER_PATH:+--tokenizer-path "$TOKENIZER_PATH"} "$@"
