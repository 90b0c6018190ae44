#!/usr/bin/env bash
# Post-hoc evaluation of one run family: FAMILY_DIR (or OUTPUT_ROOT + FAMILY_NAME), CHECKPOINT=best|latest, EVAL_BATCHES.
set -euo pipefail
FAMILY="${FAMILY_DIR:-${OUTPUT_ROOT:-out/region_interface}/${FAMILY_NAME:?set FAMILY_DIR or FAMILY_NAME}}"
OUT="${EVAL_OUTPUT_DIR:-${EVAL_OUTPUT_ROOT:-out/evals/region_interface}/$(basename "$FAMILY")}"
exec "${PYTHON_BIN:-python}" -m lbi_b200.scripts.evaluate_paper_checkpoints "$FAMILY" --output-dir "$OUT" \
  --checkpoint "${CHECKPOINT:-best}" --eval-batches "${EVAL_BATCHES:-512}" --eval-seed "${EVAL_SEED:-12345}" \
  --device "${DEVICE:-auto}" ${BATCH_SIZE:+--batch-size "$BATCH_SIZE"} ${SEQ_LEN:+--seq-len "$SEQ_LEN"}
