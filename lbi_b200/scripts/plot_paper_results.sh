#!/usr/bin/env bash
# Training-curve (and, with RUN_ABLATIONS=1, message-ablation) figures for one run family.
# RUN_ROOTS: space-separated run roots (default: $OUTPUT_ROOT/$FAMILY_NAME).
set -euo pipefail
PY="${PYTHON_BIN:-python}"
ROOTS="${RUN_ROOTS:-${OUTPUT_ROOT:-out/region_interface}/${FAMILY_NAME:?set FAMILY_NAME or RUN_ROOTS}}"
OUT="${PLOT_OUTPUT_ROOT:-${OUTPUT_ROOT:-out/region_interface}/${FAMILY_NAME:-plots}}/${PLOT_DIR_NAME:-plots}"
"$PY" -m lbi_b200.scripts.plot_training_curves $ROOTS --output-dir "$OUT" --dpi "${DPI:-150}" \
  --font-scale "${FONT_SCALE:-1.0}" --smooth-window "${SMOOTH_WINDOW:-1}" --label-mode "${LABEL_MODE:-auto}" \
  --include-variant-regex "${INCLUDE_VARIANT_REGEX:-}" --exclude-variant-regex "${EXCLUDE_VARIANT_REGEX:-}"
if [[ "${RUN_ABLATIONS:-0}" == "1" ]]; then
  "$PY" -m lbi_b200.scripts.plot_message_ablations $ROOTS --output-dir "$(dirname "$OUT")/${ABLATION_PLOT_DIR_NAME:-ablation_plots}" \
    --dpi "${DPI:-150}" --font-scale "${FONT_SCALE:-1.0}"
fi
