#!/usr/bin/env bash
# Training-curve and (RUN_ABLATIONS=1, the default) message-ablation figures for one run family.
# Run roots: the arguments, else RUN_ROOTS, else FAMILY_DIR, else OUTPUT_ROOT/FAMILY_NAME with the family name the training
# launchers derive from BACKBONE, MODEL_SCALE, TARGET_STEPS, TOKENIZER_TYPE, VOCAB_SIZE, TIE_EMBEDDINGS and FAMILY_SEQ_LEN.
# Figures go to <first root>/plots (plots_<LABEL_MODE> away from auto, plots_<PLOT_SUBDIR> when set), or below
# PLOT_OUTPUT_ROOT/FAMILY_NAME.  LABEL_MODE, REGIMES, SMOOTH_WINDOW, FONT_SCALE, DPI, INCLUDE_VARIANT_REGEX, EXCLUDE_VARIANT_REGEX.
set -euo pipefail
PY="${PYTHON_BIN:-python}"
FAMILY_NAME="${FAMILY_NAME:-$(LBI_LAUNCH_QUIET=1 "$PY" -m lbi_b200.scripts.paper_presets family-name)}"
FAMILY_DIR="${FAMILY_DIR:-${OUTPUT_ROOT:-out/region_interface}/${FAMILY_NAME}}"
if [[ $# -gt 0 ]]; then
  ROOTS=("$@")
elif [[ -n "${RUN_ROOTS:-}" ]]; then
  read -r -a ROOTS <<< "${RUN_ROOTS}"
else
  ROOTS=("${FAMILY_DIR}")
fi
LABEL_MODE="${LABEL_MODE:-auto}"
if [[ -n "${PLOT_SUBDIR:-}" ]]; then
  SUFFIX="_${PLOT_SUBDIR}"
elif [[ "${LABEL_MODE}" != "auto" ]]; then
  SUFFIX="_${LABEL_MODE}"
else
  SUFFIX=""
fi
PLOT_DIR_NAME="${PLOT_DIR_NAME:-plots${SUFFIX}}"
ABLATION_PLOT_DIR_NAME="${ABLATION_PLOT_DIR_NAME:-ablation_plots${SUFFIX}}"
if [[ -n "${PLOT_OUTPUT_ROOT:-}" ]]; then
  BASE="${PLOT_OUTPUT_ROOT%/}/${FAMILY_NAME}"
else
  BASE="${ROOTS[0]%/}"
fi
export MPLBACKEND="${MPLBACKEND:-Agg}"
"$PY" -m lbi_b200.scripts.plot_training_curves "${ROOTS[@]}" --output-dir "${BASE}/${PLOT_DIR_NAME}" --dpi "${DPI:-150}" \
  --font-scale "${FONT_SCALE:-1.0}" --smooth-window "${SMOOTH_WINDOW:-25}" --label-mode "${LABEL_MODE}" \
  ${REGIMES:+--regimes "$REGIMES"} --include-variant-regex "${INCLUDE_VARIANT_REGEX:-}" \
  --exclude-variant-regex "${EXCLUDE_VARIANT_REGEX:-}"
case "${RUN_ABLATIONS:-1}" in
  1|true|yes)
    "$PY" -m lbi_b200.scripts.plot_message_ablations "${ROOTS[@]}" --output-dir "${BASE}/${ABLATION_PLOT_DIR_NAME}" \
      --dpi "${DPI:-150}" --font-scale "${FONT_SCALE:-1.0}" --include-variant-regex "${INCLUDE_VARIANT_REGEX:-}" \
      --exclude-variant-regex "${EXCLUDE_VARIANT_REGEX:-}"
    ;;
esac
