#!/usr/bin/env bash
# One dense-baseline paper run; settings come from environment variables (BACKBONE, MODEL_SCALE, SEED, ...).
set -euo pipefail
exec "${PYTHON_BIN:-python}" -m lbi_b200.scripts.paper_presets dense "$@"
