#!/usr/bin/env bash
# One LBI paper run; settings come from environment variables (BACKBONE, MODEL_SCALE, MESSAGE_DIM, REGION_SIZE, SEED, ...).
set -euo pipefail
exec "${PYTHON_BIN:-python}" -m lbi_b200.scripts.paper_presets lbi "$@"
