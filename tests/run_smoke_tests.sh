#!/usr/bin/env bash
# End-to-end training smoke tests with a junit report (same role as the reference's tests/run_smoke_tests.sh).
#   tests/run_smoke_tests.sh [junit.xml] [extra pytest arguments]
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
report="${1:-${here}/../smoke_junit.xml}"
shift || true
cd "${here}/.."
exec python -m pytest tests/test_training_workflow_smoke.py -q --junitxml "${report}" "$@"
