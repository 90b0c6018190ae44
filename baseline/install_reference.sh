#!/usr/bin/env bash
# Places the unmodified reference source tree under baseline/_ref (git-ignored).
# `pip install --target baseline/_ref <reference>` is refused because the reference ships neither setup.py nor
# pyproject.toml (it is a flat tree of top-level packages run from its root), so the tree is copied verbatim.
set -euo pipefail
SRC="${1:-${LBI_REFERENCE_SRC:?usage: install_reference.sh <reference checkout> (or set LBI_REFERENCE_SRC)}}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
mkdir -p "$HERE/_ref"
cp -r "$SRC"/. "$HERE/_ref/"
echo "reference copied to $HERE/_ref"
