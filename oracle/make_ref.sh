#!/usr/bin/env bash
# Install the UNMODIFIED reference package (pure Python) into oracle/_ref/ so that checks and baselines that
# run away from the reference checkout can import it as `dart`.  oracle/_ref/ is a build output: it is listed in
# .gitignore and never committed.  The checkout may be read-only, so the install runs from a scratch copy.
#
#   oracle/make_ref.sh /path/to/reference/checkout
#
# Dependency resolution is skipped (--no-deps): the reference pins an older transformers release than the one
# in this image; oracle/ref_compat.py adapts the two call sites that differ, from outside the package.
set -euo pipefail
SRC="${1:?usage: oracle/make_ref.sh <reference checkout>}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
mkdir -p "$TMP/ref"
cp -r "$SRC/pyproject.toml" "$SRC/README.md" "$SRC/src" "$TMP/ref/"
[ -f "$SRC/LICENSE" ] && cp "$SRC/LICENSE" "$TMP/ref/"
mkdir -p "$HERE/_ref"
python -m pip install --quiet --no-index --no-build-isolation --no-deps --upgrade --target "$HERE/_ref" "$TMP/ref"
python - <<PY
import sys
sys.path.insert(0, "$HERE/_ref")
import dart
print("installed reference package at", dart.__file__)
PY
