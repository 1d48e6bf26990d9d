#!/usr/bin/env bash
# Installs the UNMODIFIED reference package (pi3) into baseline/_ref, which is git-ignored but
# travels to the benchmark machine with the repository.  The reference checkout is read-only and
# setuptools writes into the source tree, so the install runs from a temporary copy.
#   usage: baseline/install_ref.sh [path-to-reference-checkout]
set -euo pipefail
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
cp -r "$REF" "$TMP/ref"
rm -rf "$HERE/_ref"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" "$TMP/ref"
python - <<PY
import sys
sys.path.insert(0, "$HERE/_ref")
import pi3.models.sparse_attn.flash_attention_topk, pi3.models.layers.sparse_attention  # noqa
print("reference installed in $HERE/_ref")
PY
