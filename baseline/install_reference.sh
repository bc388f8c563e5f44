#!/usr/bin/env bash
# Installs the unmodified reference (a workspace of ten wheels sharing the PEP 420 namespace `opaque`) into
# baseline/_ref, offline.  The root distribution ships no code, so each pure-Python member is installed with
# pip into a scratch target and the namespace trees are merged (pip --target refuses to merge into an existing
# `opaque/` directory).  opaque-accounting is a Rust/maturin build and is skipped: the benchmark arm passes the noise
# multiplier directly and never calls the accountant.
#   usage: baseline/install_reference.sh /path/to/reference
set -euo pipefail
REF="${1:?usage: baseline/install_reference.sh /path/to/reference (the checkout of the reference repository)}"
HERE="$(cd "$(dirname "$0")" && pwd)"
DEST="$HERE/_ref"
SCRATCH="$(mktemp -d)"
mkdir -p "$DEST"
for member in base engine optimizers dpsgd dpftrl patches alignment auditing transformers; do
  python -m pip install --quiet --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
      --target "$SCRATCH/$member" "$REF/packages/opaque-$member"
  cp -r "$SCRATCH/$member/." "$DEST/"
done
echo "installed into $DEST:"; ls "$DEST/opaque" "$DEST/opaque/api"
