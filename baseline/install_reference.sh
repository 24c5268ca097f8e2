#!/bin/sh
# Installs the UNMODIFIED reference package (nanovllm) from its checkout into
# baseline/_ref (git-ignored) so that the GPU box, which has no checkout, can
# run the reference's own engine next to this repository's backend:
#
#     sh baseline/install_reference.sh /path/to/reference/checkout
#
# The checkout is copied to a scratch directory first because the build writes
# egg-info into the source tree.  No index is contacted; the reference's
# dependencies (torch, triton, transformers, flash-attn, xxhash) are the ones
# already in the image, hence --no-deps.
set -e
SRC="${1:?usage: sh baseline/install_reference.sh /path/to/reference/checkout}"
HERE="$(cd "$(dirname "$0")" && pwd)"
TMP="$(mktemp -d)"
cp -r "$SRC" "$TMP/src"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" --upgrade "$TMP/src"
echo "installed into $HERE/_ref"
