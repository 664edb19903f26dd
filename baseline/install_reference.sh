#!/bin/bash
# Installs the unmodified reference package (fhog) into baseline/_ref, offline.
#
#     baseline/install_reference.sh <path of the reference checkout>
#
# The reference declares the `uv_build` build backend, which is not available without a network,
# so a plain `pip install <checkout>` stops with "No module named 'uv_build'".  This recipe installs
# from a scratch copy whose only change is the [build-system] table of pyproject.toml (setuptools
# instead of uv_build, same package list); every installed .py file is byte-identical to the
# reference's.  baseline/_ref is git-ignored: it is a build product, not source of this repo.
set -euo pipefail
SRC=${1:?usage: install_reference.sh <path of the reference checkout>}
HERE=$(cd "$(dirname "$0")" && pwd)
TMP=$(mktemp -d /tmp/fhog_ref_XXXXXX)
cp -r "$SRC"/. "$TMP"/
python - "$TMP/pyproject.toml" <<'PY'
import re, sys
path = sys.argv[1]
text = open(path).read()
text = re.sub(r'\[build-system\].*?(?=\n\[)', '[build-system]\nrequires = ["setuptools"]\n'
              'build-backend = "setuptools.build_meta"\n', text, flags=re.S)
text = re.sub(r'\[project\.scripts\].*?(?=\n\[)', '', text, flags=re.S)
text += '\n[tool.setuptools]\npackages = ["fhog", "fhog.jax_refs"]\n'
open(path, "w").write(text)
PY
rm -rf "$HERE/_ref"
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" "$TMP"
rm -rf "$TMP"
for f in __init__.py triton_bwdbwd.py triton_flash.py; do
  cmp "$SRC/fhog/$f" "$HERE/_ref/fhog/$f"
done
echo "installed: $(ls "$HERE/_ref")"
