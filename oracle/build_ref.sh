#!/bin/bash
# Builds the upstream fastsafetensors (the reference) as a checker, without running its own
# build system: g++ compiles its single native source where it lies, and its pure-Python
# layer is staged beside the built module so that the package can be imported from
# oracle/_ref on a machine that has no copy of the upstream tree.
#
# Everything this script writes goes under oracle/_ref/, which is git-ignored: no upstream
# source becomes part of this repository's history.  The result is test infrastructure only
# (parity checker, and the CPU arm of bench.py); the product never imports it.
#
# usage: oracle/build_ref.sh <path-to-upstream-tree>     (or FST_UPSTREAM_TREE in the environment)
set -euo pipefail
REF="${1:-${FST_UPSTREAM_TREE:-}}"
if [ -z "$REF" ]; then
    echo "build_ref: no upstream tree given (argument or FST_UPSTREAM_TREE); keeping any prebuilt oracle/_ref" >&2
    exit 0
fi
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
PY="${PYTHON:-python}"
if [ ! -f "$REF/fastsafetensors/cpp/ext.cpp" ]; then
    echo "build_ref: upstream tree not found at $REF (keeping any prebuilt oracle/_ref)" >&2
    exit 0
fi
EXT_SUFFIX="$($PY -c 'import sysconfig; print(sysconfig.get_config_var("EXT_SUFFIX"))')"
PY_INC="$($PY -c 'import sysconfig; print(sysconfig.get_paths()["include"])')"
PB_INC="$($PY -c 'import pybind11; print(pybind11.get_include())')"
VERSION="$(sed -n 's/^version = "\(.*\)"/\1/p' "$REF/pyproject.toml" | head -1)"
mkdir -p "$OUT/fastsafetensors/copier" "$OUT/fastsafetensors/frameworks"
# 1. native module: one translation unit, plain C++17, CUDA/cuFile/numa are dlopen()ed by it
g++ -O2 -std=c++17 -fPIC -shared -fvisibility=hidden -D__MOD_NAME__=cpp \
    -I"$REF/fastsafetensors/cpp" -I"$PB_INC" -I"$PY_INC" \
    "$REF/fastsafetensors/cpp/ext.cpp" -o "$OUT/fastsafetensors/cpp$EXT_SUFFIX"
# 2. pure-Python layer, staged verbatim (git-ignored)
for f in "$REF"/fastsafetensors/*.py "$REF"/fastsafetensors/*.pyi; do cp -f "$f" "$OUT/fastsafetensors/"; done
cp -f "$REF"/fastsafetensors/copier/*.py "$OUT/fastsafetensors/copier/"
cp -f "$REF"/fastsafetensors/frameworks/*.py "$OUT/fastsafetensors/frameworks/"
# 3. minimal distribution metadata (the package reads its own version through importlib.metadata)
DI="$OUT/fastsafetensors-$VERSION.dist-info"
mkdir -p "$DI"
printf 'Metadata-Version: 2.1\nName: fastsafetensors\nVersion: %s\n' "$VERSION" > "$DI/METADATA"
echo "build_ref: built fastsafetensors $VERSION into $OUT"
