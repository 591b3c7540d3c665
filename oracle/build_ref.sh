#!/bin/bash
# Builds the reference-derived checkers into oracle/_ref/ (git-ignored) from the
# RecFlex checkout, compiling the reference's sources where they lie:
#   libref_kernels.so  the reference's device templates behind oracle/ref_kernels.cu (sm_100a)
#   libref_host.so     the reference's host text parsers behind oracle/ref_host_shim.cc
# Usage: oracle/build_ref.sh <path to the RecFlex checkout>   (or set $RECFLEX_REF)
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${1:-${RECFLEX_REF:-}}"
[ -n "$REF" ] || { echo "usage: $0 <path to the RecFlex checkout> (or set RECFLEX_REF)" >&2; exit 2; }
OUT="$HERE/_ref"
[ -d "$REF/examples/csrc/include" ] || { echo "no RecFlex checkout at $REF" >&2; exit 1; }
mkdir -p "$OUT"
INC="-I$REF/examples/csrc/include -I$REF/RecFlex/sched_basic_csrc/include"
if [ ! -f "$OUT/libref_kernels.so" ] || [ "$HERE/ref_kernels.cu" -nt "$OUT/libref_kernels.so" ]; then
  nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a --expt-relaxed-constexpr --expt-extended-lambda \
       -Xcompiler -fPIC -shared $INC "$HERE/ref_kernels.cu" -o "$OUT/libref_kernels.so"
fi
if [ ! -f "$OUT/libref_host.so" ] || [ "$HERE/ref_host_shim.cc" -nt "$OUT/libref_host.so" ]; then
  nvcc -O2 -std=c++17 -Xcompiler -fPIC -shared $INC "$HERE/ref_host_shim.cc" \
       "$REF/examples/csrc/warp_per_sample_preprocess.cu" "$REF/examples/csrc/onehot_preprocess.cu" \
       -o "$OUT/libref_host.so"
fi
echo "built: $(ls "$OUT")"
