#!/usr/bin/env bash
# Test infrastructure, not product code.
#
# Compiles the reference project's own core CUDA source, unmodified and from
# where it lies, for sm_100a.  The result (oracle/_ref/libthorfp4_ref_core.so)
# is a comparison artefact only: the GPU parity tests use its tfp4_quant /
# tfp4_quant_mx as a byte-level checker of the new quantizer, and the bench
# can time its cuBLASLt NVFP4 GEMM on the same box.  Nothing in the product
# library links or loads it.
#
# usage: oracle/build_ref.sh [path-to-reference-checkout]
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
# the checkout: first argument, else THOR_FP4_REFERENCE, else a directory `reference` beside this repository
REF="${1:-${THOR_FP4_REFERENCE:-$HERE/../../reference}}"
OUT="$HERE/_ref"
SRC="$REF/csrc/thor_fp4_core.cu"
if [ ! -f "$SRC" ]; then
  echo "build_ref: $SRC not found; skipping (prebuilt $OUT is used if present)" >&2
  exit 0
fi
mkdir -p "$OUT"
NVCC="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
if [ "$OUT/libthorfp4_ref_core.so" -nt "$SRC" ]; then
  echo "build_ref: up to date"; exit 0
fi
"$NVCC" -gencode arch=compute_100a,code=sm_100a -O2 -std=c++17 -Xcompiler -fPIC -shared \
  -o "$OUT/libthorfp4_ref_core.so" "$SRC" -lcublasLt
echo "build_ref: wrote $OUT/libthorfp4_ref_core.so"
