#!/bin/sh
# Builds oracle/_ref/libcswap_ref.so from the reference's own sources where
# they lie (CSWAP_REFERENCE names the checkout).  Nothing from the reference is copied
# into the repository: the two sparse kernels' bodies are cut into a temporary
# directory for the duration of the compile and removed afterwards.
# TEST INFRASTRUCTURE ONLY.
set -e
[ -n "$CSWAP_REFERENCE" ] || { echo "set CSWAP_REFERENCE to the reference checkout" >&2; exit 3; }
REF="$CSWAP_REFERENCE/CSWAP+/zfp"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
CUDA_INC="${CUDA_HOME:-/usr/local/cuda}/include"
[ -f "$REF/encode.cuh" ] || { echo "reference not present at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
# kernels only (PreAcc; PreGPUcompression, GPUcompression, GPUdecompression);
# the launch wrappers use <<<>>> and cannot be compiled by g++
sed -n '9,19p;134,318p' "$REF/compression.cu" > "$TMP/ref_sparse_kernels.inc"
gcc -std=c99 -O2 -fPIC -w -I"$REF" -c "$REF/bitstream.c" -o "$TMP/bitstream.o"
g++ -std=c++14 -O2 -fPIC -w -fpermissive -I"$REF" -I"$CUDA_INC" -I"$TMP" \
    -c "$HERE/ref_shim.cpp" -o "$TMP/ref_shim.o"
# shared.h defines (never called) helpers that reference the CUDA runtime
CUDA_LIB="${CUDA_HOME:-/usr/local/cuda}/lib64"
g++ -shared -o "$OUT/libcswap_ref.so" "$TMP/ref_shim.o" "$TMP/bitstream.o" \
    -L"$CUDA_LIB" -Wl,-rpath,"$CUDA_LIB" -lcudart
echo "built $OUT/libcswap_ref.so"
