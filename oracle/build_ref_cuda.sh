#!/bin/sh
# Builds oracle/_ref/libcswap_ref_cuda.so: the reference's own CUDA codec
# (cuZFP.cu, compression.cu, zfp.c, bitstream.c of CSWAP+/zfp), compiled for
# sm_100a from the sources where they lie (CSWAP_REFERENCE names the checkout),
# plus the entry points of ref_cuda_shim.cpp.  Nothing from the reference is
# copied into the repository.  TEST INFRASTRUCTURE ONLY.
set -e
[ -n "$CSWAP_REFERENCE" ] || { echo "set CSWAP_REFERENCE to the reference checkout" >&2; exit 3; }
REF="$CSWAP_REFERENCE/CSWAP+/zfp"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
NVCC="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
[ -f "$REF/cuZFP.cu" ] || { echo "reference not present at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d)"
trap 'rm -rf "$TMP"' EXIT
gcc -std=c99 -O2 -fPIC -w -I"$REF" -c "$REF/zfp.c" -o "$TMP/zfp.o"
gcc -std=c99 -O2 -fPIC -w -I"$REF" -c "$REF/bitstream.c" -o "$TMP/bitstream.o"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -O3 -w -Xcompiler -fPIC -I"$REF" \
    -c "$REF/cuZFP.cu" -o "$TMP/cuZFP.o"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -O3 -w -Xcompiler -fPIC -I"$REF" \
    -c "$REF/compression.cu" -o "$TMP/compression.o"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -O2 -w -Xcompiler -fPIC -x cu -I"$REF" \
    -c "$HERE/ref_cuda_shim.cpp" -o "$TMP/shim.o"
# -Bsymbolic: the reference's entry points carry the same names as the
# product's compatibility symbols; calls inside this library must stay inside
"$NVCC" -shared -o "$OUT/libcswap_ref_cuda.so" "$TMP/shim.o" "$TMP/cuZFP.o" "$TMP/compression.o" \
    "$TMP/zfp.o" "$TMP/bitstream.o" -Xlinker -Bsymbolic
echo "built $OUT/libcswap_ref_cuda.so"
