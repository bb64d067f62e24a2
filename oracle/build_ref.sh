#!/bin/sh
# Compiles oracle/ref_host.cpp against the reference's headers where they lie
# (REF, default /root/reference) into oracle/_ref/libhumming_ref_host.so.
# Only the checker uses it; nothing under oracle/_ref is committed.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${REF:-/root/reference}"
CUDA_INC="${CUDA_INC:-/usr/local/cuda/include}"
mkdir -p "$HERE/_ref"
g++ -O2 -std=c++17 -shared -fPIC -Wno-unknown-pragmas -Wno-attributes \
    -I"$HERE/ref_shim" -I"$REF/humming/include" -I"$CUDA_INC" \
    -o "$HERE/_ref/libhumming_ref_host.so" "$HERE/ref_host.cpp"
echo "$HERE/_ref/libhumming_ref_host.so"
