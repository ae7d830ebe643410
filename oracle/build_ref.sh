#!/bin/bash
# Builds the reference's own CUDA paged-attention kernel (triton/kernels/paged_attention.cu with its vendored XLA
# FFI headers) for sm_100a, straight from the reference checkout, into oracle/_ref/ (git-ignored).  Test
# infrastructure: the result is the "reference itself, run here" leg of the parity tests and of their same-GPU timing
# (tests/test_reference_kernel_gpu.py).  Usage: oracle/build_ref.sh [path of the reference checkout]
set -euo pipefail
REF="${1:-/root/reference}"
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC="$REF/triton/kernels/paged_attention.cu"
[ -f "$SRC" ] || { echo "no reference checkout at $REF" >&2; exit 2; }
NVCC="$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)"
mkdir -p "$HERE/_ref"
OUT="$HERE/_ref/libtlaloc_ref_kernels.so"
if [ -f "$OUT" ] && [ "$OUT" -nt "$SRC" ] && [ "$OUT" -nt "$HERE/ref_wrapper.cu" ]; then echo "$OUT"; exit 0; fi
"$NVCC" -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -lineinfo -shared -Xcompiler -fPIC \
  -I "$REF/triton/kernels" -I "$REF/triton/third_party/xla" "$HERE/ref_wrapper.cu" -o "$OUT"
echo "$OUT"
