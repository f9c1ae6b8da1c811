#!/usr/bin/env bash
# Compiles the reference's own GPU path — cuda/gemm.cu, cuda/cuda_kernel.cu (im2col kernels and
# the three convolution launchers), cuda/reverseNswapdim23.cu, cuda/denseam_kernel.cu,
# cuda/matmulam_kernel.cu, cuda/approx_mul_lut.cu — for sm_100a, unmodified, from a reference
# checkout, against the stand-in TensorFlow / Eigen names in oracle/tf_stub, and links them with
# oracle/ref_cuda_shim.cu into oracle/_ref/libref_cuda.so.  The reference's own build system is
# not run; its flags (Makefile:3-4,23: -DGOOGLE_CUDA=1 -O2 -std=c++11, MULTIPLIER=AMSIMULATOR)
# are repeated here.  The include guard of its vendored gpu_kernel_helper.h is pre-defined: that
# header pulls in TensorFlow internals and none of these files uses anything from it.
# Usage: oracle/build_ref_cuda.sh [reference_dir]
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${AMSIM_REFERENCE_DIR:-$here/../../reference}}"
if [ ! -f "$ref/cuda/cuda_kernel.cu" ] || ! command -v nvcc >/dev/null; then
  echo "no reference checkout at $ref (or no nvcc): oracle/_ref/libref_cuda.so not rebuilt"
  exit 0
fi
mkdir -p "$here/_ref"
tmp="$(mktemp -d)"
flags=(-gencode arch=compute_100a,code=sm_100a -O2 -std=c++14 -w -Xcompiler -fPIC --expt-relaxed-constexpr
       -DGOOGLE_CUDA=1 -DAMSIMULATOR=1 -DTENSORFLOW_CORE_UTIL_GPU_KERNEL_HELPER_H_
       -I "$here/tf_stub" -I "$ref" -I "$ref/cuda")
for f in gemm cuda_kernel reverseNswapdim23 denseam_kernel matmulam_kernel approx_mul_lut; do
  nvcc -x cu "${flags[@]}" -c "$ref/cuda/$f.cu" -o "$tmp/$f.o"
done
nvcc "${flags[@]}" -c "$here/ref_cuda_shim.cu" -o "$tmp/shim.o"
nvcc -shared -o "$here/_ref/libref_cuda.so" "$tmp"/*.o
rm -rf "$tmp"
echo "oracle/_ref/libref_cuda.so built from $ref"
