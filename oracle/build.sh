#!/usr/bin/env bash
# Builds the CPU oracle (test infrastructure) and, when a reference checkout is
# available, the pieces of the reference that compile on their own:
#   oracle/libamsim_oracle.so      C restatement (always)
#   oracle/_ref/libref_amsim.so    reference cuda/AMsimulator.inl as host C++
#   oracle/_ref/lut/*.bin          output of the reference's lut/lut_gen.cc
#   oracle/_ref/lut/MBM_11.bin     m = 11 LUT from cuda/FPmultMBM_fast32.inl
#   oracle/_ref/libref_model_<LUT>.so   the functional model each shipped LUT was generated from
#   oracle/_ref/libref_cuda.so     the reference's GPU kernels and launchers (oracle/build_ref_cuda.sh)
# Reference sources are compiled where they lie; nothing is copied.
# Usage: oracle/build.sh [reference_dir]
# (default: $AMSIM_REFERENCE_DIR, else the directory "reference" beside this repository)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${AMSIM_REFERENCE_DIR:-$here/../../reference}}"

gcc -O2 -fPIC -shared -fopenmp -ffp-contract=off -fno-fast-math -std=c11 \
    -o "$here/libamsim_oracle.so" "$here/amsim_oracle.c" -lm

if [ -f "$ref/cuda/AMsimulator.inl" ]; then
  mkdir -p "$here/_ref/lut"
  g++ -O2 -fPIC -shared -std=c++14 -I"$ref/cuda" \
      -o "$here/_ref/libref_amsim.so" "$here/ref_shim.cc"
  # lut/lut_gen.cc writes <MODEL>_<m>.bin into the current directory
  # (lut/lut_gen.cc:88-97); same compile line as lut/lut_gen.sh:14.
  tmp="$(mktemp -d)"
  for mul in FMBM16_MULTIPLIER FMBM14_MULTIPLIER FMBM12_MULTIPLIER FMBM10_MULTIPLIER \
             MITCHEL16_MULTIPLIER MITCHEL14_MULTIPLIER MITCHEL12_MULTIPLIER \
             MITCHEL10_MULTIPLIER BFLOAT; do
    g++ -w -D$mul -I"$ref/lut" -o "$tmp/lut_gen_$mul" "$ref/lut/lut_gen.cc"
    (cd "$here/_ref/lut" && "$tmp/lut_gen_$mul")
  done
  # the functional models themselves, for the LUT-vs-model sweep of lut/test.cc
  for pair in FMBM16_MULTIPLIER:MBM_7 FMBM14_MULTIPLIER:MBM_5 FMBM12_MULTIPLIER:MBM_3 FMBM10_MULTIPLIER:MBM_1 \
              MITCHEL16_MULTIPLIER:MIT_7 MITCHEL14_MULTIPLIER:MIT_5 MITCHEL12_MULTIPLIER:MIT_3 \
              MITCHEL10_MULTIPLIER:MIT_1 BFLOAT:ACC_7; do
    g++ -w -O1 -fPIC -shared -std=c++14 -D${pair%%:*} -I"$ref/lut" \
        -o "$here/_ref/libref_model_${pair##*:}.so" "$here/ref_models.cc"
  done
  g++ -w -O1 -D__device__= -I"$ref/cuda" -o "$tmp/gen_lut_m11" "$here/gen_lut_m11.cc"
  "$tmp/gen_lut_m11" "$here/_ref/lut/MBM_11.bin"
  rm -rf "$tmp"
  echo "oracle/_ref built from $ref"
  # the reference's own GPU kernels and launchers, for the GPU tests (needs nvcc)
  bash "$here/build_ref_cuda.sh" "$ref"
else
  echo "no reference checkout at $ref: oracle/_ref not rebuilt"
fi
