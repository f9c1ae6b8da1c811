"""Host-side sanitizer runs (stand-ins for compute-sanitizer on the device side).

* The CPU oracle, every entry point, on small ragged shapes under
  -fsanitize=address,undefined (gcc): a few seconds, always run.
* The C ABI's host code (argument checking, LUT loading, launch planning) under the same
  sanitizers: needs a two-minute nvcc build, so it only runs when AMSIM_SANITIZE_ABI=1.
  It drives the error paths that need no GPU (bad names, short files, NULL pointers, sizes).
"""
import ctypes
import os
import shutil
import subprocess
import sys

import pytest

from conftest import ROOT, lut_path

SAN = ["-fsanitize=address,undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer", "-g"]


def test_oracle_under_asan_ubsan(tmp_path):
    exe = tmp_path / "sanitize_oracle"
    subprocess.check_call(["gcc", "-std=c11", "-O1", *SAN, "-ffp-contract=off", "-fopenmp", "-I", os.path.join(ROOT, "oracle"),
                           "-o", str(exe), os.path.join(ROOT, "tests", "sanitize_oracle_main.c"),
                           os.path.join(ROOT, "oracle", "amsim_oracle.c"), "-lm"])
    for name in ("MBM_7", "MIT_5", "MBM_1"):
        # (LeakSanitizer needs ptrace, which containers often deny; leaks are not what this run is after)
        out = subprocess.run([str(exe), lut_path(name)], capture_output=True, text=True, timeout=300,
                             env=dict(os.environ, OMP_NUM_THREADS="2", ASAN_OPTIONS="detect_leaks=0"))
        assert out.returncode == 0, out.stderr[-3000:]
        assert out.stdout.startswith("checksum")


ABI_DRIVER = r'''
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "amsim.h"
#define EXPECT(cond) do { if (!(cond)) { printf("FAILED line %d: %s (%s)\n", __LINE__, #cond, amsim_last_error()); return 1; } } while (0)
int main(int argc, char** argv) {
  amsim_lut* h = NULL;
  EXPECT(amsim_lut_open(NULL, 0, &h) == AMSIM_ERR_INVALID);
  EXPECT(amsim_lut_open("", 0, &h) == AMSIM_ERR_LUT_NAME);
  EXPECT(amsim_lut_open("nounderscore.bin", 0, &h) == AMSIM_ERR_LUT_NAME);
  EXPECT(amsim_lut_open("MBM_12.bin", 0, &h) == AMSIM_ERR_LUT_NAME);
  EXPECT(amsim_lut_open("/nonexistent/MBM_7.bin", 0, &h) == AMSIM_ERR_LUT_IO);
  EXPECT(amsim_lut_open(argv[1], 0, &h) == AMSIM_ERR_LUT_SIZE);   /* a short file named MBM_7.bin */
  EXPECT(amsim_lut_open("direct:NOPE", 0, &h) == AMSIM_ERR_LUT_NAME);
  EXPECT(amsim_lut_info(NULL, NULL, NULL, NULL, NULL, NULL) == AMSIM_ERR_INVALID);
  EXPECT(amsim_lut_close(NULL) == AMSIM_OK);
  EXPECT(amsim_conv2d_fwd(NULL, NULL, NULL, NULL, NULL, 1, 8, 8, 4, 3, 3, 4, 8, 8, 1, 1, 1, 1, 0) == AMSIM_ERR_INVALID);
  EXPECT(amsim_dense_fwd(NULL, NULL, NULL, NULL, NULL, 1, 1, 1, 0) == AMSIM_ERR_INVALID);
  EXPECT(amsim_matmul(NULL, NULL, NULL, NULL, NULL, 0, 0, 1, 1, 1, 1, 0) == AMSIM_ERR_INVALID);
  int oh, ow, pt, pl;
  EXPECT(amsim_conv2d_geometry(224, 224, 7, 7, 2, 2, 1, &oh, &ow, &pt, &pl) == AMSIM_OK && oh == 112 && pt == 2);
  EXPECT(amsim_conv2d_geometry(3, 3, 5, 5, 1, 1, 0, &oh, &ow, &pt, &pl) == AMSIM_ERR_INVALID);
  EXPECT(amsim_conv2d_geometry(0, 3, 5, 5, 1, 1, 0, &oh, &ow, &pt, &pl) == AMSIM_ERR_INVALID);
  /* plans over the whole range of sizes, including ones whose products overflow 32 bits */
  size_t acc = 0;
  const int dims[] = {0, 1, 3, 64, 147, 576, 4608, 65536, 1 << 20, 0x7fffffff};
  for (unsigned a = 0; a < sizeof(dims) / 4; ++a)
    for (unsigned b = 0; b < sizeof(dims) / 4; ++b)
      for (unsigned flags = 0; flags < 4; ++flags) {
        acc += amsim_conv2d_bwd_filter_workspace(dims[a], dims[b], dims[b], dims[a], 3, 3, dims[b], dims[b], dims[b], flags);
        acc += amsim_conv2d_bwd_filter_workspace(dims[b], 7, 7, dims[a], 1, 1, dims[a], 7, 7, flags);
        acc += amsim_dense_bwd_weight_workspace(dims[a], dims[b], dims[a], flags);
      }
  for (uint32_t d = 1; d < 70000; d += 7)
    for (uint32_t n = 0; n < 0x7fffffffu - 70000u * 300u; n += 70000u * 300u + d) EXPECT(amsim_debug_fastdiv(n, d) == n / d);
  amsim_debug_reload_env();
  printf("abi host paths ok %zu %s\n", acc, amsim_version());
  return 0;
}
'''


@pytest.mark.skipif(os.environ.get("AMSIM_SANITIZE_ABI") != "1", reason="two-minute nvcc build: set AMSIM_SANITIZE_ABI=1")
def test_abi_host_code_under_asan_ubsan(tmp_path):
    nvcc = shutil.which("nvcc")
    if nvcc is None:
        pytest.skip("no nvcc")
    lib = tmp_path / "libamsim_san.so"
    host = ["-fPIC", "-fsanitize=address", "-fsanitize=undefined", "-fno-sanitize-recover=all", "-fno-omit-frame-pointer"]
    xc = [a for f in host for a in ("-Xcompiler", f)]     # one by one: nvcc splits -Xcompiler arguments at commas
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "-shared", *xc,
                           "-Xlinker", "-lasan", "-Xlinker", "-lubsan", "-o", str(lib),
                           os.path.join(ROOT, "approxtrain_b200", "csrc", "amsim.cu")])
    src = tmp_path / "abi_san.c"
    src.write_text(ABI_DRIVER)
    short = tmp_path / "MBM_7.bin"
    short.write_bytes(b"\0" * 100)
    exe = tmp_path / "abi_san"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["gcc", "-std=c99", "-O1", *SAN, "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src),
                           str(lib), "-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + str(tmp_path),
                           "-Wl,-rpath," + os.path.join(cuda, "lib64")])
    out = subprocess.run([str(exe), str(short)], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=0:protect_shadow_gap=0"))
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert "abi host paths ok" in out.stdout
