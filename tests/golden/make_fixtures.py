"""Regenerates the committed golden fixtures.  Needs a reference checkout
(default: the directory "reference" beside this repository); run from the repository root:

    python tests/golden/make_fixtures.py [reference_dir]

What it writes, and where each comes from:

* ``tests/golden/lut/<MODEL>_<m>.bin`` — the nine small LUTs, produced by
  compiling and running the reference's own ``lut/lut_gen.cc`` (see
  ``oracle/build.sh``).  Their md5s equal those of the LUT files the
  reference ships.
* ``tests/golden/prim_kat.npz`` — operand bit patterns and the products the
  REFERENCE's ``cuda/AMsimulator.inl`` returns for them (compiled as host C++,
  ``oracle/ref_shim.cc``), for every LUT: every exponent class pair in
  {0,1,64,126,127,128,129,200,254,255}^2, both signs, seeded mantissas.
* ``tests/golden/direct_kat.npz`` — operand bit patterns and the products of the
  REFERENCE's direct 32-bit models (``cuda/FPmultMBM_fast32.inl``,
  ``cuda/Mitchell_32.inl``, compiled as host C++ by ``oracle/ref_shim.cc``).
* ``tests/golden/ops_kat.npz`` — small seeded conv / dense / matmul cases with
  the CPU oracle's outputs (reference GPU semantics), a regression pin for
  the oracle and a GPU-side known-answer test that needs no oracle build.
"""
import os
import shutil
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

SMALL_LUTS = ["ACC_7", "MBM_1", "MBM_3", "MBM_5", "MBM_7", "MIT_1", "MIT_3", "MIT_5", "MIT_7"]
EXP_CLASSES = [0, 1, 64, 126, 127, 128, 129, 200, 254, 255]


def prim_operands(seed: int):
    rng = np.random.default_rng(seed)
    at, bt = [], []
    for ea in EXP_CLASSES:
        for eb in EXP_CLASSES:
            for sa in (0, 1):
                for sb in (0, 1):
                    ma = rng.integers(0, 1 << 23, size=6, dtype=np.uint32)
                    mb = rng.integers(0, 1 << 23, size=6, dtype=np.uint32)
                    ma[0] = 0
                    mb[0] = 0
                    ma[1] = (1 << 23) - 1
                    mb[1] = (1 << 23) - 1
                    at.append((np.uint32(sa) << 31) | (np.uint32(ea) << 23) | ma)
                    bt.append((np.uint32(sb) << 31) | (np.uint32(eb) << 23) | mb)
    return np.concatenate(at).astype(np.uint32), np.concatenate(bt).astype(np.uint32)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")
    subprocess.check_call(["bash", os.path.join(ROOT, "oracle", "build.sh"), ref])
    from oracle.oracle import Oracle, RefPrimitive, load_lut

    gold = os.path.join(ROOT, "tests", "golden")
    os.makedirs(os.path.join(gold, "lut"), exist_ok=True)
    for name in SMALL_LUTS:
        shutil.copyfile(os.path.join(ROOT, "oracle", "_ref", "lut", name + ".bin"),
                        os.path.join(gold, "lut", name + ".bin"))

    refp = RefPrimitive()
    at, bt = prim_operands(1234)
    prim = {"at": at, "bt": bt}
    for name in SMALL_LUTS:
        lut, m = load_lut(os.path.join(gold, "lut", name + ".bin"))
        prim["out_" + name] = refp.mul_bits_array(at, bt, lut, m)
    np.savez_compressed(os.path.join(gold, "prim_kat.npz"), **prim)

    # direct 32-bit models: the reference's cuda/FPmultMBM_fast32.inl and cuda/Mitchell_32.inl as host code
    from oracle.oracle import DIRECT_MBM32, DIRECT_MIT32
    rng = np.random.default_rng(77)
    da = rng.integers(0, 1 << 32, size=20000, dtype=np.uint64).astype(np.uint32)
    db = rng.integers(0, 1 << 32, size=20000, dtype=np.uint64).astype(np.uint32)
    # keep most exponents near 127 so that results are ordinary numbers, plus the class grid above
    da[:16000] = (da[:16000] & np.uint32(0x807FFFFF)) | (rng.integers(100, 156, size=16000).astype(np.uint32) << np.uint32(23))
    db[:16000] = (db[:16000] & np.uint32(0x807FFFFF)) | (rng.integers(100, 156, size=16000).astype(np.uint32) << np.uint32(23))
    da = np.concatenate([da, at])
    db = np.concatenate([db, bt])
    np.savez_compressed(os.path.join(gold, "direct_kat.npz"), at=da, bt=db,
                        out_MBM32=refp.direct_mul_bits_array(da, db, DIRECT_MBM32),
                        out_MIT32=refp.direct_mul_bits_array(da, db, DIRECT_MIT32))

    o = Oracle.get()
    rng = np.random.default_rng(2024)
    ops = {}
    lut7, m7 = load_lut(os.path.join(gold, "lut", "MBM_7.bin"))
    lutm, mm = load_lut(os.path.join(gold, "lut", "MIT_5.bin"))
    # conv: SAME stride 1 and VALID stride 2, with ReLU-like zeros in x
    for tag, (n, h, w, c, kh, kw, k, s, pad, lut, m) in {
        "convA": (2, 9, 8, 8, 3, 3, 16, 1, "SAME", lut7, m7),
        "convB": (1, 11, 10, 4, 5, 3, 8, 2, "VALID", lutm, mm),
        "convC": (2, 7, 7, 3, 3, 3, 5, 2, "SAME", lut7, m7),
    }.items():
        g = o.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        x = rng.standard_normal((n, h, w, c)).astype(np.float32)
        x[x < -0.5] = 0.0
        wt = rng.standard_normal((kh, kw, c, k)).astype(np.float32)
        dy = rng.standard_normal((n, g.out_h, g.out_w, k)).astype(np.float32)
        ops[tag + "_geom"] = np.array([n, h, w, c, kh, kw, k, s, 1 if pad == "SAME" else 0], np.int32)
        ops[tag + "_x"], ops[tag + "_w"], ops[tag + "_dy"] = x, wt, dy
        ops[tag + "_y"] = o.conv2d_fwd(g, x, wt, lut, m)
        ops[tag + "_dw"] = o.conv2d_bwd_filter(g, x, dy, lut, m)
        ops[tag + "_dx"] = o.conv2d_bwd_input(g, wt, dy, lut, m)
    # dense
    x = rng.standard_normal((12, 37)).astype(np.float32)
    wt = rng.standard_normal((37, 19)).astype(np.float32)
    gy = rng.standard_normal((12, 19)).astype(np.float32)
    ops["dense_x"], ops["dense_w"], ops["dense_g"] = x, wt, gy
    ops["dense_y"] = o.dense_fwd(x, wt, lut7, m7)
    ops["dense_dw"] = o.dense_bwd_weight(x, gy, lut7, m7)
    ops["dense_dx"] = o.dense_bwd_input(wt, gy, lut7, m7)
    # batched matmul with broadcast
    a = rng.standard_normal((3, 10, 21)).astype(np.float32)
    b = rng.standard_normal((1, 21, 14)).astype(np.float32)
    ops["mm_a"], ops["mm_b"] = a, b
    ops["mm_c"] = o.matmul(a, b, lut7, m7)
    np.savez_compressed(os.path.join(gold, "ops_kat.npz"), **ops)
    print("fixtures written under", gold)


if __name__ == "__main__":
    main()
