"""LUT generator: regenerating the reference's nine LUTs from its own functional
models (built as host libraries under oracle/_ref) must reproduce the shipped
files byte for byte; a numpy model checks the vectorised path without _ref."""
import hashlib
import os

import numpy as np
import pytest

from conftest import ROOT, SMALL_LUTS, lut_path
from test_oracle import REF_LUT_MD5


def test_exact_bf16_model_reproduces_acc7():
    """ACC_7 is the bfloat16 multiplier: the product of the two truncated inputs, truncated to bf16."""
    from approxtrain_b200 import lutgen

    def bf16_mul(a, b):
        c = (a.astype(np.float32) * b.astype(np.float32)).astype(np.float32)
        return (c.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
    got = lutgen.generate(bf16_mul, 7)
    want = np.fromfile(lut_path("ACC_7"), dtype=np.uint8)
    # the reference's bfloat model rounds; allow it to differ from plain truncation only in the last mantissa bit
    assert got.shape == want.shape
    assert (np.abs((got & 0x7F).astype(int) - (want & 0x7F).astype(int)) <= 1).mean() > 0.99


@pytest.mark.parametrize("name", SMALL_LUTS)
def test_regenerates_reference_luts_from_its_c_models(name, tmp_path):
    from approxtrain_b200 import lutgen
    lib = os.path.join(ROOT, "oracle", "_ref", f"libref_model_{name}.so")
    if not os.path.exists(lib):
        pytest.skip("oracle/_ref not built (no reference checkout on this machine)")
    m = int(name.split("_")[1])
    out = tmp_path / f"{name}.bin"
    lutgen.write(str(out), lutgen.c_model(lib, "ref_model_mul"), m)
    assert hashlib.md5(out.read_bytes()).hexdigest() == REF_LUT_MD5[name]


def test_file_name_must_carry_the_width(tmp_path):
    from approxtrain_b200 import lutgen
    with pytest.raises(ValueError):
        lutgen.write(str(tmp_path / "X_5.bin"), lambda a, b: a * b, 7)
    with pytest.raises(ValueError):
        lutgen.generate(lambda a, b: a * b, 12)


@pytest.mark.parametrize("m", [5, 9, 11])
def test_16_bit_entries_keep_the_products_leading_mantissa_bits(oracle, m, tmp_path):
    """Format extension: a file of 2 * 2^(2m) bytes under the usual name holds 16-bit
    little-endian entries, carry << 15 | top 15 mantissa bits.  Generated from the 32-bit
    minimally-biased model, the table reproduces model(trunc_m(a), trunc_m(b)) to 15
    mantissa bits for every operand pair with in-range exponents, where the byte format
    at m > 7 cannot (a byte holds 7 of the m bits it is asked to keep)."""
    from approxtrain_b200 import lutgen
    from oracle.oracle import DIRECT_MBM32, NO_LUT, WIDE_ENTRIES, load_lut

    def mbm32(a, b):
        return oracle.mul(a, b, NO_LUT, DIRECT_MBM32)
    path = str(tmp_path / f"MBMW_{m}.bin")
    lutgen.write(path, mbm32, m, entry_bits=16)
    assert os.path.getsize(path) == 2 << (2 * m)
    lut, mw = load_lut(path)
    assert mw == m | WIDE_ENTRIES
    rng = np.random.default_rng(m)
    n = 200000
    a = (rng.standard_normal(n) * 4).astype(np.float32)
    b = (rng.standard_normal(n) * 0.3).astype(np.float32)
    keep = np.uint32((0xFFFFFFFF << (23 - m)) & 0xFFFFFFFF)
    at, bt = a.view(np.uint32) & keep, b.view(np.uint32) & keep
    got = oracle.mul(at.view(np.float32), bt.view(np.float32), lut, mw).view(np.uint32)
    want = mbm32(at.view(np.float32), bt.view(np.float32)).view(np.uint32) & np.uint32(0xFFFFFF00)
    assert np.array_equal(got, want)
    # operands with more mantissa bits than m are truncated first, like in the byte format
    got_full = oracle.mul(a, b, lut, mw).view(np.uint32)
    assert np.array_equal(got_full, want)
    if m > 7:
        lut8 = lutgen.generate(mbm32, m)
        got8 = oracle.mul(a, b, lut8, m).astype(np.float64)
        ref = mbm32(at.view(np.float32), bt.view(np.float32)).astype(np.float64)
        err8 = np.abs(got8 - ref) / np.abs(ref)
        err16 = np.abs(got_full.view(np.float32).astype(np.float64) - ref) / np.abs(ref)
        assert err16.max() < 2.0 ** -14 and err8.mean() > 100 * err16.mean()
