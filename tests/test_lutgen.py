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
