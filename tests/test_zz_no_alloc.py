"""The filter gradient for hosts that cannot allocate device memory
(amsim_conv2d_bwd_filter_static): partial sums go to a buffer built into the
library instead of a caller-provided workspace.

Called through the C ABI, twice in a row with different inputs, and compared
bit for bit with amsim_conv2d_bwd_filter (same split plan, same summation
order, so the results must be identical).  The second call sees the buffer
exactly as the first one left it, which is the situation a long-running caller
is always in.  This file sorts last so that a run that stops at the first
failure has already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import lut_path

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _call(L, fn, lut, x, dy, dims, flags, workspace=None, stream=None, dw=None):
    n, h, w, c, kh, kw, k, oh, ow, sh, sw, pt, pl = dims
    if dw is None:
        dw = torch.full((kh, kw, c, k), float("nan"), device="cuda")
    args = [C.c_void_p(stream.cuda_stream) if stream is not None else None, lut.handle, C.c_void_p(x.data_ptr()),
            C.c_void_p(dy.data_ptr()), C.c_void_p(dw.data_ptr()), n, h, w, c, kh, kw, k, oh, ow, sh, sw, pt, pl]
    if workspace is not None:
        args += [C.c_void_p(workspace.data_ptr()) if workspace.numel() else None, workspace.numel()]
    rc = fn(*args, flags)
    torch.cuda.synchronize()
    return rc, dw


@pytest.mark.parametrize("flags", [0, 1])
def test_static_scratch_filter_grad_matches_workspace_variant(flags):
    assert torch.cuda.is_available()
    from approxtrain_b200 import _lib as L, ops
    lut = ops.get_lut(lut_path("MBM_7"), "cuda")
    from oracle.oracle import Oracle, load_lut
    oracle = Oracle.get()
    lut_bytes, m = load_lut(lut_path("MBM_7"))
    side = torch.cuda.Stream()
    # (n, h, w, c, kh, kw, k, stride, padding): all are split along the reduction in fast mode - the tiled
    # kernel twice, the one-chain-per-thread kernel of tiny outputs (LeNet-5's first filter), and a 1x1
    # convolution that runs with swapped operand roles (its scratch is the larger of two plans)
    for seed, (n, h, w, c, kh, kw, k, s, pad) in enumerate([(4, 16, 16, 32, 3, 3, 32, 1, "SAME"),
                                                            (8, 15, 15, 16, 3, 3, 24, 2, "VALID"),
                                                            (16, 28, 28, 1, 5, 5, 6, 1, "SAME"),
                                                            (4, 14, 14, 64, 1, 1, 256, 1, "VALID")]):
        oh, ow, pt, pl = ops.conv2d_geometry(h, w, kh, kw, s, s, pad)
        dims = (n, h, w, c, kh, kw, k, oh, ow, s, s, pt, pl)
        g = torch.Generator(device="cuda").manual_seed(100 + seed)
        x = torch.randn(n, h, w, c, device="cuda", generator=g).clamp_min(-0.3)
        dy = torch.randn(n, oh, ow, k, device="cuda", generator=g)
        need = L.lib.amsim_conv2d_bwd_filter_workspace(n, h, w, c, kh, kw, k, oh, ow, flags)
        if flags == 0 and seed == 0:
            assert 0 < need <= L.STATIC_SCRATCH_BYTES  # the split path really runs through the built-in buffer
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc0, want = _call(L, L.lib.amsim_conv2d_bwd_filter, lut, x, dy, dims, flags, workspace=ws)
        assert rc0 == 0, L.lib.amsim_last_error()
        out = torch.full((kh, kw, c, k), float("nan"), device="cuda")   # allocated before the memory reading below
        # the first call on a device looks up the buffer's address (one-time set-up, documented in the header)
        rc, _ = _call(L, L.lib.amsim_conv2d_bwd_filter_static, lut, x, dy, dims, flags, dw=out)
        assert rc == 0, L.lib.amsim_last_error()
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for attempt in range(2):  # two calls in a row share the buffer; the second one on another stream
            st = side if attempt else None
            if st is not None:
                st.wait_stream(torch.cuda.current_stream())
            rc, got = _call(L, L.lib.amsim_conv2d_bwd_filter_static, lut, x, dy, dims, flags, stream=st, dw=out)
            assert rc == 0, L.lib.amsim_last_error()
            assert np.array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32)), (seed, attempt)
            out.fill_(float("nan"))
            torch.cuda.synchronize()
        # the entry point took no device memory: what the driver reports as free is unchanged
        # (torch's own allocations above come from its cache and were made before the first reading)
        assert torch.cuda.mem_get_info()[0] == free_before, seed
        # and against the CPU oracle: bit-identical in deterministic mode, within the bar in fast mode
        geo = oracle.geometry(n, h, w, c, kh, kw, k, s, s, pad)
        ref = oracle.conv2d_bwd_filter(geo, x.cpu().numpy(), dy.cpu().numpy(), lut_bytes, m)
        got_np = want.cpu().numpy()
        if flags == 1:
            assert np.array_equal(got_np.view(np.uint32), ref.view(np.uint32)), seed
        else:
            err = np.linalg.norm((got_np.astype(np.float64) - ref).ravel()) / np.linalg.norm(ref.astype(np.float64).ravel())
            assert err <= 1e-5, (seed, err)


def test_static_scratch_rejects_shapes_beyond_its_size():
    from approxtrain_b200 import _lib as L, ops
    lut = ops.get_lut(lut_path("MBM_7"), "cuda")
    # 3x3x64x64 filters over 64x56x56 outputs: the split plan keeps ~13 MB of partial sums, the buffer holds 8 MiB
    n, h, w, c, kh, kw, k = 64, 56, 56, 64, 3, 3, 64
    need = L.lib.amsim_conv2d_bwd_filter_workspace(n, h, w, c, kh, kw, k, h, w, 0)
    assert need > L.STATIC_SCRATCH_BYTES
    rc = L.lib.amsim_conv2d_bwd_filter_static(None, lut.handle, None, None, None, n, h, w, c, kh, kw, k, h, w,
                                              1, 1, 1, 1, 0)
    assert rc == L.ERR_WORKSPACE
    msg = L.lib.amsim_last_error().decode()
    assert "built-in buffer" in msg and str(L.STATIC_SCRATCH_BYTES) in msg
