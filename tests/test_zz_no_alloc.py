"""GPU test of xcorr_one_to_one_noalloc_f32, the entry point for callers that cannot allocate
device memory (a real-time loop, a plug-in whose host forbids cudaMalloc after start-up, a
process whose memory pool another runtime owns).  Its partial results live in an array built
into the library instead of a caller-provided workspace.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.  The test passes alone in a fresh process and after the other tests.

Checked here: through the C ABI, on two calls in a row with different inputs (the second call
finds the first call's partial results in the shared array), the result equals the existing
workspace entry point's within the tolerance of the parity tests (1e-5 of the largest result
value; the two may use different numbers of row slices), sizes beyond the built-in array are
refused with a clear message, and NULL pointers are refused.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def _existing_entry_point(xc, left, right):
    rows, cols = left.shape[1:]
    hints = xc.make_hints(kernel="tile", combine="workspace")
    wsb = xc.workspace_bytes("one_to_one", rows, cols, 1, 1, hints)
    dl, dr = torch.from_numpy(left).cuda(), torch.from_numpy(right).cuda()
    out = torch.full((1, 2 * rows - 1, 2 * cols - 1), float("nan"), dtype=torch.float32, device="cuda")
    ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device="cuda")
    xc.run_device("one_to_one", dl.data_ptr(), dr.data_ptr(), out.data_ptr(), rows, cols, 1, 1, hints,
                  ws.data_ptr(), wsb, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def _no_alloc_entry_point(xc, left, right):
    rows, cols = left.shape[1:]
    dl, dr = torch.from_numpy(left).cuda(), torch.from_numpy(right).cuda()
    out = torch.full((1, 2 * rows - 1, 2 * cols - 1), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    xc.check(xc.lib().xcorr_one_to_one_noalloc_f32(dl.data_ptr(), dr.data_ptr(), out.data_ptr(), rows, cols,
                                                   torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return out.cpu().numpy()


def test_no_alloc_entry_point_matches_workspace_entry_point_twice(xc):
    rng = np.random.default_rng(2024)
    # first call large (fills much of the built-in array), second call small and different:
    # stale partial results of the first call must not leak into the second
    for rows, cols in ((256, 256), (48, 80), (256, 256)):
        left = rng.random((1, rows, cols), dtype=np.float32)
        right = rng.random((1, rows, cols), dtype=np.float32)
        want = _existing_entry_point(xc, left, right)
        got = _no_alloc_entry_point(xc, left, right)
        assert "combine=workspace" in xc.last_launch()
        assert not np.isnan(got).any()
        err = np.abs(got.astype(np.float64) - want).max() / np.abs(want).max()
        assert err <= REL_TOL, (rows, cols, err)


def test_no_alloc_entry_point_rejects_what_does_not_fit(xc):
    lib = xc.lib()
    assert lib.xcorr_noalloc_scratch_bytes() == 32 * 1024 * 1024
    buf = torch.zeros(16, device="cuda")
    p = buf.data_ptr()
    # (2*2000-1)^2 floats = 64 MB > 32 MiB: refused before anything is launched or read
    assert lib.xcorr_one_to_one_noalloc_f32(p, p, p, 2000, 2000, None) == 6
    msg = lib.xcorr_last_error_string().decode()
    assert "33554432" in msg and "built-in scratch" in msg
    assert lib.xcorr_one_to_one_noalloc_f32(None, p, p, 16, 16, None) == 1
    assert lib.xcorr_one_to_one_noalloc_f32(p, p, p, 0, 16, None) == 2
