"""GPU test of xcorr_one_to_one_noalloc_f32, the entry point for callers that cannot allocate
device memory (a real-time loop, a plug-in whose host forbids cudaMalloc after start-up, a
process whose memory pool another runtime owns).  Its partial results live in an array built
into the library instead of a caller-provided workspace.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.  The test passes alone in a fresh process and after the other tests.

Checked here, through the C ABI: on calls in a row with different inputs (a later call finds an
earlier call's partial results in the shared array) the result equals the existing workspace entry
point's within the tolerance of the parity tests (1e-5 of the largest result value; the two may
use different numbers of row slices); small cases also equal the CPU oracle; the sizes where the
array no longer holds enough row slices (from about 464 x 464) still work, by adding the slices
atomically, and are checked against the cuFFT path (2e-5: two float paths, neither exact); sizes
beyond the array are refused with a message that names the limit; NULL pointers are refused.
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


def test_no_alloc_entry_point_against_the_oracle(xc, oracle):
    """Small and ragged inputs (48 x 80 takes the bulk-copy staging, 33 x 37 the element-wise one,
    5 x 3 a single slice) against the CPU oracle, twice each."""
    rng = np.random.default_rng(7)
    for rows, cols in ((48, 80), (33, 37), (5, 3), (96, 96), (33, 37)):
        left = rng.random((1, rows, cols), dtype=np.float32)
        right = rng.random((1, rows, cols), dtype=np.float32)
        want = oracle.run("one_to_one", left, right, acc64=True)
        got = _no_alloc_entry_point(xc, left, right)
        assert not np.isnan(got).any(), xc.last_launch()
        err = np.abs(got.astype(np.float64) - want).max() / np.abs(want).max()
        assert err <= REL_TOL, (rows, cols, err, xc.last_launch())


def _fft_path(xc, left, right):
    rows, cols = left.shape[1:]
    wsb = xc.fft_workspace_bytes("one_to_one", rows, cols, 1, 1)
    ws = torch.empty(wsb + 256, dtype=torch.uint8, device="cuda")
    base = (ws.data_ptr() + 255) // 256 * 256
    dl, dr = torch.from_numpy(left).cuda(), torch.from_numpy(right).cuda()
    out = torch.empty((1, 2 * rows - 1, 2 * cols - 1), dtype=torch.float32, device="cuda")
    xc.run_fft_device("one_to_one", dl.data_ptr(), dr.data_ptr(), out.data_ptr(), rows, cols, 1, 1, "normalized",
                      base, wsb, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("rows,cols", [(448, 448), (464, 464), (512, 512), (1023, 1023), (256, 1024), (1024, 256)])
def test_no_alloc_entry_point_at_and_beyond_the_slice_limit(xc, rows, cols):
    """448 x 448 is the largest square whose row slices fit both the array and one SM's shared
    memory; from there on the call adds its slices atomically instead.  Every size up to the
    documented limit gives the right result (against the cuFFT path; the CPU oracle would take
    minutes at these sizes)."""
    rng = np.random.default_rng(rows * 7 + cols)
    left = rng.random((1, rows, cols), dtype=np.float32)
    right = rng.random((1, rows, cols), dtype=np.float32)
    got = _no_alloc_entry_point(xc, left, right)
    plan = xc.last_launch()
    assert "combine=workspace" in plan or "combine=atomic" in plan, plan
    if rows == 448:
        assert "combine=workspace" in plan, plan
    if rows >= 512 and cols >= 512:
        assert "combine=atomic" in plan, plan
    assert not np.isnan(got).any(), plan
    want = _fft_path(xc, left, right)
    err = np.abs(got.astype(np.float64) - want).max() / np.abs(want).max()
    assert err <= 2e-5, (rows, cols, err, plan)


def test_no_alloc_entry_point_rejects_what_does_not_fit(xc):
    lib = xc.lib()
    assert lib.xcorr_noalloc_scratch_bytes() == 32 * 1024 * 1024
    buf = torch.zeros(16, device="cuda")
    p = buf.data_ptr()
    # (2*2000-1)^2 floats = 64 MB > 32 MiB: refused before anything is launched or read
    assert lib.xcorr_one_to_one_noalloc_f32(p, p, p, 2000, 2000, None) == 6
    msg = lib.xcorr_last_error_string().decode()
    assert "33554432" in msg and "built-in scratch" in msg and "1448 x 1448" in msg
    # the largest square the array takes is accepted as a size (1449 is not)
    assert lib.xcorr_one_to_one_noalloc_f32(p, p, p, 1449, 1449, None) == 6
    assert lib.xcorr_one_to_one_noalloc_f32(None, p, p, 16, 16, None) == 1
    assert lib.xcorr_one_to_one_noalloc_f32(p, p, p, 0, 16, None) == 2
