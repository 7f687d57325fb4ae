"""Python binding (ctypes) of the B200 direct cross-correlation library.

The product is ``lib/libxcorr.so`` (C ABI in ``include/xcorr.h``) and the ``bin/cross``
host program; this module only loads the library for tests, the benchmark and scripts.
There is no CPU fallback: every call goes to the CUDA library and raises if it is missing.

The directory name contains a hyphen, so import it by path::

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location(
        "jpdc23_artifact_b200", "<repo>/jpdc23-artifact_b200/__init__.py")
    xc = importlib.util.module_from_spec(spec); sys.modules[spec.name] = xc
    spec.loader.exec_module(xc)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "lib", "libxcorr.so")
CROSS_PATH = os.path.join(PKG_DIR, "bin", "cross")
HEADER_PATH = os.path.join(os.path.dirname(PKG_DIR), "include", "xcorr.h")

MODES = {"one_to_one": 0, "one_to_many": 1, "n_to_mn": 2, "n_to_m": 3}
KERNELS = {"auto": 0, "tile": 1, "overlap_wise": 2, "warp_per_overlap": 3, "fft": 4, "warp_staged": 5}
ROW_SPLIT = {"none": 0, "rectangle": 1, "triangle": 2}
COMBINE = {"auto": 0, "store": 1, "atomic": 2, "workspace": 3}


class XcorrError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"xcorr status {status} ({what}): {detail}")
        self.status = status


class Hints(C.Structure):
    """Mirror of ``xcorr_hints`` (include/xcorr.h)."""
    _fields_ = [
        ("kernel", C.c_int32), ("combine", C.c_int32), ("overlap_rows", C.c_int32),
        ("class_lanes", C.c_int32), ("warps_x", C.c_int32), ("warps_y", C.c_int32),
        ("row_slices", C.c_int32), ("block_threads", C.c_int32), ("schedule", C.c_int32),
        ("host_chunks", C.c_int32), ("reproducible", C.c_int32),
        ("rows_per_warp", C.c_int32), ("row_split", C.c_int32), ("staged_rows", C.c_int32),
        ("staged_cols", C.c_int32), ("staged_rights", C.c_int32), ("staged_column_groups", C.c_int32),
        ("staged_warp_rows", C.c_int32), ("fused_rows", C.c_int32), ("reserved", C.c_int32 * 1),
    ]


class HostJob(C.Structure):
    """Mirror of ``xcorr_host_job`` (include/xcorr.h)."""
    _fields_ = [
        ("mode", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32),
        ("n_left", C.c_uint32), ("n_right", C.c_uint32),
        ("h_left", C.c_void_p), ("h_right", C.c_void_p), ("h_out", C.c_void_p),
        ("hints", C.POINTER(Hints)),
    ]


def make_hints(kernel="auto", combine="auto", overlap_rows=0, class_lanes=0, warps_x=0, warps_y=0,
               row_slices=0, block_threads=0, schedule=0, host_chunks=0, reproducible=0,
               rows_per_warp=0, row_split="none", staged_rows=0, staged_cols=0, staged_rights=0,
               staged_column_groups=0, staged_warp_rows=0, fused_rows=0) -> Hints:
    h = Hints()
    h.kernel = KERNELS[kernel] if isinstance(kernel, str) else int(kernel)
    h.combine = COMBINE[combine] if isinstance(combine, str) else int(combine)
    h.overlap_rows, h.class_lanes = overlap_rows, class_lanes
    h.warps_x, h.warps_y, h.row_slices, h.block_threads = warps_x, warps_y, row_slices, block_threads
    h.schedule = schedule
    h.host_chunks = host_chunks
    h.reproducible = reproducible
    h.rows_per_warp = rows_per_warp
    h.row_split = ROW_SPLIT[row_split] if isinstance(row_split, str) else int(row_split)
    h.staged_rows, h.staged_cols, h.staged_rights = staged_rows, staged_cols, staged_rights
    h.staged_column_groups, h.staged_warp_rows = staged_column_groups, staged_warp_rows
    h.fused_rows = fused_rows
    return h


def build(verbose: bool = False) -> None:
    """Compile lib/libxcorr.so and bin/cross for sm_100a (nvcc cross-compiles without a GPU)."""
    subprocess.run(["make", "-C", PKG_DIR, "all"], check=True,
                   stdout=None if verbose else subprocess.DEVNULL)


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `make -C {PKG_DIR}` (there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    u32, i32, vp, sz = C.c_uint32, C.c_int32, C.c_void_p, C.c_size_t
    hp = C.POINTER(Hints)
    L.xcorr_run_f32.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, hp, vp, sz, vp]
    L.xcorr_one_to_one_f32.argtypes = [vp, vp, vp, u32, u32, hp, vp, sz, vp]
    L.xcorr_one_to_many_f32.argtypes = [vp, vp, vp, u32, u32, u32, hp, vp, sz, vp]
    L.xcorr_n_to_mn_f32.argtypes = [vp, vp, vp, u32, u32, u32, u32, hp, vp, sz, vp]
    L.xcorr_n_to_m_f32.argtypes = [vp, vp, vp, u32, u32, u32, u32, hp, vp, sz, vp]
    L.xcorr_one_to_one_noalloc_f32.argtypes = [vp, vp, vp, u32, u32, vp]
    L.xcorr_noalloc_scratch_bytes.argtypes = []
    L.xcorr_noalloc_scratch_bytes.restype = sz
    L.xcorr_workspace_bytes.argtypes = [i32, u32, u32, u32, u32, hp]
    L.xcorr_workspace_bytes.restype = sz
    L.xcorr_describe_plan.argtypes = [i32, u32, u32, u32, u32, hp, C.c_char_p, sz]
    L.xcorr_describe_plan.restype = i32
    L.xcorr_num_results.argtypes = [i32, u32, u32]
    L.xcorr_num_results.restype = C.c_uint64
    L.xcorr_validate_input_size.argtypes = [i32, u32, u32, u32, u32]
    L.xcorr_validate_input_size.restype = i32
    L.xcorr_run_host_f32.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, hp, i32]
    L.xcorr_run_f64.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, vp]
    L.xcorr_run_host_f64.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, i32]
    L.xcorr_run_host_batch_f32.argtypes = [C.POINTER(HostJob), i32, i32]
    L.xcorr_run_host_sharded_f32.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, hp,
                                             C.POINTER(i32), i32]
    L.xcorr_shard_range.argtypes = [u32, i32, i32, C.POINTER(u32), C.POINTER(u32)]
    L.xcorr_shard_range.restype = None
    L.xcorr_release_host_cache.argtypes = []
    L.xcorr_release_host_cache.restype = None
    L.xcorr_n_to_mn_reorder_f32.argtypes = [vp, vp, u32, u32, sz, i32]
    for name in ("xcorr_last_launch_string", "xcorr_last_error_string"):
        getattr(L, name).argtypes = []
        getattr(L, name).restype = C.c_char_p
    L.xcorr_status_string.argtypes = [i32]
    L.xcorr_status_string.restype = C.c_char_p
    L.xcorr_launch_count.argtypes = []
    L.xcorr_launch_count.restype = C.c_uint64
    L.xcorr_reset_launch_count.argtypes = []
    L.xcorr_reset_launch_count.restype = None
    L.xcorr_ffma_peak_probe.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_double), vp]
    L.xcorr_dfma_peak_probe.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_double), vp]
    L.xcorr_fft_workspace_bytes.argtypes = [i32, u32, u32, u32, u32, i32]
    L.xcorr_fft_workspace_bytes.restype = sz
    L.xcorr_fft_f32.argtypes = [i32, vp, vp, vp, u32, u32, u32, u32, i32, vp, sz, vp]
    L.xcorr_check_device.argtypes = []
    L.xcorr_debug_stage_wait.argtypes = [u32, u32]
    L.xcorr_debug_stage_wait.restype = None
    L.xcorr_fft_release_plans.argtypes = []
    L.xcorr_fft_release_plans.restype = None
    _lib = L
    return L


def check(status: int) -> None:
    if status != 0:
        L = lib()
        raise XcorrError(status, L.xcorr_status_string(status).decode(),
                         L.xcorr_last_error_string().decode())


def _mode(mode) -> int:
    return MODES[mode] if isinstance(mode, str) else int(mode)


def out_shape(mode, rows: int, cols: int, n_left: int, n_right: int):
    n = int(lib().xcorr_num_results(_mode(mode), n_left, n_right))
    return (n, 2 * rows - 1, 2 * cols - 1)


def shard_range(units: int, parts: int, index: int):
    first, count = C.c_uint32(0), C.c_uint32(0)
    lib().xcorr_shard_range(units, parts, index, C.byref(first), C.byref(count))
    return first.value, count.value


def workspace_bytes(mode, rows, cols, n_left, n_right, hints: Hints | None = None) -> int:
    return int(lib().xcorr_workspace_bytes(_mode(mode), rows, cols, n_left, n_right,
                                           C.byref(hints) if hints is not None else None))


def describe_plan(mode, rows, cols, n_left, n_right, hints: Hints | None = None) -> str:
    buf = C.create_string_buffer(1024)
    check(lib().xcorr_describe_plan(_mode(mode), rows, cols, n_left, n_right,
                                    C.byref(hints) if hints is not None else None, buf, len(buf)))
    return buf.value.decode()


def run_device(mode, d_left: int, d_right: int, d_out: int, rows: int, cols: int, n_left: int,
               n_right: int, hints: Hints | None = None, d_workspace: int = 0,
               workspace_bytes_: int = 0, stream: int = 0) -> None:
    """Asynchronous launch on raw device addresses (ints), e.g. torch ``tensor.data_ptr()``."""
    check(lib().xcorr_run_f32(_mode(mode), d_left, d_right, d_out, rows, cols, n_left, n_right,
                              C.byref(hints) if hints is not None else None,
                              d_workspace or None, workspace_bytes_, stream or None))


def check_device() -> None:
    """Synchronise and raise if a launch failed or a bounded device-side wait gave up."""
    check(lib().xcorr_check_device())


FFT_LAYOUTS = {"normalized": 0, "raw": 1}


def fft_workspace_bytes(mode, rows, cols, n_left, n_right, layout="normalized") -> int:
    return int(lib().xcorr_fft_workspace_bytes(_mode(mode), rows, cols, n_left, n_right, FFT_LAYOUTS[layout]))


def fft_out_shape(mode, rows, cols, n_left, n_right, layout="normalized"):
    n = int(lib().xcorr_num_results(_mode(mode), n_left, n_right))
    return (n, 2 * rows - 1, 2 * cols - 1) if layout == "normalized" else (n, 2 * rows, 2 * cols)


def run_fft_device(mode, d_left: int, d_right: int, d_out: int, rows: int, cols: int, n_left: int,
                   n_right: int, layout="normalized", d_workspace: int = 0, workspace_bytes_: int = 0,
                   stream: int = 0) -> None:
    """The cuFFT path on raw device addresses (asynchronous).  ``layout`` "normalized" gives the
    direct path's result layout, "raw" the 2*rows x 2*cols unnormalised inverse transforms."""
    check(lib().xcorr_fft_f32(_mode(mode), d_left, d_right, d_out, rows, cols, n_left, n_right,
                              FFT_LAYOUTS[layout], d_workspace or None, workspace_bytes_, stream or None))


def run_host(mode, left: np.ndarray, right: np.ndarray, hints: Hints | None = None, device: int = 0,
             devices: list[int] | None = None, out: np.ndarray | None = None) -> np.ndarray:
    """Host arrays in, host result out (H2D, kernel, D2H).  ``devices`` shards over GPUs.
    n_to_mn uses GROUPED order (right / result l*m + t belongs to left l)."""
    left = np.ascontiguousarray(left, np.float32)
    right = np.ascontiguousarray(right, np.float32)
    if left.ndim == 2:
        left = left[None]
    if right.ndim == 2:
        right = right[None]
    nl, rows, cols = left.shape
    nr = right.shape[0]
    if right.shape[1:] != (rows, cols):
        raise ValueError("left and right matrices must have the same size")
    shape = out_shape(mode, rows, cols, nl, nr)
    if shape[0] == 0:
        check(2)
    if out is None:
        out = np.empty(shape, np.float32)
    hp = C.byref(hints) if hints is not None else None
    if devices is None:
        check(lib().xcorr_run_host_f32(_mode(mode), left.ctypes.data, right.ctypes.data,
                                       out.ctypes.data, rows, cols, nl, nr, hp, device))
    else:
        arr = (C.c_int32 * len(devices))(*devices)
        check(lib().xcorr_run_host_sharded_f32(_mode(mode), left.ctypes.data, right.ctypes.data,
                                               out.ctypes.data, rows, cols, nl, nr, hp, arr,
                                               len(devices)))
    return out


def run_device_f64(mode, left_ptr, right_ptr, out_ptr, rows, cols, n_left, n_right, stream=0) -> None:
    """``xcorr_run_f64`` on device pointers (float64, same layouts as the float entry points)."""
    check(lib().xcorr_run_f64(_mode(mode), left_ptr, right_ptr, out_ptr, rows, cols, n_left, n_right, stream))


def run_host_f64(mode, left: np.ndarray, right: np.ndarray, device: int = 0) -> np.ndarray:
    """Double precision, host arrays in, host result out (``xcorr_run_host_f64``)."""
    left = np.ascontiguousarray(left, np.float64)
    right = np.ascontiguousarray(right, np.float64)
    if left.ndim == 2:
        left = left[None]
    if right.ndim == 2:
        right = right[None]
    nl, rows, cols = left.shape
    nr = right.shape[0]
    if right.shape[1:] != (rows, cols):
        raise ValueError("left and right matrices must have the same size")
    shape = out_shape(mode, rows, cols, nl, nr)
    if shape[0] == 0:
        check(2)
    out = np.empty(shape, np.float64)
    check(lib().xcorr_run_host_f64(_mode(mode), left.ctypes.data, right.ctypes.data, out.ctypes.data,
                                   rows, cols, nl, nr, device))
    return out


def run_host_batch(jobs, device: int = 0) -> list[np.ndarray]:
    """Several problems in one call (``xcorr_run_host_batch_f32``): ``jobs`` is a list of
    ``(mode, left, right)``, ``(mode, left, right, hints)`` or ``(mode, left, right, hints, out)``;
    returns the results in order.  Arrays are used in place when they are contiguous float32
    (so page-locked buffers stay page-locked)."""
    n = len(jobs)
    arr = (HostJob * max(n, 1))()
    keep, outs = [], []
    for k, job in enumerate(jobs):
        mode, left, right = job[0], job[1], job[2]
        hints = job[3] if len(job) > 3 else None
        out = job[4] if len(job) > 4 else None
        left = np.ascontiguousarray(left, np.float32)
        right = np.ascontiguousarray(right, np.float32)
        if left.ndim == 2:
            left = left[None]
        if right.ndim == 2:
            right = right[None]
        nl, rows, cols = left.shape
        nr = right.shape[0]
        if right.shape[1:] != (rows, cols):
            raise ValueError("left and right matrices must have the same size")
        shape = out_shape(mode, rows, cols, nl, nr)
        if shape[0] == 0:
            check(2)
        if out is None:
            out = np.empty(shape, np.float32)
        arr[k].mode = _mode(mode)
        arr[k].rows, arr[k].cols, arr[k].n_left, arr[k].n_right = rows, cols, nl, nr
        arr[k].h_left, arr[k].h_right, arr[k].h_out = left.ctypes.data, right.ctypes.data, out.ctypes.data
        arr[k].hints = C.pointer(hints) if hints is not None else None
        keep.append((left, right, hints))
        outs.append(out)
    check(lib().xcorr_run_host_batch_f32(arr, n, device))
    return outs


def n_to_mn_reorder(a: np.ndarray, n_left: int, to_grouped: bool) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    dst = np.empty_like(a)
    elems = int(np.prod(a.shape[1:]))
    check(lib().xcorr_n_to_mn_reorder_f32(a.ctypes.data, dst.ctypes.data, n_left, a.shape[0], elems,
                                          1 if to_grouped else 0))
    return dst


def last_launch() -> str:
    return lib().xcorr_last_launch_string().decode()


def launch_count() -> int:
    return int(lib().xcorr_launch_count())


def reset_launch_count() -> None:
    lib().xcorr_reset_launch_count()


def ffma_peak_probe(stream: int = 0):
    flops, ms = C.c_double(0), C.c_double(0)
    check(lib().xcorr_ffma_peak_probe(C.byref(flops), C.byref(ms), stream or None))
    return flops.value, ms.value


def dfma_peak_probe(stream: int = 0):
    flops, ms = C.c_double(0), C.c_double(0)
    check(lib().xcorr_dfma_peak_probe(C.byref(flops), C.byref(ms), stream or None))
    return flops.value, ms.value
