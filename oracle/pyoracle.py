"""ctypes front end for the two CPU checkers built by oracle/Makefile.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference legs of ``bench.py``.  The CUDA library and the ``cross`` host
program never import or link anything from this directory.

* ``Oracle``  -- the C restatement (oracle/xcorr_oracle.c), always available.
* ``Reference`` -- the reference's own CPU code (repo/cross-corr/src/validate.hpp:94-298)
  compiled unmodified into oracle/_ref/libxcorr_ref.so; available where that library was
  built (it needs the reference checkout at build time only).

* ``ReferenceCuda`` (end of file) -- the reference's own CUDA kernels recompiled for sm_100,
  an optional GPU baseline.

The two CPU checkers take float32 inputs of shape (n, rows, cols) and return outputs of shape
(n_out, 2*rows-1, 2*cols-1) in the reference's result order (validate.hpp:230-291):
one_to_many ``out[t]``, n_to_mn (file order) ``out[t*n_left + r]`` pairs with left ``r``,
n_to_m ``out[r*n_right + t]``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "libxcorr_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libxcorr_ref.so")

MODES = ("one_to_one", "one_to_many", "n_to_mn", "n_to_m")


def build(quiet: bool = True) -> None:
    """Run oracle/Makefile (C restatement always; reference library when the reference
    checkout is present on this machine)."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def n_outputs(mode: str, n_left: int, n_right: int) -> int:
    if mode == "one_to_one":
        return 1
    if mode in ("one_to_many", "n_to_mn"):
        return n_right
    if mode == "n_to_m":
        return n_left * n_right
    raise ValueError(mode)


def _as3(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    if a.ndim == 2:
        a = a[None]
    assert a.ndim == 3
    return a


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class Oracle:
    """The C restatement.  ``threads`` > 1 splits the independent result matrices over
    host threads (ctypes releases the GIL); 1 is the reference's single-threaded loop."""

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        u32, vp, i = C.c_uint32, C.c_void_p, C.c_int
        fpp = C.POINTER(C.c_float)
        self.lib.oracle_one_to_one.argtypes = [fpp, fpp, vp, u32, u32, i]
        self.lib.oracle_one_to_many.argtypes = [fpp, fpp, vp, u32, u32, u32, u32, u32, i]
        self.lib.oracle_n_to_mn.argtypes = [fpp, fpp, vp, u32, u32, u32, u32, u32, u32, i]
        self.lib.oracle_n_to_m.argtypes = [fpp, fpp, vp, u32, u32, u32, u32, u32, u32, i]
        self.lib.oracle_interleaved_index.argtypes = [u32, u32, u32]
        self.lib.oracle_interleaved_index.restype = u32
        self.lib.oracle_validate_result.argtypes = [
            C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_size_t, i, C.POINTER(C.c_double)]

    def run(self, mode: str, left, right, acc64: bool = False, threads: int = 1) -> np.ndarray:
        left, right = _as3(left), _as3(right)
        rows, cols = left.shape[1:]
        assert right.shape[1:] == (rows, cols)
        nl, nr = left.shape[0], right.shape[0]
        nout = n_outputs(mode, nl, nr)
        out = np.empty((nout, 2 * rows - 1, 2 * cols - 1), np.float64 if acc64 else np.float32)
        op = out.ctypes.data_as(C.c_void_p)
        a64 = 1 if acc64 else 0

        def call(first, last):
            if mode == "one_to_one":
                return self.lib.oracle_one_to_one(_fp(left), _fp(right), op, rows, cols, a64)
            if mode == "one_to_many":
                return self.lib.oracle_one_to_many(_fp(left), _fp(right), op, rows, cols, nr,
                                                   first, last, a64)
            if mode == "n_to_mn":
                return self.lib.oracle_n_to_mn(_fp(left), _fp(right), op, rows, cols, nl, nr,
                                               first, last, a64)
            return self.lib.oracle_n_to_m(_fp(left), _fp(right), op, rows, cols, nl, nr,
                                          first, last, a64)

        threads = max(1, min(threads, nout))
        if threads == 1 or mode == "one_to_one":
            rc = call(0, nout)
            if rc:
                raise RuntimeError(f"oracle {mode} failed with code {rc}")
        else:
            bounds = np.linspace(0, nout, threads + 1).astype(int)
            with ThreadPoolExecutor(threads) as ex:
                rcs = list(ex.map(lambda k: call(int(bounds[k]), int(bounds[k + 1])), range(threads)))
            if any(rcs):
                raise RuntimeError(f"oracle {mode} failed with codes {rcs}")
        return out

    def interleaved_index(self, i: int, group_size: int, num_groups: int) -> int:
        return int(self.lib.oracle_interleaved_index(i, group_size, num_groups))

    def validate(self, result, valid, elem_f32: bool = True):
        """(max, mean, stddev, result_at_max, valid_at_max) as validate.hpp:134-188."""
        r = np.ascontiguousarray(result, np.float64).ravel()
        v = np.ascontiguousarray(valid, np.float64).ravel()
        assert r.size == v.size
        stats = (C.c_double * 5)()
        dp = C.POINTER(C.c_double)
        rc = self.lib.oracle_validate_result(r.ctypes.data_as(dp), v.ctypes.data_as(dp), r.size,
                                             1 if elem_f32 else 0, stats)
        if rc:
            raise RuntimeError("oracle_validate_result failed")
        return tuple(stats)


class Reference:
    """The reference's own CPU code (single-threaded per call, like the reference)."""

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is not built (it needs the reference checkout at build time)")
        self.lib = C.CDLL(path)
        u32 = C.c_uint32
        fpp = C.POINTER(C.c_float)
        self.lib.ref_cpu_cross_corr_f32.argtypes = [C.c_int, fpp, fpp, fpp, u32, u32, u32, u32]
        self.lib.ref_cpu_cross_corr_f64.argtypes = [C.c_int, fpp, fpp, C.POINTER(C.c_double),
                                                    u32, u32, u32, u32]
        self.lib.ref_validate_result.argtypes = [C.POINTER(C.c_double), C.POINTER(C.c_double),
                                                 u32, C.c_int, C.POINTER(C.c_double)]

    @staticmethod
    def available(path: str = REF_SO) -> bool:
        return os.path.exists(path)

    def run(self, mode: str, left, right, acc64: bool = False) -> np.ndarray:
        left, right = _as3(left), _as3(right)
        rows, cols = left.shape[1:]
        nl, nr = left.shape[0], right.shape[0]
        nout = n_outputs(mode, nl, nr)
        m = MODES.index(mode)
        if acc64:
            out = np.empty((nout, 2 * rows - 1, 2 * cols - 1), np.float64)
            rc = self.lib.ref_cpu_cross_corr_f64(m, _fp(left), _fp(right),
                                                 out.ctypes.data_as(C.POINTER(C.c_double)),
                                                 rows, cols, nl, nr)
        else:
            out = np.empty((nout, 2 * rows - 1, 2 * cols - 1), np.float32)
            rc = self.lib.ref_cpu_cross_corr_f32(m, _fp(left), _fp(right), _fp(out),
                                                 rows, cols, nl, nr)
        if rc:
            raise RuntimeError(f"reference {mode} failed with code {rc}")
        return out

    def run_threaded(self, mode: str, left, right, threads: int) -> np.ndarray:
        """Split the independent result matrices over host threads, each thread calling the
        unmodified single-threaded reference routine on its share (float path)."""
        left, right = _as3(left), _as3(right)
        nl, nr = left.shape[0], right.shape[0]
        if mode == "one_to_one" or threads <= 1:
            return self.run(mode, left, right)
        if mode == "one_to_many":
            parts = [p for p in np.array_split(np.arange(nr), threads) if len(p)]
            jobs = [("one_to_many", left, right[p[0]:p[-1] + 1]) for p in parts]
        elif mode == "n_to_m":
            parts = [p for p in np.array_split(np.arange(nl), threads) if len(p)]
            jobs = [("n_to_m", left[p[0]:p[-1] + 1], right) for p in parts]
        else:  # n_to_mn in file order: split the left index r, keep every t
            m = nr // nl
            parts = [p for p in np.array_split(np.arange(nl), threads) if len(p)]
            r4 = right.reshape(m, nl, *right.shape[1:])
            jobs = [("n_to_mn", left[p[0]:p[-1] + 1],
                     np.ascontiguousarray(r4[:, p[0]:p[-1] + 1]).reshape(-1, *right.shape[1:]))
                    for p in parts]
        with ThreadPoolExecutor(len(jobs)) as ex:
            outs = list(ex.map(lambda j: self.run(*j), jobs))
        if mode == "n_to_mn":
            m = nr // nl
            oshape = outs[0].shape[1:]
            blocks = [o.reshape(m, -1, *oshape) for o in outs]
            return np.concatenate(blocks, axis=1).reshape(-1, *oshape)
        return np.concatenate(outs, axis=0)

    def validate(self, result, valid, elem_f32: bool = True):
        r = np.ascontiguousarray(result, np.float64).ravel()
        v = np.ascontiguousarray(valid, np.float64).ravel()
        stats = (C.c_double * 5)()
        dp = C.POINTER(C.c_double)
        rc = self.lib.ref_validate_result(r.ctypes.data_as(dp), v.ctypes.data_as(dp), r.size,
                                          1 if elem_f32 else 0, stats)
        if rc:
            raise RuntimeError("ref_validate_result failed")
        return tuple(stats)


REFCUDA_SO = os.path.join(_HERE, "_ref", "libxcorr_refcuda.so")
REFCUDA_N2M_SO = os.path.join(_HERE, "_ref", "libxcorr_refcuda_n2m.so")


class ReferenceCuda:
    """The reference's own best CUDA launchers (kernels.cuh:41-256), compiled unmodified for
    sm_100 by ``make -C oracle refcuda`` / ``refcuda_n2m`` with the template limits of the best
    published arguments.  A GPU baseline and a further parity witness; optional (the build
    takes from ten minutes to hours and needs the reference checkout).

    All methods take DEVICE pointers (ints) and launch asynchronously, like the reference's
    launchers.  Arguments default to the best published ones: one_to_one ``4_8_8``
    (warps, shifts per thread, left rows), one_to_many / n_to_mn ``4_4_4_4`` (warps, shifts per
    right matrix, right matrices per thread, left rows), n_to_m ``4_4_4_4_4``.
    """

    def __init__(self, path: str = REFCUDA_SO, n2m_path: str = REFCUDA_N2M_SO):
        self.lib = C.CDLL(path)
        u32, vp = C.c_uint32, C.c_void_p
        self.lib.refcuda_overlap_wise.argtypes = [vp, vp, vp, u32, u32, u32, u32]
        self.lib.refcuda_one_to_one.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32]
        self.lib.refcuda_one_to_many.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, vp]
        for f in (self.lib.refcuda_overlap_wise, self.lib.refcuda_one_to_one, self.lib.refcuda_one_to_many):
            f.restype = C.c_int
        self.n2m = None
        if os.path.exists(n2m_path):
            self.n2m = C.CDLL(n2m_path)
            self.n2m.refcuda_n_to_m.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, u32]
            self.n2m.refcuda_n_to_m.restype = C.c_int

    @staticmethod
    def available(path: str = REFCUDA_SO) -> bool:
        return os.path.exists(path)

    @staticmethod
    def _check(rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"reference launcher {what} rejected its arguments (code {rc})")

    def overlap_wise(self, d_left, d_right, d_out, rows, cols, n_left=1, batch=1):
        """run_cross_corr_naive_original: `batch` deformed matrices per reference matrix."""
        self._check(self.lib.refcuda_overlap_wise(d_left, d_right, d_out, rows, cols, n_left, batch), "overlap_wise")

    def one_to_one(self, d_left, d_right, d_out, rows, cols, warps=4, shifts=8, left_rows=8):
        self._check(self.lib.refcuda_one_to_one(d_left, d_right, d_out, rows, cols, warps, shifts, left_rows),
                    "one_to_one")

    def one_to_many(self, d_left, d_right, d_out, rows, cols, n_right, warps=4, shifts=4, right_mats=4,
                    left_rows=4, stream=0):
        self._check(self.lib.refcuda_one_to_many(d_left, d_right, d_out, rows, cols, n_right, warps, shifts,
                                                 right_mats, left_rows, stream), "one_to_many")

    def n_to_mn(self, d_left, d_right, d_out, rows, cols, n_left, n_right, streams=(0,), **kw):
        """One one_to_many launch per left matrix on round-robin streams, grouped order
        (n_to_mn.hpp:553-571)."""
        m = n_right // n_left
        in_b, out_b = rows * cols * 4, (2 * rows - 1) * (2 * cols - 1) * 4
        for l in range(n_left):
            self.one_to_many(d_left + l * in_b, d_right + l * m * in_b, d_out + l * m * out_b, rows, cols, m,
                             stream=streams[l % len(streams)], **kw)

    def n_to_m(self, d_left, d_right, d_out, rows, cols, n_left, n_right, warps=4, shifts=4, left_mats=4,
               right_mats=4, left_rows=4):
        if self.n2m is None:
            raise RuntimeError("the reference n-to-m kernel library was not built (make -C oracle refcuda_n2m)")
        self._check(self.n2m.refcuda_n_to_m(d_left, d_right, d_out, rows, cols, n_left, n_right, warps, shifts,
                                            left_mats, right_mats, left_rows), "n_to_m")


REFCUDA_WPS_SO = os.path.join(_HERE, "_ref", "libxcorr_refcuda_wps.so")


class ReferenceWarpPerShift:
    """The reference's plain warp-per-overlap launcher ``run_ccn_warp_per_shift``
    (kernels.cuh:98-106, naive_warp_per_shift.cu:308-335), compiled unmodified for sm_100 by
    ``make -C oracle refcuda_wps``: the reference's published winner for a 16 x 16 pair.  Device
    pointers (ints), asynchronous launch on the default stream, one pair per call."""

    def __init__(self, path: str = REFCUDA_WPS_SO):
        self.lib = C.CDLL(path)
        u32, vp, i = C.c_uint32, C.c_void_p, C.c_int
        self.lib.refcuda_warp_per_shift.argtypes = [vp, vp, vp, u32, u32, u32]
        self.lib.refcuda_warp_per_shift.restype = i
        self.lib.refcuda_warp_per_shift_graph_us.argtypes = [vp, vp, vp, u32, u32, u32, u32, u32]
        self.lib.refcuda_warp_per_shift_graph_us.restype = C.c_double

    @staticmethod
    def available(path: str = REFCUDA_WPS_SO) -> bool:
        return os.path.exists(path)

    def warp_per_shift(self, d_left, d_right, d_out, rows, cols, shifts_per_block=16):
        rc = self.lib.refcuda_warp_per_shift(d_left, d_right, d_out, rows, cols, shifts_per_block)
        if rc != 0:
            raise RuntimeError(f"reference launcher warp_per_shift rejected its arguments (code {rc})")

    def graph_us(self, d_left, d_right, d_out, rows, cols, shifts_per_block=16, launches=20, replays=10):
        """Microseconds of device time per launch of the reference kernel: ``launches`` calls
        recorded into a CUDA graph on the calling thread's default stream, replayed ``replays``
        times between two events.  Negative when the capture failed."""
        return float(self.lib.refcuda_warp_per_shift_graph_us(d_left, d_right, d_out, rows, cols, shifts_per_block,
                                                              launches, replays))
