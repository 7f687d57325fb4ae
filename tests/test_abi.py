"""CPU tests of the C-ABI library: it loads, exports every symbol include/xcorr.h declares,
and its host-only entry points (planning, shard ranges, order helpers, argument checks that
fail before any CUDA call) behave.  No kernel runs here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import file_to_grouped, grouped_to_file


def declared_symbols(header_path):
    text = open(header_path).read()
    return sorted(set(re.findall(r"XCORR_API[^;(]*?\b(xcorr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(xc):
    names = declared_symbols(xc.HEADER_PATH)
    assert len(names) >= 19
    lib = C.CDLL(xc.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_hints_struct_layout(xc):
    assert C.sizeof(xc.Hints) == 20 * 4


def test_status_strings(xc):
    lib = xc.lib()
    assert lib.xcorr_status_string(0) == b"ok"
    assert lib.xcorr_status_string(2) == b"invalid size"
    assert lib.xcorr_status_string(99) == b"unknown status"


def test_num_results_and_input_rules(xc):
    lib = xc.lib()
    # one_to_one.hpp:20-22, one_to_many.hpp:15-17, n_to_mn.hpp:23-25, n_to_m.hpp:19-21
    assert lib.xcorr_validate_input_size(0, 16, 16, 1, 1) == 1
    assert lib.xcorr_validate_input_size(0, 16, 16, 1, 2) == 0
    assert lib.xcorr_validate_input_size(0, 0, 16, 1, 1) == 0
    assert lib.xcorr_validate_input_size(1, 4, 4, 1, 7) == 1
    assert lib.xcorr_validate_input_size(1, 4, 4, 2, 7) == 0
    assert lib.xcorr_validate_input_size(2, 4, 4, 3, 9) == 1
    assert lib.xcorr_validate_input_size(2, 4, 4, 3, 10) == 0
    assert lib.xcorr_validate_input_size(3, 4, 4, 3, 10) == 1
    assert lib.xcorr_validate_input_size(7, 4, 4, 1, 1) == 0
    assert lib.xcorr_num_results(0, 1, 1) == 1
    assert lib.xcorr_num_results(1, 1, 512) == 512
    assert lib.xcorr_num_results(2, 16, 2048) == 2048
    assert lib.xcorr_num_results(3, 32, 64) == 2048
    assert lib.xcorr_num_results(2, 16, 2047) == 0


def test_shard_ranges_partition_the_units(xc):
    for units, parts in [(512, 8), (16, 8), (32, 3), (5, 8), (1, 2), (2048, 7)]:
        covered = []
        sizes = []
        for i in range(parts):
            first, count = xc.shard_range(units, parts, i)
            covered.extend(range(first, first + count))
            sizes.append(count)
        assert covered == list(range(units))
        assert max(sizes) - min(sizes) <= 1
    assert xc.shard_range(10, 0, 0) == (0, 0)
    assert xc.shard_range(10, 4, 4) == (0, 0)


def test_n_to_mn_reorder_matches_reference_index(xc, oracle):
    n, m, elems = 3, 4, 6
    a = np.arange(n * m * elems, dtype=np.float32).reshape(n * m, 2, 3)
    g = xc.n_to_mn_reorder(a, n, True)
    for i in range(n * m):
        assert np.array_equal(g[oracle.interleaved_index(i, n, m)], a[i])   # matrix.hpp:614-618
    assert np.array_equal(xc.n_to_mn_reorder(g, n, False), a)
    assert np.array_equal(g, file_to_grouped(a, n))
    assert np.array_equal(grouped_to_file(g, n), a)
    with pytest.raises(xc.XcorrError):
        xc.n_to_mn_reorder(a[:5], 3, True)


def test_workspace_planning_without_a_device(xc):
    # config 2 (one pair of 256x256) needs a row split over ~all SMs -> partial images
    big = xc.workspace_bytes("one_to_one", 256, 256, 1, 1)
    out_bytes = 511 * 511 * 4
    assert big > 0 and big % out_bytes == 0 and 8 <= big // out_bytes <= 64
    # many independent pairs fill the GPU without a row split, or with atomics: no workspace
    assert xc.workspace_bytes("one_to_many", 64, 64, 1, 512) == 0
    assert xc.workspace_bytes("n_to_m", 32, 32, 32, 64) == 0
    # stream-K with partial images on request: two or three result-sized images and the counters
    sk = xc.workspace_bytes("one_to_many", 64, 64, 1, 512, xc.make_hints(kernel="tile", schedule=2, combine="workspace"))
    assert 2 * 512 * 127 * 127 * 4 <= sk <= 3 * 512 * 127 * 127 * 4 + 65536
    # explicit hints
    h = xc.make_hints(kernel="tile", combine="workspace", row_slices=4)
    assert xc.workspace_bytes("one_to_one", 16, 16, 1, 1, h) == 4 * 31 * 31 * 4
    assert xc.workspace_bytes("one_to_one", 16, 16, 1, 1, xc.make_hints(kernel="overlap_wise")) == 0
    # invalid shapes plan nothing
    assert xc.workspace_bytes("n_to_mn", 16, 16, 3, 10) == 0


def test_argument_errors_come_back_as_status_codes(xc):
    lib = xc.lib()
    # NULL pointers and bad counts are rejected before any CUDA call
    assert lib.xcorr_one_to_one_f32(None, None, None, 4, 4, None, None, 0, None) == 1
    buf = np.zeros(64, np.float32)
    p = buf.ctypes.data
    assert lib.xcorr_run_f32(2, p, p, p, 4, 4, 3, 10, None, None, 0, None) == 2
    assert lib.xcorr_run_f32(0, p, p, p, 0, 4, 1, 1, None, None, 0, None) == 2
    assert lib.xcorr_run_f32(9, p, p, p, 4, 4, 1, 1, None, None, 0, None) == 2
    assert lib.xcorr_run_host_f32(0, None, p, p, 4, 4, 1, 1, None, 0) == 1
    assert b"NULL" in lib.xcorr_last_error_string()
    assert lib.xcorr_run_host_sharded_f32(1, p, p, p, 4, 4, 1, 2, None, None, 0) == 7
    assert lib.xcorr_run_host_batch_f32(None, 3, 0) == 1
    assert lib.xcorr_run_host_batch_f32(None, -1, 0) == 2
    assert lib.xcorr_run_host_batch_f32(None, 0, 0) == 0
    job = (xc.HostJob * 1)()
    job[0].mode, job[0].rows, job[0].cols, job[0].n_left, job[0].n_right = 2, 4, 4, 3, 10
    job[0].h_left = job[0].h_right = job[0].h_out = p
    assert lib.xcorr_run_host_batch_f32(job, 1, 0) == 2           # 10 rights do not divide over 3 lefts
    job[0].h_out = None
    assert lib.xcorr_run_host_batch_f32(job, 1, 0) == 1
    assert lib.xcorr_n_to_mn_reorder_f32(None, p, 1, 1, 1, 1) == 1
    assert lib.xcorr_ffma_peak_probe(None, None, None) == 1
    assert lib.xcorr_dfma_peak_probe(None, None, None) == 1
    assert lib.xcorr_run_f64(0, None, p, p, 4, 4, 1, 1, None) == 1
    assert lib.xcorr_run_f64(2, p, p, p, 4, 4, 3, 10, None) == 2
    assert lib.xcorr_run_host_f64(1, p, None, p, 4, 4, 1, 2, 0) == 1
    assert lib.xcorr_run_host_f64(3, p, p, p, 4, 0, 1, 2, 0) == 2


def test_plans_exist_and_fit_for_a_sweep_of_shapes(xc):
    """The planner needs no device: for a sweep of modes, sizes and counts every automatic plan
    exists, fits one SM's shared memory, has a non-empty grid, and the workspace query agrees
    with the plan text."""
    import re
    rng = np.random.default_rng(7)
    shapes = [(1, 1), (2, 3), (5, 5), (16, 16), (17, 33), (31, 64), (48, 48), (64, 64), (100, 9), (96, 128),
              (200, 200), (256, 256), (300, 40), (512, 512)]
    for rows, cols in shapes:
        for mode, nl, nr in (("one_to_one", 1, 1), ("one_to_many", 1, int(rng.integers(1, 600))),
                             ("n_to_mn", 3, 3 * int(rng.integers(1, 40))), ("n_to_m", int(rng.integers(1, 20)), int(rng.integers(1, 70)))):
            text = xc.describe_plan(mode, rows, cols, nl, nr)
            if text == "kernel=warp_per_overlap":          # a handful of overlaps: the warp-per-overlap latency kernel
                assert nl * (nr if mode != "n_to_mn" else nr // nl) * (2 * rows - 1) * (2 * cols - 1) <= 8000 or \
                    (mode == "n_to_mn" and nr * (2 * rows - 1) * (2 * cols - 1) <= 8000)
                assert xc.workspace_bytes(mode, rows, cols, nl, nr) == 0
                continue
            m = re.search(r"grid=\((\d+),1,1\) block=\((\d+),1,1\) smem=(\d+) plan\{H=(\d+) W=(\d+) Hp=(\d+) Wp=(\d+) SL=(\d+) "
                          r"ML=(\d+) WX=(\d+) WY=(\d+) .* S=(\d+) schedule=([a-z-]+) tasks=(\d+) nstage=(\d+) "
                          r"combine=([a-z]+) workspace=(\d+)\}", text)
            assert m, text
            grid, block, smem, H, W, Hp, Wp, SL, ML, WX, WY, S = (int(v) for v in m.groups()[:12])
            sched, tasks, nstage, comb, ws = m.group(13), int(m.group(14)), int(m.group(15)), m.group(16), int(m.group(17))
            assert (H, W) == (rows, cols) and Hp >= H and Wp >= W and Wp % 16 == 0 and SL * ML == 32, text
            assert 1 <= grid and 32 <= block <= 512 and block == 32 * WX * WY and smem <= 227 * 1024, text
            assert tasks >= 1 and nstage >= 1 and (S == 1 or sched == "static"), text
            assert ws == xc.workspace_bytes(mode, rows, cols, nl, nr), text
            assert (ws > 0) == (comb in ("workspace", "fixup")), text


def test_planner_choices_for_the_benchmark_shapes(xc):
    """The per-shape choices the measurements led to, checked without a device (a B200 is assumed):
    the warp queue against a static plan whose last wave of blocks is under-filled (64x64 1x512:
    128 equal blocks on 148 SMs), stream-K kept where it is balanced already (48x48 16x128), fused
    rows only for 17..32 columns with one class per thread and never under stream-K (under the
    queue for 32x32 32x64, in static blocks for its shards), 16-warp blocks for the queue with one
    class per thread, the warp-per-overlap kernel for a handful of overlaps, hints that override
    all of it."""
    c3 = xc.describe_plan("one_to_many", 64, 64, 1, 512)
    assert "schedule=warp-queue" in c3 and "grid=(148,1,1)" in c3 and "combine=store" in c3 and "fused=0" in c3
    assert "tile<TY=1>" in c3 and "block=(512,1,1)" in c3
    c4 = xc.describe_plan("n_to_m", 32, 32, 32, 64)
    assert "schedule=warp-queue" in c4 and "fused=1" in c4 and "tile<TY=1>" in c4 and "combine=store" in c4
    sat = xc.describe_plan("one_to_many", 32, 32, 1, 4000)        # a full static plan, yet the queue is estimated 6 % faster
    assert "schedule=warp-queue" in sat
    # small shapes of 17..32 columns: static blocks with fused rows where they fill the GPU (timed 19 against
    # 23 us of stream-K), stream-K where they do not, or where ragged rows would be staged word by word by few threads
    mid = xc.describe_plan("n_to_mn", 24, 24, 32, 256)
    assert "schedule=static" in mid and "fused=1" in mid
    assert "schedule=stream-k" in xc.describe_plan("n_to_m", 32, 32, 8, 8)
    assert "schedule=stream-k" in xc.describe_plan("one_to_many", 17, 30, 1, 100)
    c5 = xc.describe_plan("n_to_mn", 48, 48, 16, 2048)
    assert "schedule=stream-k" in c5 and "fused=0" in c5
    small = xc.describe_plan("n_to_m", 32, 32, 4, 64)
    assert "schedule=static" in small and "fused=1" in small and "tile<TY=1>" in small
    assert "fused=0" in xc.describe_plan("n_to_m", 32, 32, 4, 64, xc.make_hints(kernel="tile", fused_rows=2))
    assert "fused=0" in xc.describe_plan("n_to_m", 32, 32, 4, 64, xc.make_hints(kernel="tile", schedule=2, overlap_rows=1))
    assert "fused=0" in xc.describe_plan("n_to_m", 32, 32, 4, 64, xc.make_hints(kernel="tile", overlap_rows=2))
    assert "fused=0" in xc.describe_plan("n_to_m", 48, 48, 4, 64, xc.make_hints(kernel="tile", overlap_rows=1))
    assert xc.describe_plan("one_to_one", 16, 16, 1, 1) == "kernel=warp_per_overlap"
    assert xc.describe_plan("one_to_one", 24, 24, 1, 1) == "kernel=warp_per_overlap"
    assert xc.describe_plan("one_to_one", 32, 32, 1, 1) == "kernel=warp_per_overlap"
    assert xc.describe_plan("one_to_many", 16, 16, 1, 8) == "kernel=warp_per_overlap"
    assert "kernel=tile" in xc.describe_plan("one_to_one", 40, 40, 1, 1)
    assert "kernel=tile" in xc.describe_plan("one_to_one", 2, 40, 1, 1)
    assert "kernel=tile" in xc.describe_plan("one_to_many", 16, 16, 1, 9)
    assert "kernel=tile" in xc.describe_plan("one_to_one", 16, 16, 1, 1, xc.make_hints(reproducible=1, kernel="tile"))
    forced = xc.describe_plan("n_to_mn", 48, 48, 16, 2048, xc.make_hints(kernel="tile", schedule=3))
    assert "schedule=warp-queue" in forced and "KG=" in forced and "KL=" in forced
    # a queue round stages several matrix groups, and the rows of several left matrices where the groups
    # of one left are few
    import re
    q = xc.describe_plan("n_to_m", 32, 32, 32, 64, xc.make_hints(kernel="tile", schedule=3, overlap_rows=1, class_lanes=2,
                                                                 warps_x=12, warps_y=1))
    kg, kl = (int(v) for v in re.search(r"KG=(\d+) KL=(\d+)", q).groups())
    assert kg >= 2 and kl == 2 and "fused=1" in q


def test_header_is_plain_c(xc, tmp_path):
    """include/xcorr.h compiles as C99 with warnings on, and a C program links against the
    library and calls a host-only entry point: the boundary is a C ABI, not a C++ one."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    src = tmp_path / "t.c"
    src.write_text('#include <stdio.h>\n#include "xcorr.h"\n'
                   'int main(void) { xcorr_hints h = {0}; unsigned first = 0, count = 0; (void)h;\n'
                   '  float buf[16] = {0};\n'
                   '  xcorr_host_job jobs[1] = { { XCORR_N_TO_MN, 2, 2, 3, 4, buf, buf, buf, NULL } };\n'
                   '  if (xcorr_run_host_batch_f32(jobs, 1, 0) != XCORR_ERR_INVALID_SIZE) return 3;  /* 4 rights, 3 lefts */\n'
                   '  xcorr_shard_range(10, 3, 1, &first, &count);\n'
                   '  printf("%u %u %llu %s\\n", first, count, (unsigned long long)xcorr_num_results(XCORR_N_TO_M, 3, 4),\n'
                   '         xcorr_status_string(XCORR_ERR_WORKSPACE)); return 0; }\n')
    exe = tmp_path / "t"
    inc = os.path.dirname(xc.HEADER_PATH)
    libdir = os.path.dirname(xc.LIB_PATH)
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{inc}", str(src), "-o", str(exe),
                        f"-L{libdir}", "-lxcorr", f"-Wl,-rpath,{libdir}", "-Wl,-rpath,/usr/local/cuda/lib64"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.split()[:3] == ["3", "3", "12"], (r.stdout, r.stderr)
