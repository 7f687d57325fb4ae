"""Tests of the `cross` host program: command line, algorithm registry, matrix file format,
timing CSV, exit codes.  The CPU tests use the cpu_* algorithms (no GPU needed); the GPU
tests run the CUDA-backed algorithms and compare the files they write with the oracle."""
import json
import os
import subprocess

import numpy as np
import pytest

from conftest import grouped_to_file, seeded_inputs

# the reference's registry (repo/cross-corr/src/main.cpp:368-402) without its FFT entries
EXPECTED_NAMES = sorted("""
cpu_one_to_one cpu_one_to_many cpu_n_to_mn cpu_n_to_m
nai_orig_one_to_one nai_orig_one_to_many nai_orig_n_to_mn nai_orig_n_to_m
nai_shuffle_one_to_one nai_shuffle_work_distribution_one_to_one
nai_shuffle_multimat_right_one_to_one nai_shuffle_multimat_right_one_to_many
nai_shuffle_multimat_right_work_distribution_one_to_one
nai_shuffle_multimat_right_work_distribution_one_to_many
nai_shuffle_multimat_right_work_distribution_n_to_mn
nai_shuffle_multimat_right_work_distribution_n_to_m
nai_shuffle_multimat_both_work_distribution_local_mem_n_to_m
nai_shuffle_multimat_both_work_distribution_n_to_m
nai_shuffle_multirow_both_multimat_both_n_to_m
nai_shuffle_multirow_right_one_to_one nai_shuffle_multirow_both_one_to_one
nai_shuffle_multirow_both_local_mem_one_to_one
nai_shuffle_multirow_right_multimat_right_one_to_one
nai_shuffle_multirow_right_multimat_right_one_to_many
nai_shuffle_multirow_right_multimat_right_n_to_mn
nai_shuffle_multirow_both_multimat_right_one_to_many
nai_shuffle_multirow_both_multimat_right_n_to_mn
nai_warp_per_shift_one_to_one nai_warp_per_shift_simple_indexing_one_to_one
nai_warp_per_shift_work_distribution_one_to_one
nai_warp_per_shift_shared_mem_one_to_one nai_warp_per_shift_shared_mem_one_to_many
nai_warp_per_shift_shared_mem_n_to_mn nai_warp_per_shift_shared_mem_n_to_m
nai_block_per_shift_one_to_one
fft_orig_one_to_one fft_reduced_transfer_one_to_one fft_orig_one_to_many fft_reduced_transfer_one_to_many
fft_orig_n_to_mn fft_reduced_transfer_n_to_mn fft_better_n_to_m
""".split())


@pytest.fixture(scope="session")
def cross(xc):
    if not os.path.exists(xc.CROSS_PATH):
        xc.build()
    return xc.CROSS_PATH


def run(cross, *args, cwd=None):
    return subprocess.run([cross, *map(str, args)], capture_output=True, text=True, cwd=cwd, timeout=600)


def write_matrices(path, arr):
    """The reference's input format (benchmark/input_generator.py:20-32): header
    '# rows,cols,count' then one comma-separated line per matrix row."""
    arr = np.asarray(arr)
    n, rows, cols = arr.shape
    np.savetxt(path, arr.reshape(n * rows, cols), delimiter=",", header=f"{rows},{cols},{n}")


def read_matrices(path):
    with open(path) as f:
        head = f.readline()
    assert head.startswith("# ")
    rows, cols, n = (int(v) for v in head[2:].split(","))
    data = np.loadtxt(path, delimiter=",", skiprows=1, ndmin=2)
    assert data.shape == (rows * n, cols)
    return data.reshape(n, rows, cols)


# ---- no GPU needed --------------------------------------------------------------------------------
def test_list_prints_the_registry_sorted(cross):
    r = run(cross, "list")
    assert r.returncode == 0
    assert r.stdout.split() == EXPECTED_NAMES


def test_help_and_unknown_command(cross):
    assert run(cross).returncode == 0 and "Usage:" in run(cross).stdout
    assert run(cross, "--help").returncode == 0
    r = run(cross, "frobnicate")
    assert r.returncode == 1 and "Unknown command frobnicate" in r.stderr


def test_input_command(cross):
    assert run(cross, "input", "one_to_one", 16, 16, 1, 1).stdout == "Valid\n"
    assert run(cross, "input", "one_to_one", 16, 16, 1, 2).stdout == "Invalid\n"
    assert run(cross, "input", "one_to_many", 16, 16, 1, 200).stdout == "Valid\n"
    assert run(cross, "input", "n_to_mn", 16, 16, 4, 10).stdout == "Invalid\n"
    assert run(cross, "input", "n_to_mn", 16, 16, 4, 12).stdout == "Valid\n"
    assert run(cross, "input", "n_to_m", 0, 16, 4, 12).stdout == "Invalid\n"
    r = run(cross, "input", "many_to_many", 1, 1, 1, 1)
    assert r.returncode == 1 and "Unknown algorithm type" in r.stderr
    assert run(cross, "input", "n_to_m", 1, 1).returncode == 1


@pytest.mark.parametrize("mode,rows,cols,nl,nr", [
    ("one_to_one", 5, 7, 1, 1), ("one_to_many", 6, 6, 1, 3), ("n_to_mn", 4, 5, 2, 6), ("n_to_m", 3, 8, 2, 3)])
def test_cpu_algorithms_write_the_reference_result(cross, oracle, tmp_path, mode, rows, cols, nl, nr):
    left, right = seeded_inputs(rows, cols, nl, nr, 17)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    r = run(cross, "run", "-o", tmp_path / "out.csv", f"cpu_{mode}", tmp_path / "l.csv", tmp_path / "r.csv",
            cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert "Loading inputs" in r.stdout and "No validation" in r.stdout
    got = read_matrices(tmp_path / "out.csv")
    want = oracle.run(mode, left, right)                     # n_to_mn: file order both sides
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 5.1e-7                # six printed decimals
    assert not os.path.exists(tmp_path / "measurements.csv")  # benchmark_type None writes no timings


def test_output_format_is_fixed_six_decimals_with_header(cross, tmp_path):
    left = np.array([[[1.0, 2.0], [3.0, 4.0]]], np.float32)
    right = np.array([[[0.5, 0.25], [2.0, 1.0]]], np.float32)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    assert run(cross, "run", "--out", tmp_path / "o.csv", "cpu_one_to_one", tmp_path / "l.csv",
               tmp_path / "r.csv", cwd=tmp_path).returncode == 0
    lines = open(tmp_path / "o.csv").read().splitlines()
    assert lines[0] == "# 3,3,1"
    assert lines[1] == "1.000000,4.000000,4.000000"          # shifts (-1,-1), (0,-1), (1,-1)
    assert lines[2] == "3.250000,11.000000,9.000000"
    assert lines[3] == "0.750000,2.500000,2.000000"


def test_non_square_results_are_written_row_by_row(cross, oracle, tmp_path):
    left, right = seeded_inputs(2, 9, 1, 1, 3)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    assert run(cross, "run", "-o", tmp_path / "o.csv", "cpu_one_to_one", tmp_path / "l.csv", tmp_path / "r.csv",
               cwd=tmp_path).returncode == 0
    got = read_matrices(tmp_path / "o.csv")
    assert got.shape == (1, 3, 17)
    assert np.abs(got - oracle.run("one_to_one", left, right)).max() <= 5.1e-7


def test_timing_csv_layouts(cross, tmp_path):
    left, right = seeded_inputs(6, 6, 1, 1, 4)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    base = ["cpu_one_to_one", tmp_path / "l.csv", tmp_path / "r.csv"]
    # Compute: one label, adaptive repetition until min_time
    r = run(cross, "run", "-b", "Compute", "-m", "0.01", "-t", tmp_path / "c.csv", *base, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    rows = open(tmp_path / "c.csv").read().splitlines()
    assert rows[0] == "Computation,Computation_iterations"
    ns, it = (int(v) for v in rows[1].split(","))
    assert ns > 0 and it >= 1 and ns * it >= 0.01e9 * 0.9
    # CommonSteps: the seven step labels (cross_corr.hpp:168-176)
    r = run(cross, "run", "-b", "CommonSteps", "-m", "0.001", "-t", tmp_path / "s.csv", "--no_progress", *base,
            cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    rows = open(tmp_path / "s.csv").read().splitlines()
    labels = ["Load", "Prepare", "Transfer", "Run", "Finalize", "Free", "Store"]
    assert rows[0] == ",".join(f"{l},{l}_iterations" for l in labels)
    assert len(rows[1].split(",")) == 14 and r.stdout == ""
    # append + outer loops: no second header, one row per loop; outputs get _<loop> suffixes
    r = run(cross, "run", "-b", "Compute", "-m", "0.001", "-a", "-l", "2", "-t", tmp_path / "c.csv",
            "-o", tmp_path / "res.csv", *base, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert len(open(tmp_path / "c.csv").read().splitlines()) == 4
    assert os.path.exists(tmp_path / "res_0.csv") and os.path.exists(tmp_path / "res_1.csv")
    # default timing file name
    r = run(cross, "run", "-b", "Compute", "-m", "0.001", *base, cwd=tmp_path)
    assert r.returncode == 0 and os.path.exists(tmp_path / "measurements.csv")


def test_validate_option_and_command(cross, oracle, tmp_path):
    left, right = seeded_inputs(7, 5, 1, 2, 6)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    base = ["cpu_one_to_many", tmp_path / "l.csv", tmp_path / "r.csv"]
    # --validate without a value recomputes on the CPU: zero error, human-readable block
    r = run(cross, "run", "-v", *base, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert "Difference from valid values:" in r.stdout and "Max: 0" in r.stdout
    # machine-readable form with --no_progress (validate.hpp:58-66)
    r = run(cross, "run", "--validate", "--no_progress", *base, cwd=tmp_path)
    assert r.stdout.splitlines() == ["Max,Mean,Stddev", "0.000000e+00,0.000000e+00,0.000000e+00"]
    # --validate <file>, given the way the reference's driver does (executable.py:137-145)
    assert run(cross, "run", "-o", tmp_path / "valid.csv", *base, cwd=tmp_path).returncode == 0
    r = run(cross, "run", "--validate", tmp_path / "valid.csv", "--no_progress", *base, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    mx = float(r.stdout.splitlines()[1].split(",")[0])
    assert 0 <= mx < 1e-3                                     # file holds six decimals; small corner sums
    # `cross validate`: template first, files to check after it
    wrong = oracle.run("one_to_many", left, right) * 1.001
    write_matrices(tmp_path / "wrong.csv", wrong)
    r = run(cross, "validate", "-c", "-p", tmp_path / "valid.csv", tmp_path / "valid.csv", tmp_path / "wrong.csv")
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    assert lines[0] == "Max,Mean,Stddev" and float(lines[1].split(",")[0]) == 0.0
    assert abs(float(lines[2].split(",")[0]) - 1e-3) < 1e-4


def write_binary(path, a):
    a = np.ascontiguousarray(a, "<f4")
    n, rows, cols = a.shape
    with open(path, "wb") as f:
        f.write(b"XCORRMAT" + np.array([cols, rows, n], "<u4").tobytes() + a.tobytes())


def read_binary(path):
    raw = open(path, "rb").read()
    assert raw[:8] == b"XCORRMAT"
    cols, rows, n = np.frombuffer(raw[8:20], "<u4")
    return np.frombuffer(raw[20:], "<f4").reshape(n, rows, cols)


def test_binary_matrix_files(cross, oracle, tmp_path):
    """Paths ending in .bin are binary matrix files (header + float32 data), for inputs, results
    and validation templates alike; n_to_mn keeps the file order t*n + l in both formats."""
    left, right = seeded_inputs(6, 9, 2, 6, 17)
    write_binary(tmp_path / "l.bin", left)
    write_binary(tmp_path / "r.bin", right)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    r = run(cross, "run", "-o", tmp_path / "o.bin", "cpu_n_to_mn", tmp_path / "l.bin", tmp_path / "r.bin", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    got = read_binary(tmp_path / "o.bin")
    want = oracle.run("n_to_mn", left, right)
    assert got.shape == want.shape and np.array_equal(got, want)          # same float arithmetic, no text rounding
    # mixed formats: text in, binary template
    r = run(cross, "run", "--validate", tmp_path / "o.bin", "--no_progress", "cpu_n_to_mn", tmp_path / "l.csv",
            tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert float(r.stdout.splitlines()[1].split(",")[0]) < 1e-5           # text inputs carry full precision here
    r = run(cross, "validate", "-c", "-p", tmp_path / "o.bin", tmp_path / "o.bin")
    assert r.returncode == 0 and float(r.stdout.splitlines()[1].split(",")[0]) == 0.0
    # broken files: loading-step errors
    (tmp_path / "bad.bin").write_bytes(b"NOTAMATRIXFILE")
    assert run(cross, "run", "cpu_one_to_one", tmp_path / "bad.bin", tmp_path / "bad.bin").returncode == 3
    (tmp_path / "short.bin").write_bytes(open(tmp_path / "l.bin", "rb").read()[:-8])
    r = run(cross, "run", "cpu_n_to_mn", tmp_path / "short.bin", tmp_path / "r.bin")
    assert r.returncode == 3 and "file ends inside matrix" in r.stderr


def test_exit_codes(cross, tmp_path):
    left, right = seeded_inputs(4, 4, 1, 1, 1)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    l, rr = tmp_path / "l.csv", tmp_path / "r.csv"
    r = run(cross, "run", "nai_fastest_ever", l, rr)
    assert r.returncode == 1 and 'Unknown algorithm "nai_fastest_ever", expected one of' in r.stderr
    assert run(cross, "run", "--bogus", "cpu_one_to_one", l, rr).returncode == 1
    assert run(cross, "run", "cpu_one_to_one", l).returncode == 1
    assert run(cross, "run", "-b", "Sometimes", "cpu_one_to_one", l, rr).returncode == 1
    assert run(cross, "run", "-d", "quad", "cpu_one_to_one", l, rr).returncode == 1      # double is accepted here
    r = run(cross, "run", "cpu_one_to_one", l, tmp_path / "missing.csv")
    assert r.returncode == 3 and "data loading step" in r.stderr
    (tmp_path / "badfft.json").write_text(json.dumps({"hadamard_threads_per_block": 0}))
    r = run(cross, "run", "--args_path", tmp_path / "badfft.json", "fft_orig_one_to_one", l, rr)
    assert r.returncode == 1 and "Invalid algorithm argument value" in r.stderr
    # wrong matrix counts for the mode, sizes that differ, broken files: computation-step errors
    write_matrices(tmp_path / "two.csv", np.zeros((2, 4, 4), np.float32))
    assert run(cross, "run", "cpu_one_to_one", l, tmp_path / "two.csv").returncode == 3
    write_matrices(tmp_path / "big.csv", np.zeros((1, 5, 4), np.float32))
    r = run(cross, "run", "cpu_one_to_one", l, tmp_path / "big.csv")
    assert r.returncode == 3 and "expected ref and target to be the same size" in r.stderr
    (tmp_path / "short.csv").write_text("# 2,2,1\n1,2\n3\n")
    r = run(cross, "run", "cpu_one_to_one", tmp_path / "short.csv", tmp_path / "short.csv")
    assert r.returncode == 3 and "too short" in r.stderr
    (tmp_path / "nohdr.csv").write_text("1,2\n3,4\n")
    assert run(cross, "run", "cpu_one_to_one", tmp_path / "nohdr.csv", tmp_path / "nohdr.csv").returncode == 3
    # algorithm arguments outside their range: exit 1 before anything is loaded
    (tmp_path / "bad.json").write_text(json.dumps({"warps_per_thread_block": 0}))
    r = run(cross, "run", "--args_path", tmp_path / "bad.json", "nai_shuffle_one_to_one", l, rr)
    assert r.returncode == 1 and "Invalid algorithm argument value" in r.stderr
    (tmp_path / "bad2.json").write_text(json.dumps({"distribution_type": "hexagon"}))
    assert run(cross, "run", "--args_path", tmp_path / "bad2.json", "nai_shuffle_work_distribution_one_to_one",
               l, rr).returncode == 1
    (tmp_path / "bad3.json").write_text(json.dumps({"shifts_per_thread_block": 16, "shared_mem_rows": 8}))
    assert run(cross, "run", "--args_path", tmp_path / "bad3.json", "nai_warp_per_shift_shared_mem_one_to_one",
               l, rr).returncode == 1
    (tmp_path / "broken.json").write_text("{ \"warps_per_thread_block\": ")
    assert run(cross, "run", "--args_path", tmp_path / "broken.json", "nai_shuffle_one_to_one", l, rr).returncode == 2


def test_double_data_type_on_the_cpu(cross, oracle, tmp_path):
    """`run --data_type double` (refused upstream, main.cpp:431-438): the cpu_* names compute in
    double from the full-precision text inputs; files, statistics and timing labels as for single."""
    rng = np.random.default_rng(5)
    left, right = rng.random((2, 7, 9)), rng.random((6, 7, 9))          # float64 values
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    r = run(cross, "run", "--data_type", "double", "--out", tmp_path / "o.csv", "--validate", "--no_progress",
            "-b", "Compute", "-m", "0.001", "-t", tmp_path / "t.csv", "cpu_n_to_mn", tmp_path / "l.csv", tmp_path / "r.csv",
            cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    import scipy.signal
    got = read_matrices(tmp_path / "o.csv")
    for t in range(3):
        for l in range(2):                       # file order: right / result t*n + l belongs to left l
            want = scipy.signal.correlate2d(left[l], right[t * 2 + l], mode="full")
            assert np.abs(got[t * 2 + l] - want).max() <= 5.1e-7
    assert r.stdout.splitlines()[0] == "Max,Mean,Stddev" and float(r.stdout.splitlines()[1].split(",")[0]) < 1e-12
    assert open(tmp_path / "t.csv").read().splitlines()[0] == "Computation,Computation_iterations"
    assert run(cross, "run", "--data_type", "half", "cpu_one_to_one", tmp_path / "l.csv", tmp_path / "r.csv").returncode == 1
    assert run(cross, "run", "--data_type", "double", "fft_orig_one_to_one", tmp_path / "l.csv", tmp_path / "r.csv").returncode == 1


@pytest.mark.gpu
@pytest.mark.parametrize("alg,mode,rows,cols,nl,nr,bench", [
    ("nai_shuffle_multirow_both_one_to_one", "one_to_one", 33, 20, 1, 1, "Algorithm"),
    ("nai_shuffle_multirow_both_multimat_right_one_to_many", "one_to_many", 16, 24, 1, 7, "CommonSteps"),
    ("nai_shuffle_multirow_both_multimat_right_n_to_mn", "n_to_mn", 12, 12, 3, 9, "Compute"),
    ("nai_orig_n_to_m", "n_to_m", 9, 17, 2, 5, "None"),
])
def test_double_data_type_on_the_gpu(cross, tmp_path, alg, mode, rows, cols, nl, nr, bench):
    """Every direct algorithm name runs its mode in double with --data_type double: result files in
    the reference's file order equal scipy's float64 correlation, the timing file carries the
    benchmark type's labels."""
    import scipy.signal
    rng = np.random.default_rng(11)
    left, right = rng.random((nl, rows, cols)), rng.random((nr, rows, cols))
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    r = run(cross, "run", "-d", "double", "-o", tmp_path / "o.csv", "-v", "-p", "-b", bench, "-m", "0.002",
            "-t", tmp_path / "t.csv", alg, tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    got = read_matrices(tmp_path / "o.csv")
    pairs = {"one_to_one": [(0, 0)], "one_to_many": [(0, t) for t in range(nr)],
             "n_to_mn": [(i % nl, i) for i in range(nr)], "n_to_m": [(l, t) for l in range(nl) for t in range(nr)]}[mode]
    assert got.shape[0] == len(pairs)
    for k, (l, t) in enumerate(pairs):
        want = scipy.signal.correlate2d(left[l], right[t], mode="full")
        assert np.abs(got[k] - want).max() <= 5.1e-7, (alg, k)
    assert float(r.stdout.splitlines()[1].split(",")[0]) < 1e-12          # --validate: CPU double recompute
    if bench != "None":
        head = open(tmp_path / "t.csv").read().splitlines()[0]
        assert head == {"Algorithm": "Kernel,Kernel_iterations", "Compute": "Computation,Computation_iterations",
                        "CommonSteps": "Load,Load_iterations,Prepare,Prepare_iterations,Transfer,Transfer_iterations,"
                                       "Run,Run_iterations,Finalize,Finalize_iterations,Free,Free_iterations,"
                                       "Store,Store_iterations"}[bench]


# ---- GPU --------------------------------------------------------------------------------------------
GPU_ALGS = [
    ("nai_orig_one_to_one", "one_to_one", 24, 24, 1, 1, {}),
    ("nai_shuffle_multirow_both_one_to_one", "one_to_one", 40, 33, 1, 1,
     {"warps_per_thread_block": 4, "shifts_per_thread": 8, "left_rows_per_iteration": 8}),
    ("nai_shuffle_work_distribution_one_to_one", "one_to_one", 32, 32, 1, 1, {"rows_per_thread": 5}),
    ("nai_warp_per_shift_one_to_one", "one_to_one", 16, 16, 1, 1, {"shifts_per_thread_block": 16}),
    ("nai_warp_per_shift_shared_mem_one_to_many", "one_to_many", 16, 20, 1, 5, {}),
    ("nai_block_per_shift_one_to_one", "one_to_one", 9, 9, 1, 1, {"block_size": 64}),
    ("nai_shuffle_multirow_both_multimat_right_one_to_many", "one_to_many", 32, 32, 1, 9,
     {"right_matrices_per_thread": 4}),
    ("nai_shuffle_multirow_both_multimat_right_n_to_mn", "n_to_mn", 16, 24, 3, 12, {}),
    ("nai_orig_n_to_mn", "n_to_mn", 8, 8, 2, 6, {}),
    ("nai_shuffle_multirow_both_multimat_both_n_to_m", "n_to_m", 24, 16, 3, 5, {}),
    ("nai_shuffle_multimat_both_work_distribution_n_to_m", "n_to_m", 20, 20, 2, 3, {"rows_per_thread": 7}),
]


@pytest.mark.gpu
@pytest.mark.parametrize("alg,mode,rows,cols,nl,nr,args", GPU_ALGS)
def test_gpu_algorithms_files_match_the_oracle(cross, oracle, tmp_path, alg, mode, rows, cols, nl, nr, args):
    """Files in, files out, in the reference's FILE order for every mode (n_to_mn: right and
    result matrix t*n + l belong to left l) -- the grouping the library wants stays inside."""
    left, right = seeded_inputs(rows, cols, nl, nr, 23)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    (tmp_path / "args.json").write_text(json.dumps(args))
    r = run(cross, "run", "--out", tmp_path / "o.csv", "--validate", "--times", tmp_path / "t.csv", "--no_progress",
            "--args_path", tmp_path / "args.json", "--benchmark_type", "Algorithm", "--outer_loops", "1",
            "--min_time", "0.01", alg, tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    want = oracle.run(mode, left, right, acc64=True)
    got = read_matrices(tmp_path / "o.csv")
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7
    # --validate (in-process CPU recompute): Max relative element error is float rounding
    stats = r.stdout.splitlines()
    assert stats[0] == "Max,Mean,Stddev" and float(stats[1].split(",")[0]) < 1e-4
    # timing CSV: Kernel, Kernel_iterations, then the algorithm's properties in registry order
    head, row = open(tmp_path / "t.csv").read().splitlines()[:2]
    cols_ = head.split(",")
    assert cols_[:2] == ["Kernel", "Kernel_iterations"]
    vals = row.split(",")
    assert len(vals) == len(cols_) and int(vals[0]) > 0 and int(vals[1]) >= 1
    for k, v in args.items():
        assert vals[cols_.index(k)] == str(v)


# one small shape per mode, ragged in both directions, counts that leave partial matrix groups
ALL_NAMES_SHAPES = {"one_to_one": (19, 21, 1, 1), "one_to_many": (18, 20, 1, 11),
                    "n_to_mn": (12, 17, 3, 9), "n_to_m": (14, 13, 3, 5)}


@pytest.mark.gpu
@pytest.mark.parametrize("alg", EXPECTED_NAMES)
def test_every_registry_name_writes_the_oracle_result(cross, oracle, tmp_path, alg):
    """Every name `cross list` prints (main.cpp:368-409), default arguments: the result file
    equals the oracle's.  FFT names are run with --normalize so that the file has the direct
    algorithms' layout."""
    mode = next(m for m in ("one_to_one", "one_to_many", "n_to_mn", "n_to_m") if alg.endswith(m))
    rows, cols, nl, nr = ALL_NAMES_SHAPES[mode]
    left, right = seeded_inputs(rows, cols, nl, nr, 41)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    extra = ["--normalize"] if alg.startswith("fft") else []
    r = run(cross, "run", "--out", tmp_path / "o.csv", *extra, alg, tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    want = oracle.run(mode, left, right, acc64=True)
    got = read_matrices(tmp_path / "o.csv")
    assert got.shape == want.shape
    # the file holds six decimals (matrix.hpp:169-185): half a unit of the last one on top of the tolerance
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7, alg


STAGED_KEYS = [
    ("nai_warp_per_shift_shared_mem_one_to_one", "one_to_one", 40, 37, 1, 1,
     {"shifts_per_thread_block": 4, "shared_mem_row_size": 16, "shared_mem_rows": 8}),
    ("nai_warp_per_shift_shared_mem_one_to_one", "one_to_one", 33, 70, 1, 1,
     {"shifts_per_thread_block": 8, "shared_mem_row_size": 32, "shared_mem_rows": 8, "column_group_per_block": True}),
    ("nai_warp_per_shift_shared_mem_one_to_one", "one_to_one", 21, 50, 1, 1,
     {"shifts_per_thread_block": 16, "shared_mem_rows": 16, "strided_load": False}),
    ("nai_warp_per_shift_shared_mem_one_to_many", "one_to_many", 20, 24, 1, 13,
     {"shifts_per_thread_block": 8, "shared_mem_rows": 12, "right_matrices_per_block": 3}),
    ("nai_warp_per_shift_shared_mem_n_to_mn", "n_to_mn", 16, 18, 3, 15,
     {"right_matrices_per_block": 4, "column_group_per_block": True, "shared_mem_row_size": 8}),
    ("nai_warp_per_shift_shared_mem_n_to_m", "n_to_m", 17, 16, 2, 9,
     {"right_matrices_per_block": 8, "strided_load": False}),
    ("nai_warp_per_shift_work_distribution_one_to_one", "one_to_one", 30, 22, 1, 1,
     {"rows_per_warp": 4, "distribution_type": "rectangle"}),
    ("nai_warp_per_shift_work_distribution_one_to_one", "one_to_one", 30, 22, 1, 1,
     {"rows_per_warp": 7, "distribution_type": "triangle"}),
    ("nai_warp_per_shift_work_distribution_one_to_one", "one_to_one", 9, 40, 1, 1,
     {"rows_per_warp": 2, "distribution_type": "none"}),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", range(len(STAGED_KEYS)))
def test_warp_per_overlap_families_honour_their_keys(cross, oracle, tmp_path, case):
    """The shared-memory warp-per-overlap names and the row-split one: every JSON key of the
    reference's classes (one_to_one.hpp:470-680, one_to_many.hpp:395-499) shapes the launch --
    the results under each setting equal the oracle's, and the timing file echoes the values."""
    alg, mode, rows, cols, nl, nr, args = STAGED_KEYS[case]
    left, right = seeded_inputs(rows, cols, nl, nr, 43 + case)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    (tmp_path / "args.json").write_text(json.dumps(args))
    r = run(cross, "run", "--out", tmp_path / "o.csv", "--times", tmp_path / "t.csv", "--args_path", tmp_path / "args.json",
            "--benchmark_type", "Algorithm", "--min_time", "0.002", alg, tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    want = oracle.run(mode, left, right, acc64=True)
    got = read_matrices(tmp_path / "o.csv")
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7
    head, row = open(tmp_path / "t.csv").read().splitlines()[:2]
    for k, v in args.items():
        shown = {True: "1", False: "0"}.get(v, str(v)) if isinstance(v, bool) else str(v)
        assert row.split(",")[head.split(",").index(k)] == shown


@pytest.mark.gpu
def test_gpu_property_columns_follow_the_reference_order(cross, tmp_path):
    left, right = seeded_inputs(16, 16, 2, 4, 2)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    r = run(cross, "run", "-b", "Algorithm", "-m", "0.001", "-t", tmp_path / "t.csv",
            "nai_warp_per_shift_shared_mem_n_to_m", tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    head, row = open(tmp_path / "t.csv").read().splitlines()
    assert head == ("Kernel,Kernel_iterations,shifts_per_thread_block,shared_mem_row_size,shared_mem_rows,"
                    "strided_load,column_group_per_block,right_matrices_per_block,num_cuda_streams")
    assert row.split(",")[2:] == ["16", "32", "16", "1", "0", "8", "8"]


@pytest.mark.gpu
def test_gpu_devices_option_shards_without_changing_results(cross, tmp_path):
    import torch
    ndev = min(torch.cuda.device_count(), 2)
    left, right = seeded_inputs(16, 16, 4, 8, 5)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    outs = []
    for nd in sorted({1, ndev}):
        r = run(cross, "run", "--devices", nd, "-o", tmp_path / f"o{nd}.csv",
                "nai_shuffle_multirow_both_multimat_both_n_to_m", tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
        assert r.returncode == 0, r.stderr
        outs.append(read_matrices(tmp_path / f"o{nd}.csv"))
    # automatic plans depend on the shard's matrix counts, so sums may be taken in another order
    for o in outs:
        assert o.shape == outs[0].shape
        assert np.abs(o - outs[0]).max() <= 2e-6 * np.abs(outs[0]).max() + 1.1e-6
    r = run(cross, "run", "--devices", 99, "nai_orig_n_to_m", tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 2 and "--devices" in r.stderr


FFT_ALGS = [
    ("fft_orig_one_to_one", "one_to_one", 16, 16, 1, 1, {"hadamard_threads_per_block": 128}),
    ("fft_reduced_transfer_one_to_one", "one_to_one", 13, 10, 1, 1, {}),
    ("fft_orig_one_to_many", "one_to_many", 12, 12, 1, 5, {}),
    ("fft_reduced_transfer_n_to_mn", "n_to_mn", 8, 10, 2, 6, {"scatter_items_per_thread": 4}),
    ("fft_better_n_to_m", "n_to_m", 9, 9, 2, 3, {}),
]


@pytest.mark.gpu
@pytest.mark.parametrize("alg,mode,rows,cols,nl,nr,args", FFT_ALGS)
def test_fft_algorithms_raw_and_normalized_files(cross, oracle, tmp_path, alg, mode, rows, cols, nl, nr, args):
    """The FFT registry names: without --normalize the output file holds the raw inverse
    transforms (2H x 2W per pair, as the reference's fft classes store them) and
    `cross validate --normalize` brings them to the template's layout; with --normalize the
    file is directly comparable with the direct algorithms' output."""
    left, right = seeded_inputs(rows, cols, nl, nr, 29)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    (tmp_path / "args.json").write_text(json.dumps(args))
    want = oracle.run(mode, left, right, acc64=True)
    write_matrices(tmp_path / "valid.csv", want.astype(np.float32))
    common = ["--args_path", tmp_path / "args.json", "--no_progress", "--benchmark_type", "Algorithm",
              "--min_time", "0.005", "--times", tmp_path / "t.csv"]
    r = run(cross, "run", "--out", tmp_path / "norm.csv", "--normalize", "--validate", *common, alg,
            tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    got = read_matrices(tmp_path / "norm.csv")
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7
    assert float(r.stdout.splitlines()[1].split(",")[0]) < 1e-3
    head, row = open(tmp_path / "t.csv").read().splitlines()[:2]
    assert head.split(",")[:2] == ["Kernel", "Kernel_iterations"]
    for k, v in args.items():
        assert row.split(",")[head.split(",").index(k)] == str(v)
    # raw result file
    r = run(cross, "run", "--out", tmp_path / "raw.csv", "--validate", "--no_progress", alg,
            tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert float(r.stdout.splitlines()[1].split(",")[0]) < 1e-3
    raw = read_matrices(tmp_path / "raw.csv")
    assert raw.shape == (want.shape[0], 2 * rows, 2 * cols)
    assert abs(raw[0, 0, 0] / (4.0 * rows * cols) - want[0, rows - 1, cols - 1]) <= 1e-4 * np.abs(want).max()
    r = run(cross, "validate", "--normalize", "-c", "-p", tmp_path / "valid.csv", tmp_path / "raw.csv")
    assert r.returncode == 0, r.stderr
    assert float(r.stdout.splitlines()[1].split(",")[0]) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("alg,mode,nl,nr", [("nai_shuffle_multirow_both_multimat_right_one_to_many", "one_to_many", 1, 40),
                                            ("nai_shuffle_multirow_both_multimat_both_n_to_m", "n_to_m", 6, 7),
                                            ("nai_shuffle_multirow_both_multimat_right_n_to_mn", "n_to_mn", 4, 12),
                                            ("fft_orig_one_to_many", "one_to_many", 1, 9)])
def test_pipelined_computation_steps(cross, oracle, tmp_path, alg, mode, nl, nr):
    """--pipelined (or XCORR_PIPELINED=1): transfer, kernels and copy-back as one overlapped call
    of the host-buffer entry point; same files, `Computation` timing in Compute mode."""
    left, right = seeded_inputs(40, 48, nl, nr, 31)
    write_matrices(tmp_path / "l.csv", left)
    write_matrices(tmp_path / "r.csv", right)
    want = oracle.run(mode, left, right, acc64=True)
    extra = ["--normalize"] if alg.startswith("fft") else []
    r = run(cross, "run", "--pipelined", "-b", "Compute", "-m", "0.005", "-t", tmp_path / "t.csv", "-o", tmp_path / "o.csv",
            *extra, alg, tmp_path / "l.csv", tmp_path / "r.csv", cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    got = read_matrices(tmp_path / "o.csv")
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7
    assert open(tmp_path / "t.csv").read().splitlines()[0].startswith("Computation,Computation_iterations")
    env = dict(os.environ, XCORR_PIPELINED="1")
    r = subprocess.run([cross, "run", "-o", str(tmp_path / "o2.csv"), *extra, alg, str(tmp_path / "l.csv"),
                        str(tmp_path / "r.csv")], cwd=tmp_path, env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert np.abs(read_matrices(tmp_path / "o2.csv") - want).max() <= 1e-5 * np.abs(want).max() + 5.1e-7
