"""Tests of the benchmark driver (jpdc23-artifact_b200/benchmark/benchmark.py): a definition in
the reference's benchmark.yml format is expanded into runs, measured through `cross`, stored under
the reference's file names and summarised.  CPU tests use the cpu_* algorithms."""
import csv
import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "jpdc23-artifact_b200", "benchmark", "benchmark.py")

DEFINITION = """
benchmark:
  name: small
  config:
    min_measure_seconds: 0.01
    data_type: single
  groups:
    - name: many
      config:
        sizes: ["8x8x1x3", "6x10x1x2"]
        benchmark_type: Compute
        inner_iterations: 2
        outer_iterations: 2
      runs:
        - name: plain
          algorithm: {alg_many}
        - name: fan
          algorithm: {alg_many}
          args:
            warps_per_thread_block: [4, 8]
            shifts_per_thread: [2]
            left_rows_per_iteration: [1, 2]
    - name: pairs
      config:
        sizes: ["5x7x2x6"]
        benchmark_type: {pairs_type}
      runs:
        - algorithm: {alg_n2mn}
"""


@pytest.fixture(scope="module")
def driver():
    spec = importlib.util.spec_from_file_location("xcorr_benchmark_driver", DRIVER)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def cross(xc):
    if not os.path.exists(xc.CROSS_PATH):
        xc.build()
    return xc.CROSS_PATH


def drive(*args):
    return subprocess.run([sys.executable, DRIVER, *map(str, args)], capture_output=True, text=True, timeout=900)


def test_argument_lists_fan_out_like_the_reference(driver):
    runs = driver.expand_runs(3, dict(name="mb", algorithm="nai_shuffle_multirow_both_one_to_one",
                                      args=dict(warps_per_thread_block=[4, 8], shifts_per_thread=[1, 2, 4],
                                                left_rows_per_iteration=[2], note="x")))
    assert len(runs) == 6
    assert runs[0]["name"] == "mb__4_1__" and runs[-1]["name"] == "mb__8_4__"
    assert all(r["alg_type"] == "one_to_one" and r["idx"] == 3 for r in runs)
    assert runs[1]["args"] == dict(left_rows_per_iteration=2, note="x", warps_per_thread_block=4, shifts_per_thread=2)
    single = driver.expand_runs(0, dict(algorithm="cpu_n_to_mn"))
    assert [r["name"] for r in single] == ["0_cpu_n_to_mn____"] and single[0]["alg_type"] == "n_to_mn"
    with pytest.raises(ValueError):
        driver.expand_runs(0, dict(algorithm="nonsense"))
    assert driver.parse_size("16x24x2x8") == (16, 24, 2, 8)
    with pytest.raises(ValueError):
        driver.parse_size("16x24x2")
    assert [driver.pairs_of(t, 4, 8) for t in ("one_to_one", "one_to_many", "n_to_mn", "n_to_m")] == [1, 8, 8, 32]


def check_results(out, driver, n_fan):
    res = out / "many" / "results"
    names = sorted(p.name for p in res.iterdir())
    assert "0-0-plain____-8x8x1x3-time.csv" in names and "0-1-plain____-6x10x1x2-time.csv" in names
    assert sum(n.startswith("1-0-fan__") for n in names) == n_fan
    with (res / "0-0-plain____-8x8x1x3-time.csv").open() as f:
        rows = list(csv.reader(f))
    assert rows[0][:2] == ["Computation", "Computation_iterations"]    # GPU algorithms append their properties
    assert len(rows) == 1 + 2 * 2                      # outer x inner iterations, appended
    meta = json.loads((out / "many" / "group.json").read_text())
    assert meta["config"]["benchmark_type"] == "Compute" and len(meta["runs"]) == 1 + n_fan
    records = driver.summarise(out)
    assert len(records) == 2 * (1 + n_fan) + 1
    for r in records:
        assert r["time_ns"] > 0 and r["ns_per_fma"] > 0 and r["gflops"] > 0
    r0 = next(r for r in records if r["size"] == "8x8x1x3" and r["run"] == "plain____")
    assert r0["ns_per_fma"] == pytest.approx(r0["time_ns"] / (3 * 8 ** 4))
    assert r0["ns_per_overlap"] == pytest.approx(r0["time_ns"] / (3 * 15 * 15))


def test_cpu_groups_are_measured_stored_and_summarised(driver, cross, tmp_path):
    definition = tmp_path / "def.yml"
    definition.write_text(DEFINITION.format(alg_many="cpu_one_to_many", alg_n2mn="cpu_n_to_mn", pairs_type="Compute"))
    out = tmp_path / "out"
    p = drive("-e", cross, "benchmark", definition, "-o", out)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "measured 11, skipped 0, failed 0" in p.stdout
    check_results(out, driver, n_fan=4)
    assert (out / "many" / "inputs" / "0-left-8x8x1x3.bin").stat().st_size == 20 + 4 * 64
    # continue: nothing to do; one group only; rerun measures again
    p = drive("-e", cross, "benchmark", "-c", definition, "-o", out)
    assert "measured 0, skipped 11, failed 0" in p.stdout
    p = drive("-e", cross, "benchmark", "-r", definition, "pairs", "-o", out)
    assert "measured 1, skipped 0, failed 0" in p.stdout
    p = drive("summary", out)
    assert p.returncode == 0 and "11 measurements" in p.stdout and (out / "summary.csv").exists()
    p = drive("clear", definition, "pairs", "-o", out)
    assert p.returncode == 0 and not (out / "pairs").exists() and (out / "many").exists()
    assert drive("benchmark", definition, "nosuchgroup", "-o", out).returncode != 0
    # text inputs in the reference's CSV format
    p = drive("-e", cross, "benchmark", "--text", definition, "pairs", "-o", tmp_path / "text")
    assert p.returncode == 0, p.stdout + p.stderr
    head = (tmp_path / "text" / "pairs" / "inputs" / "0-right-5x7x2x6.csv").read_text().splitlines()[0]
    assert head == "# 5,7,6"


def test_failed_runs_are_logged_and_counted(cross, tmp_path):
    definition = tmp_path / "def.yml"
    definition.write_text(DEFINITION.format(alg_many="cpu_one_to_many", alg_n2mn="cpu_no_such_n_to_mn",
                                            pairs_type="Compute"))
    p = drive("-e", cross, "benchmark", definition, "pairs", "-o", tmp_path / "out")
    assert p.returncode == 1 and "failed 1" in p.stdout
    assert "0_cpu_no_such_n_to_mn____" in (tmp_path / "out" / "pairs" / "failed_runs.log").read_text()


@pytest.mark.gpu
def test_gpu_groups_with_the_reference_argument_names(driver, cross, tmp_path):
    """The registry names and tuning keys of the reference's benchmark.yml run unchanged; Algorithm
    mode yields the Kernel column that the summary reads."""
    definition = tmp_path / "def.yml"
    definition.write_text(DEFINITION.format(alg_many="nai_shuffle_multirow_both_multimat_right_one_to_many",
                                            alg_n2mn="nai_shuffle_multirow_both_multimat_right_n_to_mn",
                                            pairs_type="Algorithm"))
    out = tmp_path / "out"
    p = drive("-e", cross, "benchmark", definition, "-o", out)
    assert p.returncode == 0, p.stdout + p.stderr
    check_results(out, driver, n_fan=4)
    with (out / "pairs" / "results" / "0-0-0_nai_shuffle_multirow_both_multimat_right_n_to_mn____-5x7x2x6-time.csv").open() as f:
        assert next(csv.reader(f))[0] == "Kernel"
