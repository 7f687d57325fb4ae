#!/usr/bin/env python3
"""Benchmark driver for the `cross` executable: reads a benchmark definition in the format of the
reference's benchmark/benchmark.yml (groups -> config {sizes, data_type, benchmark_type,
outer_iterations, inner_iterations, min_measure_seconds, validate, keep} and runs {name, algorithm,
args with lists that fan out into every combination}), generates the inputs, runs every
(size, run, argument combination) through `cross run` and leaves one timing CSV per measurement,
named as the reference names them (benchmark/benchmark.py:517-524,
`<run idx>-<input idx>-<run name>-<size>-time.csv`), so scripts that read the reference's result
folders read these.  Written on PyYAML (the reference needs ruamel.yaml).

    benchmark.py benchmark definition.yml [group ...] -o out_dir [-e path/to/cross] [-r | -c] [-v]
    benchmark.py summary out_dir            # time per FMA / per overlap, best run per size
    benchmark.py clear definition.yml [group ...] -o out_dir
    benchmark.py list [-e path/to/cross]

Differences from the reference driver: inputs are seeded (group index, size index) and written as
binary matrix files (`.bin`; `--text` writes the reference's CSV text); `summary` prints tables
where the reference plots with R; external (non-`cross`) runs are not supported.
"""
from __future__ import annotations

import argparse
import csv
import itertools
import json
import re
import shutil
import struct
import subprocess as sp
import sys
from pathlib import Path

import numpy as np
import yaml

HERE = Path(__file__).resolve().parent
DEFAULT_EXE = HERE.parent / "bin" / "cross"
ALG_TYPE = re.compile(r".*_([^_]+_to_[^_]+)$")


def parse_size(text: str) -> tuple[int, int, int, int]:
    """'rows x cols x left matrices x right matrices' (benchmark.yml: sizes)."""
    parts = [int(p) for p in str(text).lower().split("x")]
    if len(parts) != 4 or min(parts) <= 0:
        raise ValueError(f"size must be ROWSxCOLSxLEFTxRIGHT with positive numbers, got {text!r}")
    return parts[0], parts[1], parts[2], parts[3]


def pairs_of(alg_type: str, n_left: int, n_right: int) -> int:
    return {"one_to_one": 1, "one_to_many": n_right, "n_to_mn": n_right, "n_to_m": n_left * n_right}[alg_type]


def write_matrices(path: Path, rows: int, cols: int, count: int, seed: int, text: bool) -> None:
    """uniform[0,1) matrices, stacked; binary `XCORRMAT` file or the reference's CSV text
    (benchmark/input_generator.py:20-32: header '# rows,cols,count', %.18e values)."""
    values = np.random.default_rng(seed).random((count * rows, cols))
    if text:
        np.savetxt(path, values, delimiter=",", header=f"{rows},{cols},{count}")
    else:
        with path.open("wb") as f:
            f.write(b"XCORRMAT" + struct.pack("<III", cols, rows, count))
            f.write(values.astype("<f4").tobytes())


def expand_runs(idx: int, data: dict) -> list[dict]:
    """One run entry -> one run per combination of its list-valued arguments
    (benchmark/benchmark.py:112-153; same names: base__v1_v2__)."""
    algorithm = data["algorithm"]
    m = ALG_TYPE.fullmatch(algorithm)
    if not m:
        raise ValueError(f"invalid algorithm name {algorithm}")
    base = data.get("name", f"{idx}_{algorithm}")
    args = data.get("args", {}) or {}
    generate = {k: v for k, v in args.items() if isinstance(v, list) and len(v) > 1}
    singles = {k: (v[0] if isinstance(v, list) else v) for k, v in args.items() if k not in generate}
    if not generate:
        return [dict(idx=idx, name=f"{base}____", algorithm=algorithm, alg_type=m.group(1), args=singles)]
    keys = list(generate)
    runs = []
    for combo in itertools.product(*(generate[k] for k in keys)):
        suffix = "_".join(str(v) for v in combo)
        runs.append(dict(idx=idx, name=f"{base}__{suffix}__", algorithm=algorithm, alg_type=m.group(1),
                         args={**singles, **dict(zip(keys, combo))}))
    return runs


DEFAULTS = dict(data_type="single", benchmark_type="Compute", outer_iterations=1, inner_iterations=1,
                min_measure_seconds=1.0, validate=False, keep=False)


def load_definition(path: Path) -> dict:
    data = yaml.safe_load(path.read_text())
    bench = data["benchmark"]
    if "groups" not in bench:
        raise ValueError("benchmark definition has no groups")
    return bench


def group_config(bench: dict, group: dict) -> dict:
    cfg = dict(DEFAULTS)
    cfg.update(bench.get("config", {}) or {})
    cfg.update(group.get("config", {}) or {})
    if "sizes" not in cfg:
        raise ValueError(f"group {group.get('name')} has no sizes")
    return cfg


def result_paths(result_dir: Path, run: dict, in_idx: int, size: str) -> tuple[Path, Path]:
    stem = f"{run['idx']}-{in_idx}-{run['name']}-{size}"
    return result_dir / f"{stem}-time.csv", result_dir / f"{stem}-output_stats.csv"


def cross_command(exe: Path, run: dict, cfg: dict, args_path: Path, left: Path, right: Path, times: Path,
                  append: bool, out_path: Path | None, validate: bool) -> list[str]:
    """The command line the reference's driver builds (benchmark/external/executable.py:117-145)."""
    cmd = [str(exe), "run"]
    if out_path is not None:
        cmd += ["--out", str(out_path)]
    if validate:
        cmd += ["--validate"]
    if append:
        cmd += ["--append"]
    cmd += ["--times", str(times), "--no_progress", "--args_path", str(args_path),
            "--data_type", str(cfg["data_type"]), "--benchmark_type", str(cfg["benchmark_type"]),
            "--outer_loops", str(cfg["inner_iterations"]), "--min_time", str(cfg["min_measure_seconds"]),
            run["algorithm"], str(left), str(right)]
    return cmd


def run_group(bench: dict, g_idx: int, group: dict, out_dir: Path, exe: Path, policy: str, text: bool,
              verbose: bool) -> tuple[int, int, int]:
    """Runs one group; returns (measured, skipped, failed)."""
    cfg = group_config(bench, group)
    gdir = out_dir / group["name"]
    in_dir, res_dir, data_dir = gdir / "inputs", gdir / "results", gdir / "outputs"
    if policy == "rerun" and res_dir.exists():
        shutil.rmtree(res_dir)
    for d in (in_dir, res_dir):
        d.mkdir(parents=True, exist_ok=True)
    runs = [r for i, entry in enumerate(group["runs"]) for r in expand_runs(i, entry)]
    (gdir / "group.json").write_text(json.dumps(dict(name=group["name"], config=cfg, runs=runs), indent=1))
    measured = skipped = failed = 0
    ext = "csv" if text else "bin"
    for in_idx, size in enumerate(cfg["sizes"]):
        rows, cols, n_left, n_right = parse_size(size)
        left, right = in_dir / f"{in_idx}-left-{size}.{ext}", in_dir / f"{in_idx}-right-{size}.{ext}"
        if not left.exists():
            write_matrices(left, rows, cols, n_left, 1000 + 100 * g_idx + in_idx, text)
        if not right.exists():
            write_matrices(right, rows, cols, n_right, 2000 + 100 * g_idx + in_idx, text)
        for run in runs:
            times, _ = result_paths(res_dir, run, in_idx, size)
            if policy == "continue" and times.exists() and times.stat().st_size > 0:
                skipped += 1
                continue
            args_path = in_dir / f"{run['idx']}-{run['name']}-args.json"
            args_path.write_text(json.dumps(run["args"]))
            ok = True
            for it in range(int(cfg["outer_iterations"])):
                out_path = None
                if cfg["keep"]:
                    odir = data_dir / times.name[:-len("-time.csv")]
                    odir.mkdir(parents=True, exist_ok=True)
                    out_path = odir / f"{it}.csv"
                cmd = cross_command(exe, run, cfg, args_path, left, right, times, it != 0, out_path,
                                    bool(cfg["validate"]))
                if verbose:
                    print("Command:", " ".join(cmd))
                res = sp.run(cmd, capture_output=True, text=True)
                if res.returncode != 0:
                    ok = False
                    with (gdir / "failed_runs.log").open("a") as f:
                        f.write(f"{run['idx']} {in_idx} {run['name']} {size}: exit {res.returncode}: "
                                f"{(res.stderr or res.stdout).strip()[:500]}\n")
                    if times.exists():
                        times.unlink()
                    break
            measured += ok
            failed += not ok
            print(f"[{group['name']}] {size} {run['name']}: {'ok' if ok else 'FAILED'}", flush=True)
    return measured, skipped, failed


# The label of the time column that a benchmark type's CSV is summarised by.
MAIN_LABEL = {"Algorithm": "Kernel", "Compute": "Computation", "CommonSteps": "Run"}


def read_times(path: Path) -> dict[str, float]:
    """Mean of every time column (ns) of a `cross --times` file; '<label>_iterations' columns dropped."""
    with path.open() as f:
        rows = [r for r in csv.reader(f) if r]
    if len(rows) < 2:
        return {}
    cols = {}
    for j, label in enumerate(rows[0]):
        if label.endswith("_iterations"):
            continue
        try:
            vals = [float(r[j]) for r in rows[1:] if j < len(r) and r[j] != ""]
        except ValueError:               # a property column of the algorithm (e.g. a distribution name)
            continue
        if vals:
            cols[label] = sum(vals) / len(vals)
    return cols


def summarise(out_dir: Path) -> list[dict]:
    """One record per measurement: mean time, time per FMA and per overlap -- the quantities of the
    reference's plots (plots/plot_n_to_m.R:30,58) -- and GFLOP/s."""
    records = []
    for gfile in sorted(out_dir.glob("*/group.json")):
        meta = json.loads(gfile.read_text())
        label = MAIN_LABEL.get(str(meta["config"]["benchmark_type"]), "Computation")
        for in_idx, size in enumerate(meta["config"]["sizes"]):
            rows, cols, n_left, n_right = parse_size(size)
            for run in meta["runs"]:
                times, _ = result_paths(gfile.parent / "results", run, in_idx, size)
                if not times.exists():
                    continue
                t = read_times(times)
                ns = t.get(label, next(iter(t.values()), None) if t else None)
                if ns is None or ns <= 0:
                    continue
                pairs = pairs_of(run["alg_type"], n_left, n_right)
                fma = pairs * rows * rows * cols * cols
                overlaps = pairs * (2 * rows - 1) * (2 * cols - 1)
                records.append(dict(group=meta["name"], size=size, run=run["name"], algorithm=run["algorithm"],
                                    args=json.dumps(run["args"], sort_keys=True), time_ns=ns,
                                    ns_per_fma=ns / fma, ns_per_overlap=ns / overlaps,
                                    gflops=2.0 * fma / ns))
    return records


def print_summary(out_dir: Path) -> int:
    records = summarise(out_dir)
    if not records:
        print("no measurements found under", out_dir)
        return 1
    with (out_dir / "summary.csv").open("w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(records[0]))
        w.writeheader()
        w.writerows(records)
    best: dict[tuple[str, str], dict] = {}
    for r in records:
        key = (r["group"], r["size"])
        if key not in best or r["time_ns"] < best[key]["time_ns"]:
            best[key] = r
    print(f"{'group':24s} {'size':20s} {'best run':44s} {'time us':>11s} {'ps/FMA':>9s} {'ns/overlap':>11s} {'GFLOP/s':>10s}")
    for (group, size), r in best.items():
        print(f"{group:24s} {size:20s} {r['run']:44s} {r['time_ns'] / 1e3:11.2f} {r['ns_per_fma'] * 1e3:9.3f} "
              f"{r['ns_per_overlap']:11.3f} {r['gflops']:10.1f}")
    print(f"{len(records)} measurements -> {out_dir / 'summary.csv'}")
    return 0


def selected_groups(bench: dict, names: list[str]) -> list[tuple[int, dict]]:
    groups = list(enumerate(bench["groups"]))
    if not names:
        return groups
    known = {g["name"] for _, g in groups}
    for n in names:
        if n not in known and not (n.isdigit() and int(n) < len(groups)):
            raise SystemExit(f"unknown group {n!r}; the definition has: {', '.join(sorted(known))}")
    return [(i, g) for i, g in groups if g["name"] in names or str(i) in names]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-e", "--executable_path", type=Path, default=DEFAULT_EXE, help="the cross executable")
    sub = ap.add_subparsers(dest="command", required=True)
    b = sub.add_parser("benchmark", help="run the groups of a benchmark definition")
    ex = b.add_mutually_exclusive_group()
    ex.add_argument("-r", "--rerun", action="store_true", help="delete earlier results of the groups first")
    ex.add_argument("-c", "--cont", action="store_true", help="keep earlier results, measure what is missing")
    b.add_argument("-o", "--output_path", type=Path, default=Path("output"))
    b.add_argument("-v", "--verbose", action="store_true")
    b.add_argument("--text", action="store_true", help="inputs as the reference's CSV text instead of binary files")
    b.add_argument("benchmark_definition_path", type=Path)
    b.add_argument("groups", nargs="*")
    c = sub.add_parser("clear", help="delete inputs and results of the groups")
    c.add_argument("-o", "--output_path", type=Path, default=Path("output"))
    c.add_argument("benchmark_definition_path", type=Path)
    c.add_argument("groups", nargs="*")
    s = sub.add_parser("summary", help="tables of time per FMA / per overlap from a result folder")
    s.add_argument("output_path", type=Path)
    sub.add_parser("list", help="algorithms of the executable")
    a = ap.parse_args(argv)

    if a.command == "list":
        return sp.run([str(a.executable_path), "list"]).returncode
    if a.command == "summary":
        return print_summary(a.output_path)
    bench = load_definition(a.benchmark_definition_path)
    groups = selected_groups(bench, a.groups)
    if a.command == "clear":
        for _, g in groups:
            shutil.rmtree(a.output_path / g["name"], ignore_errors=True)
        return 0
    if not a.executable_path.exists():
        raise SystemExit(f"executable {a.executable_path} not found (build it with `make -C jpdc23-artifact_b200`)")
    policy = "rerun" if a.rerun else "continue" if a.cont else "overwrite"
    totals = [0, 0, 0]
    for g_idx, g in groups:
        for k, v in enumerate(run_group(bench, g_idx, g, a.output_path, a.executable_path, policy, a.text, a.verbose)):
            totals[k] += v
    print(f"measured {totals[0]}, skipped {totals[1]}, failed {totals[2]}")
    return 1 if totals[2] else 0


if __name__ == "__main__":
    sys.exit(main())
