"""Shared fixtures: marker registration, loaders for the package (by path: its directory
name has a hyphen) and for the CPU checkers under oracle/, seeded inputs."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_INIT = os.path.join(ROOT, "jpdc23-artifact_b200", "__init__.py")
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the GPU box)")


def load_package():
    name = "jpdc23_artifact_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, PKG_INIT)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def xc():
    mod = load_package()
    if not os.path.exists(mod.LIB_PATH):
        mod.build()
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def oracle():
    import pyoracle
    return pyoracle.Oracle()


@pytest.fixture(scope="session")
def reference():
    import pyoracle
    if not pyoracle.Reference.available():
        pytest.skip("oracle/_ref/libxcorr_ref.so not built on this machine")
    return pyoracle.Reference()


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "reference_cases.npz")
    data = np.load(path)
    cases = []
    for line in data["cases"]:
        name, mode, rows, cols, nl, nr, seed = str(line).split("|")
        cases.append(dict(name=name, mode=mode, rows=int(rows), cols=int(cols), n_left=int(nl),
                          n_right=int(nr), seed=int(seed),
                          left=data[f"{name}/left"], right=data[f"{name}/right"],
                          f32=data[f"{name}/f32"], f64=data[f"{name}/f64"]))
    return cases


def seeded_inputs(rows, cols, n_left, n_right, seed):
    """uniform[0,1) float32 -- the value distribution of the reference's input generator
    (benchmark/input_generator.py:20-32), seeded."""
    left = np.random.default_rng(seed).random((n_left, rows, cols), dtype=np.float32)
    right = np.random.default_rng(seed + 1000).random((n_right, rows, cols), dtype=np.float32)
    return left, right


def grouped_to_file(a, n_left):
    """n_to_mn result/right array from grouped order (l*m + t) to file order (t*n + l)."""
    m = a.shape[0] // n_left
    return np.ascontiguousarray(a.reshape(n_left, m, *a.shape[1:]).swapaxes(0, 1)).reshape(a.shape)


def file_to_grouped(a, n_left):
    m = a.shape[0] // n_left
    return np.ascontiguousarray(a.reshape(m, n_left, *a.shape[1:]).swapaxes(0, 1)).reshape(a.shape)
