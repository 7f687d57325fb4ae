"""CPU tests of the checkers themselves: the C restatement against the committed fixtures
(produced by the reference's own CPU code) and, where it is built, against that code live."""
import numpy as np
import pytest
from scipy.signal import correlate2d

from conftest import seeded_inputs


def test_oracle_matches_golden_bitwise(oracle, golden):
    assert len(golden) >= 10
    for c in golden:
        f32 = oracle.run(c["mode"], c["left"], c["right"], acc64=False)
        f64 = oracle.run(c["mode"], c["left"], c["right"], acc64=True)
        assert f32.dtype == np.float32 and f32.shape == c["f32"].shape, c["name"]
        assert np.array_equal(f32, c["f32"]), c["name"]      # same loop order, same rounding
        assert np.array_equal(f64, c["f64"]), c["name"]


def test_golden_inputs_are_reproducible(golden):
    for c in golden:
        left, right = seeded_inputs(c["rows"], c["cols"], c["n_left"], c["n_right"], c["seed"])
        assert np.array_equal(left, c["left"]) and np.array_equal(right, c["right"]), c["name"]


@pytest.mark.parametrize("mode,rows,cols,nl,nr", [
    ("one_to_one", 2, 9, 1, 1), ("one_to_one", 31, 33, 1, 1), ("one_to_many", 9, 6, 1, 4),
    ("n_to_mn", 7, 7, 2, 6), ("n_to_m", 10, 3, 3, 2)])
def test_oracle_matches_reference_live(oracle, reference, mode, rows, cols, nl, nr):
    left, right = seeded_inputs(rows, cols, nl, nr, 7 + rows)
    assert np.array_equal(oracle.run(mode, left, right), reference.run(mode, left, right))
    assert np.array_equal(oracle.run(mode, left, right, acc64=True),
                          reference.run(mode, left, right, acc64=True))


def test_oracle_definition_known_answers(oracle):
    # corners and centre of the definition (validate.hpp:95-132)
    left = np.arange(1, 13, dtype=np.float32).reshape(3, 4)
    right = np.arange(2, 14, dtype=np.float32).reshape(3, 4)
    out = oracle.run("one_to_one", left, right, acc64=True)[0]
    assert out.shape == (5, 7)
    assert out[0, 0] == left[0, 0] * right[2, 3]          # shift (-(W-1), -(H-1))
    assert out[-1, -1] == left[2, 3] * right[0, 0]
    assert out[2, 3] == float((left * right).sum())       # zero shift = dot product
    assert np.allclose(out, correlate2d(left.astype(np.float64), right.astype(np.float64), "full"))


def test_oracle_agrees_with_scipy(oracle):
    left, right = seeded_inputs(13, 21, 1, 1, 99)
    out = oracle.run("one_to_one", left, right, acc64=True)[0]
    ref = correlate2d(left[0].astype(np.float64), right[0].astype(np.float64), "full")
    assert np.abs(out - ref).max() <= 1e-12 * np.abs(ref).max()


def test_oracle_threads_do_not_change_results(oracle):
    left, right = seeded_inputs(9, 8, 3, 6, 5)
    for mode in ("one_to_many", "n_to_mn", "n_to_m"):
        l = left[:1] if mode == "one_to_many" else left
        assert np.array_equal(oracle.run(mode, l, right, threads=1), oracle.run(mode, l, right, threads=4))


def test_oracle_rejects_bad_counts(oracle):
    left, right = seeded_inputs(4, 4, 3, 7, 1)
    with pytest.raises(RuntimeError):
        oracle.run("n_to_mn", left, right)                 # 7 % 3 != 0 (validate.hpp:254-261)


def test_validate_statistics_match_reference(oracle, reference):
    rng = np.random.default_rng(3)
    valid = rng.random(500)
    result = valid * (1 + 1e-6 * rng.standard_normal(500))
    result[:5] = 0.0
    valid[:5] = 1e-7                                       # both tiny -> error forced to 0
    for f32 in (True, False):
        a = oracle.validate(result, valid, elem_f32=f32)
        b = reference.validate(result, valid, elem_f32=f32)
        assert np.allclose(a[:3], b[:3], rtol=1e-12, atol=0)


def test_interleave_index_is_its_own_inverse(oracle):
    n, m = 3, 5
    seen = set()
    for i in range(n * m):
        g = oracle.interleaved_index(i, n, m)              # file -> grouped
        assert g == (i % n) * m + i // n
        assert oracle.interleaved_index(g, m, n) == i      # grouped -> file
        seen.add(g)
    assert seen == set(range(n * m))
