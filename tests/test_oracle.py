"""The numpy oracle against fixtures produced by the reference's own sb_ref.py (see tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from cases import CASES, digest, inv_temp_of, make_inputs
from oracle import sb_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: z[k] for k in z.files}


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_fixture(name):
    spec = CASES[name]
    gold = load(name)
    q, k, v, do, drem = make_inputs(spec)
    assert digest([q, k, v, do, drem]) == str(gold["input_digest"]), "seeded inputs differ from the fixture's"
    ends = orc.ends_from_lengths(spec["lengths"])
    res = orc.sb_varlen_fwd_bwd(q, k, v, do, drem, ends, inv_temp_of(spec), spec["attend_current"], np.float64)
    # the reference computes in float32 (its own float32-vs-float64 floor is ~1e-6)
    for key, got in zip(("o", "rem", "dq", "dk", "dv"), res):
        err = np.abs(got - gold[key]).max()
        assert err < 2e-5, (name, key, err)


def test_oracle_float32_faithful_matches_fixture():
    """Same arithmetic as the reference: float32 and the triangular-matmul suffix sum."""
    spec = CASES["c1"]
    gold = load("c1")
    q, k, v, _, _ = make_inputs(spec)
    ends = orc.ends_from_lengths(spec["lengths"])
    o, rem = orc.sb_varlen_fwd(q, k, v, ends, inv_temp_of(spec), False, np.float32, faithful=True)
    assert np.abs(o - gold["o"]).max() < 5e-6
    assert np.abs(rem - gold["rem"]).max() < 5e-6


def test_known_answers():
    """q = 0 gives beta = 1/2 everywhere: A_ij = 2^-(i-j), rem_i = 2^-i; row 0 attends nothing."""
    H, L, D = 1, 12, 8
    rng = np.random.RandomState(0)
    q = np.zeros((H, L, D))
    k = rng.randn(H, L, D)
    v = rng.randn(H, L, D)
    o, rem, att, beta = orc.sb_dense_fwd(q, k, v, 0.3, return_att=True)
    i, j = np.meshgrid(np.arange(L), np.arange(L), indexing="ij")
    want = np.where(j < i, 0.5 ** (i - j).clip(0), 0.0)
    assert np.allclose(att[0], want, atol=1e-14)
    assert np.allclose(rem[0], 0.5 ** np.arange(L), atol=1e-14)
    assert np.allclose(o[0, 0], 0) and rem[0, 0] == 1
    assert np.allclose(att.sum(-1) + rem, 1, atol=1e-14)


def test_row_slabs_equal_full():
    spec = CASES["tiny_edges"]
    q, k, v, do, drem = make_inputs(spec)
    L = 65
    a = sum(spec["lengths"]) - L
    it = inv_temp_of(spec)
    full = orc.sb_dense_bwd(q[:, a:], k[:, a:], v[:, a:], do[:, a:], drem[:, a:], it)
    o1, r1 = orc.sb_rows_fwd(q, k, v, a, 20, 50, it)
    assert np.allclose(o1, full[0][:, 20:50], atol=1e-12) and np.allclose(r1, full[1][:, 20:50], atol=1e-12)
    dq1 = orc.sb_rows_dq(q, k, v, do, drem, a, 20, 50, it)
    assert np.allclose(dq1, full[2][:, 20:50], atol=1e-12)


def test_backward_is_gradient_by_finite_differences():
    rng = np.random.RandomState(1)
    H, L, D = 1, 9, 4
    q, k, v, do = (rng.randn(H, L, D) for _ in range(4))
    drem = rng.randn(H, L)
    it = 0.5

    def loss(q_, k_, v_):
        o, rem = orc.sb_dense_fwd(q_, k_, v_, it)
        return (o * do).sum() + (rem * drem).sum()

    _, _, dq, dk, dv = orc.sb_dense_bwd(q, k, v, do, drem, it)
    eps = 1e-6
    for arr, grad, idx in ((q, dq, 0), (k, dk, 1), (v, dv, 2)):
        for pos in [(0, 5, 1), (0, 2, 3), (0, 8, 0)]:
            args = [q.copy(), k.copy(), v.copy()]
            args[idx][pos] += eps
            hi = loss(*args)
            args[idx][pos] -= 2 * eps
            lo = loss(*args)
            assert abs((hi - lo) / (2 * eps) - grad[pos]) < 1e-6
