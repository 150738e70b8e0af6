"""GPU suite: the opt-in truly symmetric P = (p + p^T) / 2N (a "next" row of the scope table; the reference's
fixed-width symmetrisation, src/util/math_utils.cu:269-291, drops the mirror image of one-directional edges).
Checked against a float64 sparse-matrix evaluation of the same definition: the stored entries (fixed-width part
plus the per-row extra lists) sum to 1, and the attractive force agrees to 1e-5 through the blocked kernel, the
row-major kernels, one tile and several."""
import numpy as np
import pytest

from conftest import mixture, rel_l2

pytestmark = pytest.mark.gpu


def symmetric_force_f64(p, ids, Y):
    """F_i = sum_j P_ij (y_i - y_j) / (1 + |y_i - y_j|^2) with P = (A + A^T) / 2N, A_ij = p_j|i on the neighbour list."""
    import scipy.sparse as sp
    n, k = p.shape
    rows = np.repeat(np.arange(n), k)
    A = sp.csr_matrix((p.astype(np.float64).ravel(), (rows, ids.ravel().astype(np.int64))), shape=(n, n))
    P = ((A + A.T) / (2.0 * n)).tocoo()
    y = Y.astype(np.float64)
    dx, dy = y[0, P.row] - y[0, P.col], y[1, P.row] - y[1, P.col]
    w = P.data / (1.0 + dx * dx + dy * dy)
    F = np.zeros((2, n))
    np.add.at(F[0], P.row, w * dx)
    np.add.at(F[1], P.row, w * dy)
    return F, P


@pytest.mark.parametrize("n,k,blocked_expected", [(3000, 40, 1), (70000, 30, 1)])
def test_symmetric_force_vs_sparse_float64(engine, monkeypatch, n, k, blocked_expected):
    monkeypatch.delenv("B200TSNE_ATTRACTIVE", raising=False)
    X = mixture(n, 16, 9)
    ids, d2 = engine.knn(X, k)
    p, _, _ = engine.perplexity(d2, k / 3.0, 1e-3)
    Y = np.random.default_rng(1).normal(0, 2.0, (2, n)).astype(np.float32)
    F64, P64 = symmetric_force_f64(p, ids, Y)
    F, P_fixed, n_extra, s_extra, blocked = engine.attractive_symmetric(p, ids, Y, X=X)
    assert blocked == blocked_expected
    assert np.array_equal(P_fixed, engine.symmetrize(p, ids))          # the fixed-width part is the reference's P
    keys = np.arange(n, dtype=np.int64)[:, None] * n + ids            # directed edges i -> j
    back = ids.astype(np.int64) * n + np.arange(n, dtype=np.int64)[:, None]
    one_way = ~np.isin(back.ravel(), keys.ravel()) & (ids.ravel() != np.repeat(np.arange(n), k))
    assert n_extra == int(one_way.sum()) and 0 < n_extra < n * k
    assert abs(float(P_fixed.astype(np.float64).sum()) + s_extra - 1.0) < 1e-4
    assert rel_l2(F, F64) < 1e-5
    # the reference's form is a different matrix: the extra entries matter
    assert rel_l2(engine.attractive(P_fixed, ids, Y), F64) > 1e-3
    # the same through the row-major kernels
    monkeypatch.setenv("B200TSNE_ATTRACTIVE", "rows")
    F_rows, _, n_extra2, _, blocked2 = engine.attractive_symmetric(p, ids, Y, X=X)
    assert blocked2 == 0 and n_extra2 == n_extra
    assert rel_l2(F_rows, F64) < 1e-5


def test_symmetric_rows_longer_than_a_segment(engine, monkeypatch):
    """A hub: one point is everybody's neighbour but has few itself, so its row gets thousands of extra entries
    (more than the 1,024 slots the builder walks at a time)."""
    monkeypatch.delenv("B200TSNE_ATTRACTIVE", raising=False)
    n, k, hub = 6000, 12, 17
    rng = np.random.default_rng(2)
    ids = np.empty((n, k), np.int32)
    pool = np.arange(n)
    for i in range(n):
        cand = pool[(pool != i) & (pool != hub)]
        m = k - 1 if i == hub else k - 2
        ids[i, 0] = i
        ids[i, 1:1 + m] = rng.choice(cand, m, replace=False)
        if i != hub:
            ids[i, k - 1] = hub
    p = rng.random((n, k)).astype(np.float32)
    p[:, 0] = 0.0
    p /= p.sum(1, keepdims=True)
    Y = rng.normal(0, 3.0, (2, n)).astype(np.float32)
    F, _, n_extra, _, blocked = engine.attractive_symmetric(p, ids, Y)
    assert blocked == 1 and n_extra > 4000
    F64, _ = symmetric_force_f64(p, ids, Y)
    assert rel_l2(F, F64) < 1e-5


def test_session_with_symmetric_affinities(engine, oracle_cpu):
    """The loop with the symmetric P: the first iteration moves the points by the symmetric force, and the run stays
    finite and separates the clusters."""
    n, k = 8000, 45
    X = mixture(n, 20, 4)
    Y0 = (1e-4 * np.random.default_rng(1).standard_normal((2, n))).astype(np.float32)
    out = {}
    for sym in (False, True):
        with engine.Session(n, k) as s:
            s.set_symmetric(sym)
            s.affinities_from_points(X, 15.0, 1e-3)
            s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
            s.set_embedding(Y0)
            s.run(1)
            Y1 = s.get_embedding()
            s.run(399)
            out[sym] = (Y1, s.get_embedding())
    assert rel_l2(out[True][0] - Y0, out[False][0] - Y0) > 1e-2          # another force
    Y = out[True][1]
    assert np.isfinite(Y).all()
    lab = np.arange(n) % 4
    cent = np.stack([Y[:, lab == c].mean(1) for c in range(4)])
    near = np.linalg.norm(Y.T[:, None] - cent[None], axis=2).argmin(1)
    assert (near == lab).mean() > 0.99
