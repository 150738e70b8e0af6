"""GPU suite: the attractive force from the column-blocked copy of P (csrc/attractive_blocked.cu) against the
reference kernel's golden output, the CPU oracle, the live reference kernel and the row-major kernel.
Arithmetic to match: ComputePijxQijKernelV3 + reduce_sum_kernel, src/kernels/attr_forces.cu:129-184.
Bar: 1e-5 relative L2, as for the row-major kernel."""
import numpy as np
import pytest

from conftest import mixture, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_blocked_vs_reference_golden(engine, oracle_cpu, golden, tag):
    """One tile (1 500 points): every row is one group; with and without an order taken from points."""
    P, ids, Y = golden["P"], golden["ids"], golden["Y_" + tag]
    F, epg = engine.attractive_blocked(P, ids, Y)
    assert epg > 2.5
    assert rel_l2(F, golden["Fattr_" + tag]) < 1e-5
    assert rel_l2(F, oracle_cpu.attractive(P, ids, Y)) < 1e-5
    Xfake = np.random.default_rng(1).normal(size=(P.shape[0], 7)).astype(np.float32)   # any order must give the same force
    F2, _ = engine.attractive_blocked(P, ids, Y, X=Xfake)
    assert rel_l2(F2, golden["Fattr_" + tag]) < 1e-5


def _graph(engine, n, d, k, seed):
    X = mixture(n, d, seed)
    ids, d2 = engine.knn(X, k)
    p, _, _ = engine.perplexity(d2, k / 3.0, 1e-3)
    return X, ids, engine.symmetrize(p, ids)


def test_blocked_many_tiles_vs_rows_and_oracle(engine, oracle_cpu):
    """70 000 points = 3 tiles; cell order from the points; whole range and a rank's share of the rows."""
    n, k = 70000, 48
    X, ids, P = _graph(engine, n, 16, k, 3)
    rng = np.random.default_rng(0)
    for scale in (1e-4, 3.0):
        Y = rng.normal(0, scale, (2, n)).astype(np.float32)
        F_rows = engine.attractive(P, ids, Y)
        F, epg = engine.attractive_blocked(P, ids, Y, X=X)
        assert epg > 2.5
        assert rel_l2(F, F_rows) < 1e-5
        assert rel_l2(F, oracle_cpu.attractive(P, ids, Y)) < 1e-5
        lo, hi = 17500, 35000
        Fp, _ = engine.attractive_blocked(P, ids, Y, X=X, row_lo=lo, row_hi=hi)
        assert rel_l2(Fp[:, lo:hi], F_rows[:, lo:hi]) < 1e-5
        assert (Fp[:, :lo] == 0).all() and (Fp[:, hi:] == 0).all()
        Fn, _ = engine.attractive_blocked(P, ids, Y)          # natural order: the 4 components are interleaved
        assert rel_l2(Fn, F_rows) < 1e-5


def test_blocked_sparse_rows_markers_and_unfilled_slots(engine, oracle_cpu, monkeypatch):
    """A graph without locality (rows miss most tiles, so nearly every group needs a row marker), unfilled
    slots (id -1) and zero values.  The builder declines such a graph unless forced."""
    n, k = 120000, 9
    rng = np.random.default_rng(5)
    ids = rng.integers(0, n, (n, k), dtype=np.int32)
    ids[:, 0] = np.arange(n)
    ids[rng.random((n, k)) < 0.1] = -1
    P = (rng.random((n, k)) / (n * k)).astype(np.float32)
    P[rng.random((n, k)) < 0.05] = 0.0
    P[:, 0] = 0.0
    Y = rng.normal(0, 5.0, (2, n)).astype(np.float32)
    monkeypatch.delenv("B200TSNE_ATTRACTIVE", raising=False)
    with pytest.raises(engine.TsneError):
        engine.attractive_blocked(P, ids, Y)
    monkeypatch.setenv("B200TSNE_ATTRACTIVE", "blocked")
    F, epg = engine.attractive_blocked(P, ids, Y)
    assert epg < 2.5
    assert rel_l2(F, engine.attractive(P, ids, Y)) < 1e-5
    # the oracle follows the reference, which knows no unfilled slots: give it the same graph with those slots
    # pointing at point 0 with value 0
    assert rel_l2(F, oracle_cpu.attractive(np.where(ids < 0, 0.0, P).astype(np.float32), np.where(ids < 0, 0, ids).astype(np.int32), Y)) < 1e-5
    # long rows: more than 128 slots per row (the row-major path switches kernels there too)
    n2, k2 = 40000, 300
    ids2 = rng.integers(0, n2, (n2, k2), dtype=np.int32)
    P2 = (rng.random((n2, k2)) / (n2 * k2)).astype(np.float32)
    Y2 = rng.normal(0, 1.0, (2, n2)).astype(np.float32)
    F2, _ = engine.attractive_blocked(P2, ids2, Y2)
    assert rel_l2(F2, engine.attractive(P2, ids2, Y2)) < 1e-5


def test_blocked_vs_live_reference_kernel(engine):
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref/libtsnecuda_ref.so was not built (needs the reference tree)")
    n, k = 40000, 60
    X, ids, P = _graph(engine, n, 20, k, 8)
    Y = np.random.default_rng(2).normal(0, 2.0, (2, n)).astype(np.float32)
    F, _ = engine.attractive_blocked(P, ids, Y, X=X)
    assert rel_l2(F, ref.attractive(P, ids, Y)) < 1e-5


def test_session_uses_the_blocked_copy_and_matches_the_row_kernel(engine, oracle_cpu, monkeypatch):
    """The loop with the blocked copy and with the row-major kernel: same forces to rounding, so the same KL."""
    n, k = 40000, 60
    X = mixture(n, 20, 8)
    Y0 = (1e-4 * np.random.default_rng(1).standard_normal((2, n))).astype(np.float32)
    out = {}
    for mode in ("blocked", "rows"):
        if mode == "rows":
            monkeypatch.setenv("B200TSNE_ATTRACTIVE", "rows")
        else:
            monkeypatch.delenv("B200TSNE_ATTRACTIVE", raising=False)
        with engine.Session(n, k) as s:
            s.affinities_from_points(X, 20.0, 1e-3)
            assert s.attractive_mode()[0] == (1 if mode == "blocked" else 0)
            P, ids = s.get_affinities()
            s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
            s.set_embedding(Y0)
            s.run(1)
            Y1 = s.get_embedding()
            s.run(299)
            out[mode] = (P, ids, Y1, oracle_cpu.kl_divergence(P, ids, s.get_embedding()))
    assert np.array_equal(out["blocked"][0], out["rows"][0]) and np.array_equal(out["blocked"][1], out["rows"][1])
    assert rel_l2(out["blocked"][2], out["rows"][2]) < 1e-5
    assert abs(out["blocked"][3] - out["rows"][3]) / out["rows"][3] < 0.01


def test_state_in_cell_order_and_in_natural_order_agree(engine, oracle_cpu, monkeypatch):
    """On one GPU the session keeps embedding, momentum and gains in the blocked copy's point order and converts at
    its entry points (B200TSNE_ATTRACTIVE_RESIDENT=0 keeps the natural order and converts around the kernel instead).
    Both must show the caller the same values: after one iteration to rounding (the kernel's atomics add in any
    order), the optimizer state row by row, an embedding set after the affinities or before them, and a state
    saved in one form must resume in the other."""
    n, k = 30000, 40
    X = mixture(n, 16, 5)
    Y0 = (1e-4 * np.random.default_rng(2).standard_normal((2, n))).astype(np.float32)
    got = {}
    for mode in ("resident", "natural"):
        if mode == "natural":
            monkeypatch.setenv("B200TSNE_ATTRACTIVE_RESIDENT", "0")
        else:
            monkeypatch.delenv("B200TSNE_ATTRACTIVE_RESIDENT", raising=False)
        with engine.Session(n, k) as s:
            s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
            s.set_embedding(Y0)                      # before the affinities: converted when the copy is built
            s.affinities_from_points(X, 15.0, 1e-3)
            assert s.attractive_mode()[0] == 1
            assert np.array_equal(s.get_embedding(), Y0)
            s.run(1)
            Y1 = s.get_embedding()
            s.run(9)
            got[mode] = (Y1,) + tuple(s.get_state())
    assert rel_l2(got["resident"][0], got["natural"][0]) < 1e-5
    Ya, ma, ga, step_a = got["resident"][1:]
    Yb, mb, gb, step_b = got["natural"][1:]
    assert step_a == step_b == 10
    assert rel_l2(Ya, Yb) < 1e-4 and rel_l2(ma, mb) < 1e-3 and np.mean(ga != gb) < 1e-3
    # a state saved from the cell-ordered session resumes in a natural-order one (env still "0") and continues alike
    with engine.Session(n, k) as s:
        s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
        s.affinities_from_points(X, 15.0, 1e-3)
        s.set_state(Ya, ma, ga, step_a)
        Y2, m2, g2, st2 = s.get_state()
        assert np.array_equal(Y2, Ya) and np.array_equal(m2, ma) and np.array_equal(g2, ga) and st2 == step_a
