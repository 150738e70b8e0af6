"""GPU parity suite: every stage of the CUDA path, called through the C ABI with host buffers,
against the CPU oracle, the golden vectors of the reference's CUDA kernels and (when the reference
build travelled with the repository) the reference's kernels run live on the same inputs.

Bars: neighbour ids, symmetrised P and the update are bit-exact; forces within 1e-4 relative L2;
conditional p within 2*epsilon of the search tolerance (a row may stop one bisection step apart)."""
import numpy as np
import pytest

from conftest import mixture, rel_l2

pytestmark = pytest.mark.gpu
G = 390


# ------------------------------------------------------------------------------------- kNN
@pytest.mark.parametrize("n,d,k", [(1, 3, 1), (31, 1, 2), (33, 5, 33), (257, 50, 90), (1000, 97, 150), (5000, 50, 90),
                                   (700, 33, 1)])
def test_knn_bit_exact(engine, oracle_cpu, n, d, k):
    X = mixture(n, d, seed=n + d)
    ids, d2 = engine.knn(X, k)
    ids_o, d2_o = oracle_cpu.knn(X, k)
    assert np.array_equal(ids, ids_o)
    assert np.array_equal(d2, d2_o)


@pytest.mark.parametrize("pairs", ["bf16", "tf32"])
@pytest.mark.parametrize("n,d,k", [(3000, 50, 90), (70000, 30, 150), (420000, 50, 90)])
def test_knn_tensor_core_paths(engine, oracle_cpu, monkeypatch, n, d, k, pairs):
    """Online threshold (small), sample -> full (medium) and sample -> strided -> full (large) variants of the
    tensor-core search, with both operand forms of the filter (bf16 pairs are the default): exact on sampled
    queries, and the SIMT fallback is only needed for a few rows."""
    from tsne_cuda_b200 import datasets
    monkeypatch.setenv("B200TSNE_KNN_FILTER", pairs)
    X = datasets.gaussian_mixture(n, d, seed=n)
    ids, d2 = engine.knn(X, k)
    st = engine.knn_last_stats()
    assert st["tensor_core"] == 1 and st["rows_recomputed"] <= 0.01 * n and st["filter_error_ratio"] < 0.5
    lo = n // 3
    ids_o, d2_o = oracle_cpu.knn(X, k, q_lo=lo, q_hi=lo + 64)
    assert np.array_equal(ids[lo:lo + 64], ids_o) and np.array_equal(d2[lo:lo + 64], d2_o)
    assert np.array_equal(ids[:, 0], np.arange(n)) and (np.diff(d2, axis=1) >= 0).all()


def test_knn_tensor_core_matches_simt_everywhere(engine, monkeypatch):
    X = mixture(9000, 40, 12)
    X[100:300] = X[100]                      # 200 identical points: more ties than candidates, the proof cannot close
    a = engine.knn(X, 60)
    assert engine.knn_last_stats()["tensor_core"] == 1 and engine.knn_last_stats()["rows_recomputed"] >= 200
    monkeypatch.setenv("B200TSNE_KNN", "simt")
    b = engine.knn(X, 60)
    assert engine.knn_last_stats()["tensor_core"] == 0
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_knn_tensor_core_windows_and_cells(engine, monkeypatch):
    """The fixed-threshold scans split into database windows (as for a database image much larger than L2), on
    queries and database ranges that differ and are visited by cells: same lists as the SIMT search."""
    from tsne_cuda_b200 import datasets
    X = datasets.gaussian_mixture(150000, 24, seed=5)
    monkeypatch.setenv("B200TSNE_KNN_WINDOW_TILES", "37")
    a = engine.knn(X, 50, q_lo=1000, q_hi=40000, db_lo=5000, db_hi=149000)
    assert engine.knn_last_stats()["tensor_core"] == 1
    monkeypatch.delenv("B200TSNE_KNN_WINDOW_TILES")
    monkeypatch.setenv("B200TSNE_KNN", "simt")
    b = engine.knn(X, 50, q_lo=1000, q_hi=40000, db_lo=5000, db_hi=149000)
    assert engine.knn_last_stats()["tensor_core"] == 0
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


@pytest.mark.parametrize("pairs", ["bf16", "tf32"])
@pytest.mark.parametrize("n,d,k", [(20000, 100, 40), (30000, 784, 90), (17000, 65, 150)])
def test_knn_tensor_core_wide_points(engine, monkeypatch, n, d, k, pairs):
    """More inner dimensions than one shared-memory image holds: the chunked tensor-core kernel, same lists as the
    SIMT search on every row, with both operand forms of the filter."""
    from tsne_cuda_b200 import datasets
    monkeypatch.setenv("B200TSNE_KNN_FILTER", pairs)
    X = datasets.mnist_shaped(n, d, seed=n) if d == 784 else datasets.gaussian_mixture(n, d, seed=n)
    a = engine.knn(X, k)
    st = engine.knn_last_stats()
    assert st["tensor_core"] == 1 and st["rows_recomputed"] <= 0.02 * n and st["filter_error_ratio"] < 0.5
    monkeypatch.setenv("B200TSNE_KNN", "simt")
    b = engine.knn(X, k)
    assert engine.knn_last_stats()["tensor_core"] == 0
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_cached_device_memory_can_be_released(engine):
    """Freed device memory stays in the device's pool for the next call; releasing it to the driver must leave the
    library usable (and the result unchanged)."""
    X = mixture(3000, 20, 9)
    a = engine.knn(X, 30)
    engine.release_cached_memory()
    b = engine.knn(X, 30)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_knn_ties_and_duplicates(engine, oracle_cpu):
    X = np.zeros((300, 4), np.float32)
    X[100:200] = 1.0
    X[200:] = np.random.default_rng(0).integers(0, 2, (100, 4))
    ids, d2 = engine.knn(X, 40)
    ids_o, d2_o = oracle_cpu.knn(X, 40)
    assert np.array_equal(ids, ids_o) and np.array_equal(d2, d2_o)
    assert np.array_equal(ids[0], np.arange(40))


def test_knn_ranges_and_padding(engine, oracle_cpu):
    X = mixture(500, 20, 3)
    a = engine.knn(X, 16, q_lo=100, q_hi=163, db_lo=37, db_hi=401)
    b = oracle_cpu.knn(X, 16, q_lo=100, q_hi=163, db_lo=37, db_hi=401)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    ids, d2 = engine.knn(X, 12, db_lo=10, db_hi=15)     # database smaller than K
    ids_o, d2_o = oracle_cpu.knn(X, 12, db_lo=10, db_hi=15)
    assert np.array_equal(ids, ids_o) and (ids[:, 5:] == -1).all() and np.isinf(d2[:, 5:]).all()
    empty = engine.knn(X, 4, q_lo=7, q_hi=7)
    assert empty[0].shape == (0, 4)


def test_knn_database_shards_merge_to_full(engine, oracle_cpu):
    X = mixture(900, 30, 4)
    full = engine.knn(X, 20)
    parts = [engine.knn(X, 20, db_lo=lo, db_hi=hi) for lo, hi in ((0, 450), (450, 900))]
    ids, d2 = oracle_cpu.knn_merge(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    assert np.array_equal(ids, full[0]) and np.array_equal(d2, full[1])


# ------------------------------------------------------------------------------------- P
def test_perplexity_vs_oracle_and_golden(engine, oracle_cpu, golden):
    perp, eps = float(golden["perplexity"]), float(golden["eps"])
    p, betas, mx = engine.perplexity(golden["d2"], perp, eps)
    assert mx == golden["d2"].max()
    assert rel_l2(p, golden["p"]) < 2 * eps                      # reference's CUDA kernels
    assert np.abs(p - golden["p"]).max() < 2 * eps * golden["p"].max() + 1e-7
    p_o, b_o = oracle_cpu.perplexity(golden["dhat"], perp, eps, True)
    assert rel_l2(p, p_o) < 2 * eps and rel_l2(betas, b_o) < 2 * eps
    assert np.allclose(p.sum(1), 1.0, atol=1e-5) and (p[:, 0] == 0).all()


@pytest.mark.parametrize("k", [1, 2, 31, 33, 150, 1023])
def test_perplexity_row_lengths(engine, oracle_cpu, k):
    rng = np.random.default_rng(k)
    d2 = np.sort(rng.random((64, k)).astype(np.float32) * 50, axis=1)
    d2[:, 0] = 0
    p, _, _ = engine.perplexity(d2, min(30.0, max(1.5, k / 3)), 1e-4)
    dh, _ = oracle_cpu.max_normalize(d2)
    p_o = oracle_cpu.perplexity(dh, min(30.0, max(1.5, k / 3)), 1e-4)
    if k == 1:
        assert np.isnan(p).all() == np.isnan(p_o).all()          # 0/0 in both: a single self slot has no mass
    else:
        assert rel_l2(p, p_o) < 2e-4


def test_perplexity_max_override_for_sharded_rows(engine, golden):
    full, _, mx = engine.perplexity(golden["d2"], 15.0, 1e-4)
    part, _, _ = engine.perplexity(golden["d2"][:700], 15.0, 1e-4, max_override=mx)
    assert np.array_equal(part, full[:700])


def test_symmetrize_bit_exact(engine, oracle_cpu, golden):
    P = engine.symmetrize(golden["p"], golden["ids"])
    assert np.array_equal(P, golden["P"])                        # reference's CUDA kernel
    assert np.array_equal(P, oracle_cpu.symmetrize(golden["p"], golden["ids"]))


# ------------------------------------------------------------------------------------- forces
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_forces_vs_reference_golden(engine, oracle_cpu, golden, tag):
    Y = golden["Y_" + tag]
    Fa = engine.attractive(golden["P"], golden["ids"], Y)
    assert rel_l2(Fa, golden["Fattr_" + tag]) < 1e-5
    Fr, Z, w, yt = engine.repulsive(Y, True)
    Fr_o, Z_o, w_o, yt_o, _ = oracle_cpu.repulsive(Y, True)
    err_ref = rel_l2(golden["Frep_" + tag], Fr_o)     # the reference's own fp32 rounding noise vs fp64 convolution
    err_mine = rel_l2(Fr, Fr_o)
    # 1e-4 against the reference's CUDA path wherever the reference itself is that accurate; where its
    # own noise is larger (tag b) this path must be at least as close to the fp64 evaluation as it is
    assert rel_l2(Fr, golden["Frep_" + tag]) < max(1e-4, 2 * err_ref)
    assert err_mine < max(1e-4, 1.5 * err_ref)
    assert abs(Z - float(golden["Z_" + tag])) / abs(float(golden["Z_" + tag])) < 1e-4
    assert rel_l2(w, w_o) < 1e-4 and rel_l2(yt, yt_o) < 1e-4
    nodes = golden["sample_nodes"]
    assert rel_l2(yt.reshape(-1, 4)[nodes], golden["yt_%s_sample" % tag]) < 1e-4
    assert rel_l2(w.astype(np.float64).sum(1), golden["w_%s_rows" % tag]) < 1e-4


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_apply_forces_bit_exact_vs_reference_golden(engine, golden, tag):
    Y2, g2, o2 = engine.apply_forces(golden["Y_" + tag], golden["Fattr_" + tag], golden["Frep_" + tag],
                                     golden["gains_" + tag], golden["old_" + tag], 200.0, float(golden["Z_" + tag]),
                                     float(golden["mom_" + tag]), float(golden["exag_" + tag]))
    assert np.array_equal(g2, golden["gainsnext_" + tag])
    assert np.array_equal(o2, golden["oldnext_" + tag])
    assert np.array_equal(Y2, golden["Ynext_" + tag])


def test_attractive_row_ranges_and_linearity(engine, oracle_cpu, golden):
    P, ids, Y = golden["P"], golden["ids"], golden["Y_c"]
    F = engine.attractive(P, ids, Y)
    part = engine.attractive(P, ids, Y, 200, 777)
    assert np.array_equal(part[:, 200:777], F[:, 200:777]) and (part[:, :200] == 0).all() and (part[:, 777:] == 0).all()
    assert rel_l2(engine.attractive(2 * P, ids, Y), 2 * F.astype(np.float64)) < 1e-6
    assert rel_l2(F, oracle_cpu.attractive(P, ids, Y)) < 1e-5


def test_repulsive_edge_cases(engine, oracle_cpu):
    # all points identical: the reference divides by zero here; this path must stay finite
    Y = np.full((2, 100), 0.25, np.float32)
    F, Z = engine.repulsive(Y)
    assert np.isfinite(F).all() and np.isfinite(Z)
    assert abs(Z - 100 * 99) < 1e-2 * 100 * 99 and np.abs(F).max() < 1e-2
    # points exactly on the grid's corners and box edges
    Y = np.zeros((2, 131 * 2), np.float32)
    Y[0, :131] = np.linspace(-3, 3, 131)
    Y[1, 131:] = np.linspace(-3, 3, 131)
    F, Z = engine.repulsive(Y)
    F_o, Z_o = oracle_cpu.repulsive(Y)
    assert rel_l2(F, F_o) < 1e-4 and abs(Z - Z_o) / Z_o < 1e-4
    # a single point
    F, Z = engine.repulsive(np.array([[1.5], [-2.0]], np.float32))
    assert np.isfinite(F).all() and abs(Z) < 1e-3


@pytest.mark.parametrize("n,scale", [(1, 1.0), (31, 1e-4), (33, 3.0), (1000, 30.0), (4097, 1.0)])
def test_repulsive_odd_sizes_vs_oracle(engine, oracle_cpu, n, scale):
    Y = np.random.default_rng(n).normal(0, scale, (2, n)).astype(np.float32)
    F, Z = engine.repulsive(Y)
    F_o, Z_o = oracle_cpu.repulsive(Y)
    if n > 1:
        assert rel_l2(F, F_o) < 2e-4
        assert abs(Z - Z_o) <= 1e-4 * abs(Z_o) + 1e-3


# ------------------------------------------------------------------------------------- live reference
def test_stages_vs_live_reference_kernels(engine, oracle_cpu):
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref/libtsnecuda_ref.so was not built (needs the reference tree)")
    X = mixture(3000, 50, 21)
    ids, d2 = engine.knn(X, 60)
    dhat = ref.max_normalize(d2)
    p, _, _ = engine.perplexity(d2, 20.0, 1e-3)
    p_r = ref.perplexity(dhat, 20.0, 1e-3)
    assert rel_l2(p, p_r) < 2e-3
    assert np.array_equal(engine.symmetrize(p_r, ids), ref.symmetrize(p_r, ids))
    P = ref.symmetrize(p_r, ids)
    rng = np.random.default_rng(0)
    for scale in (1e-4, 0.05, 2.0, 15.0):
        Y = rng.normal(0, scale, (2, 3000)).astype(np.float32)
        assert rel_l2(engine.attractive(P, ids, Y), ref.attractive(P, ids, Y)) < 1e-5
        F, Z = engine.repulsive(Y)
        F_r, Z_r = ref.repulsive(Y)
        F_o, _ = oracle_cpu.repulsive(Y)
        assert rel_l2(F, F_r) < max(1e-4, 2 * rel_l2(F_r, F_o))
        assert abs(Z - Z_r) / abs(Z_r) < 1e-4


@pytest.mark.parametrize("shift,scale", [(0.0, 1.0), (300.0, 1.0), (0.0, 1e-18), (0.0, 1e12)])
def test_knn_tensor_core_exact_whatever_the_norms(engine, monkeypatch, shift, scale):
    """The filter's keys lose accuracy with |x_i||x_j|: far from the origin the proof closes for fewer rows (they go to
    the SIMT search), at tiny or huge scales the bf16 pairs lose their low parts or their range.  Whatever happens to
    the filter, the lists must equal the SIMT search's on every row."""
    rng = np.random.default_rng(5)
    X = ((rng.standard_normal((70000, 8)) + shift) * scale).astype(np.float32)
    a = engine.knn(X, 30)
    assert engine.knn_last_stats()["tensor_core"] == 1
    monkeypatch.setenv("B200TSNE_KNN", "simt")
    b = engine.knn(X, 30)
    assert engine.knn_last_stats()["tensor_core"] == 0
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
