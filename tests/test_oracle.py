"""CPU suite: the oracle against the golden vectors of the reference's CUDA kernels, against an
independent float64 restatement, and against properties the algorithm guarantees."""
import numpy as np
import pytest

from conftest import mixture, rel_l2
from oracle import np64

G = 390


def grid_digest(g, nodes):
    g = np.asarray(g, np.float64)
    return g.sum(1), g.sum(0), g.reshape(-1, 4)[nodes]


# ------------------------------------------------------------------ pins against the reference
def test_perplexity_matches_reference_golden(golden, oracle_cpu):
    p = oracle_cpu.perplexity(golden["dhat"], float(golden["perplexity"]), float(golden["eps"]))
    # libm exp/log here, fast device intrinsics there: a row may stop one bisection step apart,
    # which moves p by O(eps); rows must agree to 2*eps and the bulk far better
    assert rel_l2(p, golden["p"]) < 2e-4
    assert np.abs(p - golden["p"]).max() < 2e-4 * golden["p"].max() + 1e-7
    assert np.allclose(p.sum(1), 1.0, atol=1e-5)


def test_max_normalize_matches_reference_golden(golden, oracle_cpu):
    dhat, m = oracle_cpu.max_normalize(golden["d2"])
    assert np.array_equal(dhat, golden["dhat"])
    assert m == golden["d2"].max()


def test_symmetrize_matches_reference_golden_bitwise(golden, oracle_cpu):
    assert np.array_equal(oracle_cpu.symmetrize(golden["p"], golden["ids"]), golden["P"])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_forces_match_reference_golden(golden, oracle_cpu, tag):
    Y = golden["Y_" + tag]
    Fa = oracle_cpu.attractive(golden["P"], golden["ids"], Y)
    assert rel_l2(Fa, golden["Fattr_" + tag]) < 1e-6
    Fr, Z, w, yt, phi = oracle_cpu.repulsive(Y, True)
    # The oracle convolves in fp64, the reference in fp32 (cuFFT): at the end of early exaggeration
    # (tag b: tight clusters, x*phi1 - phi2 cancels heavily) the reference's own rounding noise is
    # 1.2e-4 of the force, so the pin is 3e-4 here and 1e-4 elsewhere.
    assert rel_l2(Fr, golden["Frep_" + tag]) < (3e-4 if tag == "b" else 1e-4)
    assert abs(Z - float(golden["Z_" + tag])) / abs(float(golden["Z_" + tag])) < 1e-4
    nodes = golden["sample_nodes"]
    for name, grid, tol in (("w", w, 1e-4), ("yt", yt, 1e-5)):
        rows, cols, sample = grid_digest(grid, nodes)
        assert rel_l2(rows, golden["%s_%s_rows" % (name, tag)]) < tol
        assert rel_l2(cols, golden["%s_%s_cols" % (name, tag)]) < tol
        assert rel_l2(sample, golden["%s_%s_sample" % (name, tag)]) < tol
    assert rel_l2(phi, golden["phi_" + tag]) < 1e-5


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_apply_forces_matches_reference_golden(golden, oracle_cpu, tag):
    Y2, g2, o2 = oracle_cpu.apply_forces(golden["Y_" + tag], golden["Fattr_" + tag], golden["Frep_" + tag],
                                         golden["gains_" + tag], golden["old_" + tag], 200.0, float(golden["Z_" + tag]),
                                         float(golden["mom_" + tag]), float(golden["exag_" + tag]))
    # gains follow a sign rule and are exact; positions differ by FMA contraction on the device only
    assert np.array_equal(g2, golden["gainsnext_" + tag])
    # (momentum*u - eta*gain*grad subtracts two terms of similar size: bound the error by their scale)
    scale = max(np.abs(golden["oldnext_" + tag]).max(), np.abs(golden["old_" + tag]).max())
    assert np.abs(o2 - golden["oldnext_" + tag]).max() <= 4e-6 * scale
    assert np.abs(Y2 - golden["Ynext_" + tag]).max() <= 4e-6 * max(scale, np.abs(Y2).max())


def test_full_run_quality_matches_reference_golden(golden, oracle_cpu):
    """The oracle's own 1000-iteration run from the same P and Y0 ends at the reference's KL / 10-NN."""
    Y, _, _, _ = oracle_cpu.iterate(golden["P"], golden["ids"], golden["Y_a"], 1000, 200.0)
    kl = oracle_cpu.kl_divergence(golden["P"], golden["ids"], Y)
    nnp = oracle_cpu.nn_preservation(golden["ids"], Y, 10)
    assert abs(kl - float(golden["kl_fit"])) / float(golden["kl_fit"]) < 0.01
    assert abs(nnp - float(golden["nnp_fit"])) < 0.005 + 0.01  # 0.5 points + run-to-run spread of float atomics


# ------------------------------------------------------------------ independent float64 restatement
def test_knn_exact_vs_float64(oracle_cpu):
    X = mixture(700, 17, 5)
    ids, d2 = oracle_cpu.knn(X, 25)
    ids64, d64 = np64.knn(X, 25)
    assert np.array_equal(ids, ids64)
    assert np.allclose(d2, d64, rtol=1e-5)
    assert (ids[:, 0] == np.arange(700)).all() and (d2[:, 0] == 0).all()


def test_knn_ties_broken_by_index(oracle_cpu):
    X = np.zeros((50, 3), np.float32)
    X[25:] = 1.0
    ids, d2 = oracle_cpu.knn(X, 10)
    assert np.array_equal(ids[0], np.arange(10))
    assert np.array_equal(ids[30], np.arange(25, 35))
    assert (d2[:, :10] == 0).all()


def test_knn_database_shards_merge_to_full(oracle_cpu):
    X = mixture(400, 9, 6)
    full = oracle_cpu.knn(X, 12)
    parts = [oracle_cpu.knn(X, 12, db_lo=lo, db_hi=hi) for lo, hi in ((0, 130), (130, 131), (131, 400))]
    ids, d2 = oracle_cpu.knn_merge(np.stack([p[0] for p in parts]), np.stack([p[1] for p in parts]))
    assert np.array_equal(ids, full[0]) and np.array_equal(d2, full[1])


def test_knn_small_database_pads_with_minus_one(oracle_cpu):
    X = mixture(5, 4, 1)
    ids, d2 = oracle_cpu.knn(X, 8)
    assert (ids[:, 5:] == -1).all() and np.isinf(d2[:, 5:]).all() and (ids[:, :5] >= 0).all()


def test_stages_vs_float64(oracle_cpu):
    X = mixture(500, 12, 2)
    ids, d2 = oracle_cpu.knn(X, 20)
    dh, _ = oracle_cpu.max_normalize(d2)
    p = oracle_cpu.perplexity(dh, 8.0, 1e-5)
    assert rel_l2(p, np64.perplexity(dh, 8.0, 1e-5)) < 1e-4
    P = oracle_cpu.symmetrize(p, ids)
    assert rel_l2(P, np64.symmetrize(p.astype(np.float64), ids)) < 1e-6
    assert 0.5 < P.sum() <= 1.0 + 1e-5
    rng = np.random.default_rng(0)
    for scale in (1e-4, 1.0, 25.0):
        Y = rng.normal(0, scale, (2, 500)).astype(np.float32)
        assert rel_l2(oracle_cpu.attractive(P, ids, Y), np64.attractive(P, ids, Y)) < 1e-6
        F, Z, w, yt, _ = oracle_cpu.repulsive(Y, True)
        F64, Z64, w64, yt64 = np64.repulsive(Y)
        assert rel_l2(w, w64) < 1e-4 and rel_l2(yt, yt64) < 1e-4
        assert rel_l2(F, F64) < 2e-4 and abs(Z - Z64) / Z64 < 1e-4


def test_interpolation_approximates_exact_sums(oracle_cpu):
    rng = np.random.default_rng(3)
    Y = rng.normal(0, 2.0, (2, 800)).astype(np.float32)
    F, Z = oracle_cpu.repulsive(Y)
    Fe, Ze = oracle_cpu.repulsive_exact(Y)
    assert rel_l2(F, Fe) < 1e-3 and abs(Z - Ze) / Ze < 1e-4


def test_spread_conserves_charge_and_shards_add_up(oracle_cpu):
    rng = np.random.default_rng(4)
    Y = rng.normal(0, 5.0, (2, 1000)).astype(np.float32)
    mn, mx = oracle_cpu.minmax(Y)
    w = oracle_cpu.spread(Y, mn, mx)
    tot = w.reshape(-1, 4).astype(np.float64).sum(0)
    expect = np.array([1000, Y[0].sum(), Y[1].sum(), (Y[0] ** 2 + Y[1] ** 2).sum()], np.float64)
    assert np.allclose(tot, expect, rtol=1e-4, atol=1e-2)
    parts = oracle_cpu.spread(Y, mn, mx, 0, 333).astype(np.float64) + oracle_cpu.spread(Y, mn, mx, 333, 1000)
    assert rel_l2(parts, w) < 1e-6


def test_z_equals_grid_inner_product(oracle_cpu):
    """sum_i Z_i = sum_nodes [(w1+w4) y1 - 2 w2 y2 - 2 w3 y3 + w1 y4]: interpolation is linear, so the
    per-point sum equals an inner product of the two grids (what a sharded run may use instead of a
    second all-reduce)."""
    rng = np.random.default_rng(5)
    Y = rng.normal(0, 3.0, (2, 600)).astype(np.float32)
    F, Z, w, yt, phi = oracle_cpu.repulsive(Y, True)
    w, yt = w.astype(np.float64), yt.astype(np.float64)
    zs = ((w[..., 0] + w[..., 3]) * yt[..., 0] - 2 * w[..., 1] * yt[..., 1] - 2 * w[..., 2] * yt[..., 2] + w[..., 0] * yt[..., 3]).sum()
    assert abs((zs - 600) - Z) / abs(Z) < 1e-4


def test_apply_forces_vs_float64(oracle_cpu):
    rng = np.random.default_rng(6)
    n = 300
    Y, a, r, u = [rng.normal(0, 1, (2, n)).astype(np.float32) for _ in range(4)]
    g = rng.uniform(0.01, 3, (2, n)).astype(np.float32)
    Y2, g2, u2 = oracle_cpu.apply_forces(Y, a, r, g, u, 150.0, 321.0, 0.8, 4.0)
    Y64, g64, u64 = np64.apply_forces(Y.astype(np.float64), a, r, g, u, 150.0, 321.0, 0.8, 4.0)
    assert np.allclose(g2, g64, rtol=1e-6) and np.allclose(u2, u64, rtol=1e-4, atol=1e-5) and np.allclose(Y2, Y64, rtol=1e-4, atol=1e-4)
    assert (g2 >= 0.01).all()


def test_perplexity_hits_target_and_handles_duplicates(oracle_cpu):
    X = mixture(300, 6, 8)
    X[10] = X[11]  # duplicate point: distance 0 in slot 1 is a legitimate neighbour, only slot 0 is the self slot
    ids, d2 = oracle_cpu.knn(X, 30)
    dh, _ = oracle_cpu.max_normalize(d2)
    p = oracle_cpu.perplexity(dh, 10.0, 1e-4)
    assert (p[:, 0] == 0).all() and p[10, 1] > 0
    H = -(np.where(p > 0, p * np.log(np.where(p > 0, p, 1)), 0)).sum(1)
    assert np.abs(H - np.log(10.0)).max() < 5e-4
