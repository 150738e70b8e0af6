"""Generates tests/golden/ref_small.npz from the reference's own CUDA kernels.

Run on a GPU box with oracle/_ref/libtsnecuda_ref.so present (built by `python oracle/build.py --ref`
from the reference tree):

    python tests/golden/make_golden.py <output.npz>

Inputs are seeded; the exact neighbour list comes from the CPU oracle's canonical search (the
reference's own search is FAISS, which is not installed).  Every other array is an output of the
reference's host wrappers called through oracle/ref_build/ref_harness.cu.  The two 390x390x4 grids
are stored as marginal sums plus a fixed sample of nodes to keep the fixture small.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import cpu, ref  # noqa: E402

SAMPLE_NODES = np.random.default_rng(99).integers(0, 390 * 390, 4096)


def grid_digest(g):
    g = np.asarray(g, np.float64)
    flat = g.reshape(-1, 4)
    return dict(rows=g.sum(1).astype(np.float64), cols=g.sum(0).astype(np.float64), sample=flat[SAMPLE_NODES].astype(np.float32))


def main(out):
    rng = np.random.default_rng(1234)
    N, D, K = 1500, 20, 45
    mu = rng.normal(0, 10, (4, D))
    X = (mu[np.arange(N) % 4] + rng.normal(0, 1, (N, D))).astype(np.float32)
    ids, d2 = cpu.knn(X, K)
    dhat = ref.max_normalize(d2)
    p = ref.perplexity(dhat, 15.0, 1e-4)
    P = ref.symmetrize(p, ids)
    data = dict(X=X, ids=ids, d2=d2, dhat=dhat, p=p, P=P, perplexity=np.float32(15.0), eps=np.float32(1e-4),
                sample_nodes=SAMPLE_NODES)
    # three embeddings: start of the run, end of early exaggeration, late
    Y = (1e-4 * rng.standard_normal((2, N))).astype(np.float32)
    gains = np.ones((2, N), np.float32)
    old = np.zeros((2, N), np.float32)
    checkpoints = {0: "a", 250: "b", 750: "c"}
    for step in range(751):
        if step in checkpoints:
            tag = checkpoints[step]
            Fa = ref.attractive(P, ids, Y)
            Fr, Z, w, yt, phi = ref.repulsive(Y, True)
            exag, mom = (12.0, 0.5) if step < 250 else (1.0, 0.8)
            Y2, g2, o2 = ref.apply_forces(Y, Fa, Fr, gains, old, 200.0, Z, mom, exag)
            data.update({"Y_" + tag: Y.copy(), "gains_" + tag: gains.copy(), "old_" + tag: old.copy(), "Fattr_" + tag: Fa,
                         "Frep_" + tag: Fr, "Z_" + tag: np.float32(Z), "phi_" + tag: phi, "Ynext_" + tag: Y2,
                         "gainsnext_" + tag: g2, "oldnext_" + tag: o2, "exag_" + tag: np.float32(exag),
                         "mom_" + tag: np.float32(mom)})
            for nm, g in (("w", w), ("yt", yt)):
                for k, v in grid_digest(g).items():
                    data["%s_%s_%s" % (nm, tag, k)] = v
        Fa = ref.attractive(P, ids, Y)
        Fr, Z = ref.repulsive(Y)
        exag, mom = (12.0, 0.5) if step < 250 else (1.0, 0.8)
        Y, gains, old = ref.apply_forces(Y, Fa, Fr, gains, old, 200.0, Z, mom, exag)
    # end-to-end through the reference's own entry point (neighbours injected), quality numbers
    ref.set_knn(ids, d2)
    Y0 = data["Y_a"]
    Yfit = ref.fit_transform(X, Y0, perplexity=15.0, num_neighbors=K, perplexity_search_epsilon=1e-4, iterations=1000)
    ref.clear_knn()
    data["Yfit"] = Yfit
    data["kl_fit"] = np.float64(cpu.kl_divergence(P, ids, Yfit))
    data["nnp_fit"] = np.float64(cpu.nn_preservation(ids, Yfit, 10))
    np.savez_compressed(out, **data)
    print("wrote", out, os.path.getsize(out), "bytes; KL", data["kl_fit"], "10-NN", data["nnp_fit"])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_small.npz"))
