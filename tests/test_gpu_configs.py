"""GPU suite: the benchmark's other configurations (BASELINE.json configs 0-2) end to end at full size, with
synthetic inputs of the stated shapes.  Checks: neighbours exact on sampled queries, finite embedding,
classes separated, 10-NN preservation well above chance."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,classes", [("c0", 4), ("c1", 10), ("c2", 10)])
def test_configuration_end_to_end(engine, oracle_cpu, name, classes):
    from tsne_cuda_b200 import TSNE, datasets
    X, hp = datasets.make(name)
    N, D = X.shape
    K = hp["num_neighbors"]
    t0 = time.time()
    with engine.Session(N, K) as s:
        s.affinities_from_points(X, hp["perplexity"], 1e-3)
        P, ids = s.get_affinities()
    t_aff = time.time() - t0
    lo = N // 2
    ids_o, _ = oracle_cpu.knn(X, K, q_lo=lo, q_hi=lo + 32)
    assert np.array_equal(ids[lo:lo + 32], ids_o)
    assert 0.3 < P.sum() <= 1.0 + 1e-4
    Y0 = np.asfortranarray(datasets.initial_embedding(N).T)
    t0 = time.time()
    Y = TSNE(perplexity=hp["perplexity"], num_neighbors=K, learning_rate=hp["learning_rate"],
             early_exaggeration=hp["early_exaggeration"], n_iter=1000).fit_transform(X, Y0)
    t_fit = time.time() - t0
    print("%s: N=%d D=%d K=%d affinities %.2f s, fit_transform(1000 iterations) %.2f s" % (name, N, D, K, t_aff, t_fit))
    assert np.isfinite(Y).all()
    lab = np.arange(N) % classes
    cent = np.stack([Y[lab == c].mean(0) for c in range(classes)])
    nearest = np.linalg.norm(Y[:, None, :] - cent[None], axis=2).argmin(1)
    assert (nearest == lab).mean() > 0.95
    sub = np.random.default_rng(0).choice(N, 2000, replace=False)
    d = ((Y[sub, None, :] - Y[None, :, :]) ** 2).sum(-1) if N <= 8000 else None
    if d is not None:
        nn = np.argsort(d, axis=1)[:, 1:11]
        hits = np.mean([len(set(nn[r]) & set(ids[sub[r], 1:11])) / 10.0 for r in range(len(sub))])
        assert hits > 0.1
