"""GPU suite: the tensor-core neighbour search at the benchmark configurations' own sizes, every row compared
bit for bit (ids and squared distances) with the SIMT search, which computes the canonical exact fp32 brute
force (ties by index) that tests/test_gpu_stages.py pins to the CPU oracle.
Reference call site: util::KNearestNeighbors, src/util/distance_utils.cu:79-121."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_tensor_core_search_equals_simt_on_every_row(engine, oracle_cpu, monkeypatch, name):
    from tsne_cuda_b200 import datasets
    X, hp = datasets.make(name)
    K = hp["num_neighbors"]
    monkeypatch.delenv("B200TSNE_KNN", raising=False)
    ids, d2 = engine.knn(X, K)
    st = engine.knn_last_stats()
    assert st["tensor_core"] == 1 and st["filter_error_ratio"] < 1.0, st
    monkeypatch.setenv("B200TSNE_KNN", "simt")
    ids_s, d2_s = engine.knn(X, K)
    assert engine.knn_last_stats()["tensor_core"] == 0
    assert np.array_equal(ids, ids_s)
    assert np.array_equal(d2, d2_s)
    # and the SIMT search itself against the CPU oracle on a sample of rows of this very input
    lo = X.shape[0] // 3
    ids_o, d2_o = oracle_cpu.knn(X, K, q_lo=lo, q_hi=lo + 16)
    assert np.array_equal(ids_s[lo:lo + 16], ids_o) and np.array_equal(d2_s[lo:lo + 16], d2_o)
