"""GPU test of b200tsne_knn_noalloc, the neighbour search for hosts that may not allocate device memory
inside the call (their own pool owns the device, or the allocator's implicit synchronisation is not
acceptable): the caller hands in device buffers, the library's scratch is a fixed array in its image.

Collected last on purpose (file name): a stop-at-first-failure run has then exercised everything else."""
import ctypes as C

import numpy as np
import pytest

from conftest import mixture

pytestmark = pytest.mark.gpu


def _search(engine, torch, X, K):
    """One call through the C ABI on caller-owned device buffers; returns host copies."""
    N, D = X.shape
    x_d = torch.from_numpy(X).cuda()
    ids_d = torch.empty((N, K), dtype=torch.int32, device="cuda")
    d2_d = torch.empty((N, K), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    rc = engine.lib.b200tsne_knn_noalloc(C.c_void_p(x_d.data_ptr()), N, D, K, C.c_void_p(ids_d.data_ptr()),
                                         C.c_void_p(d2_d.data_ptr()), None)
    assert rc == 0, engine.lib.b200tsne_last_error()
    torch.cuda.synchronize()   # the call only queues the work
    return ids_d.cpu().numpy(), d2_d.cpu().numpy()


def test_no_alloc_search_matches_allocating_search_twice(engine):
    torch = pytest.importorskip("torch")
    assert engine.lib.b200tsne_knn_noalloc_max_elements() == 4 << 20
    # two calls in a row with different shapes: the second must not see anything of the first in the scratch
    for n, d, k, seed in ((3000, 20, 15, 1), (1777, 33, 40, 2)):
        X = mixture(n, d, seed)
        ids, d2 = _search(engine, torch, X, k)
        ids_ref, d2_ref = engine.knn(X, k)          # the existing entry point (allocates its own scratch)
        assert np.array_equal(ids, ids_ref)          # integer output: bit-exact
        assert np.array_equal(d2, d2_ref)            # canonical fp32 distances: bit-exact as well


def test_no_alloc_search_rejects_oversized_input(engine):
    torch = pytest.importorskip("torch")
    limit = engine.lib.b200tsne_knn_noalloc_max_elements()
    buf = torch.zeros(16, device="cuda")
    n = limit // 8 + 1                               # n * 8 > limit: refused before anything is read
    rc = engine.lib.b200tsne_knn_noalloc(C.c_void_p(buf.data_ptr()), n, 8, 4, C.c_void_p(buf.data_ptr()),
                                         C.c_void_p(buf.data_ptr()), None)
    assert rc == -4 and b"exceeds the built-in scratch" in engine.lib.b200tsne_last_error()
    assert engine.lib.b200tsne_knn_noalloc(None, 10, 8, 4, None, None, None) == -1
