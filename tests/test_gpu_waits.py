"""GPU suite: the bounded device-side waits are made to run out (no fault, no hang) and the device stays usable.

The two waits are the meeting of the ranks over peer memory (csrc/peer.cu) and the shared-memory barrier wait
of the tensor-core kNN pipeline (csrc/knn_tc.cu).  The self-test entry point sets up a meeting whose second
rank is local memory nobody writes, and a barrier that expects an arrival that never comes, each with a limit
of a few milliseconds."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_waits_give_up_and_leave_the_device_usable(engine, oracle_cpu):
    for limit in (5, 40):
        r = engine.selftest_bounded_waits(limit)
        assert r["peer"][0] == -5 and r["barrier"][0] == -5, r
        # gave up after the limit, not much later (the second meeting on the failed exchange returns at once)
        assert limit * 0.9 <= r["peer"][1] < limit + 50, r
        assert limit * 0.9 <= r["barrier"][1] < limit + 50, r
    # the context is intact: a search right after it is exact
    X = np.random.default_rng(0).normal(size=(3000, 50)).astype(np.float32)
    ids, d2 = engine.knn(X, 90)
    assert engine.knn_last_stats()["tensor_core"] == 1
    ids_o, d2_o = oracle_cpu.knn(X, 90, q_lo=100, q_hi=132)
    assert np.array_equal(ids[100:132], ids_o) and np.array_equal(d2[100:132], d2_o)
    with pytest.raises(engine.TsneError):
        engine.selftest_bounded_waits(0)
