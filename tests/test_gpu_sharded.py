"""GPU suite for the point-sharded path (needs 2 GPUs; skipped otherwise): two ranks, NCCL exchanges issued
by the library, results against a single-GPU session on the same inputs."""
import os
import socket

import numpy as np
import pytest

from conftest import mixture, rel_l2

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, X, Y0, K, knn_shard, exchange, out):
    import torch
    import torch.distributed as dist
    # "p2p-slices": peer memory with the slice-owner form of the grid sum, which is the default from four ranks on
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      B200TSNE_KNN_SHARD=knn_shard, B200TSNE_EXCHANGE="nccl" if exchange == "nccl" else "p2p",
                      B200TSNE_GRID_SUM="slices" if exchange == "p2p-slices" else "all")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    from tsne_cuda_b200 import distributed
    try:
        s = distributed.open_session(X.shape[0], K, rank, rank, world)
        mode = s.exchange_mode()
        s.affinities_from_points(X, 20.0, 1e-4)
        P, ids = s.get_affinities()
        s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
        s.set_embedding(Y0)
        s.run(1)
        Y1 = s.get_embedding()
        s.run(199)
        Y200 = s.get_embedding()
        st = s.stats()
        s.close()
        out.put((rank, "ok", P, ids, Y1, Y200, mode))
    except Exception as e:  # report instead of leaving the peer in a collective
        out.put((rank, "FAILED: %r" % (e,), None, None, None, None, None))
    finally:
        distributed.release_communicators()
        dist.destroy_process_group()


@pytest.mark.parametrize("knn_shard,exchange", [("queries", "p2p"), ("queries", "nccl"), ("database", "p2p"), ("queries", "p2p-slices")])
def test_two_ranks_match_one(engine, oracle_cpu, knn_shard, exchange):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from tsne_cuda_b200.distributed import shard_rows
    N, D, K = 3001, 24, 40          # N not divisible by the number of ranks
    X = mixture(N, D, 3)
    Y0 = (1e-4 * np.random.default_rng(0).standard_normal((2, N))).astype(np.float32)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, X, Y0, K, knn_shard, exchange, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
    assert [r[1] for r in res] == ["ok", "ok"], [r[1] for r in res]
    assert [r[6] for r in res] == [1 if exchange == "nccl" else 2] * 2   # the exchange under test is the one that ran
    with engine.Session(N, K) as s:
        s.affinities_from_points(X, 20.0, 1e-4)
        P1, ids1 = s.get_affinities()
        s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
        s.set_embedding(Y0)
        s.run(1)
        Y1 = s.get_embedding()
        s.run(199)
        Y200 = s.get_embedding()
    for r in range(2):
        lo, hi = shard_rows(N, 2, r)
        assert np.array_equal(res[r][3], ids1[lo:hi])          # neighbour ids: exact under either sharding of the search
        assert np.array_equal(res[r][2], P1[lo:hi])            # P: same global maximum, same rows
        assert rel_l2(res[r][4], Y1) < 1e-5                    # one iteration: forces agree (grid summed in another order)
    assert np.array_equal(res[0][4], res[1][4]) and np.array_equal(res[0][5], res[1][5])   # ranks hold the same embedding
    kl1 = oracle_cpu.kl_divergence(P1, ids1, Y200)
    kl2 = oracle_cpu.kl_divergence(P1, ids1, res[0][5])
    assert abs(kl1 - kl2) / kl1 < 0.02


def _rank_late(rank, world, port, X, Y0, K, out):
    import time
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", B200TSNE_EXCHANGE="p2p")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    from tsne_cuda_b200 import _lib, distributed
    try:
        s = distributed.open_session(X.shape[0], K, rank, rank, world)
        mode = s.exchange_mode()
        s.affinities_from_points(X, 20.0, 1e-4)
        s.set_schedule(200.0, 12.0, 250, 0.5, 0.8)
        s.set_embedding(Y0)
        s.set_peer_timeout_ms(300)
        s.run(4)                                  # both ranks in step
        dist.barrier()
        if rank == 1:
            time.sleep(1.5)                       # a host-made late arrival, five times the limit
        t0 = time.time()
        try:
            s.run(60)
            status = "ok"
        except _lib.TsneError as e:
            status = str(e)
        dt = time.time() - t0
        s.close()
        out.put((rank, status, dt, mode))
    except Exception as e:
        out.put((rank, "FAILED: %r" % (e,), 0.0, None))
    finally:
        distributed.release_communicators()
        dist.destroy_process_group()


def test_late_rank_ends_the_run_quickly_on_both_ranks(engine):
    """A rank that arrives later than the meeting's limit: the waiting rank gives up once (not once per meeting),
    tells the late rank through the abort word, and both return the communicator status within seconds; both
    then close cleanly.  Nothing faults or hangs: the late arrival is made on the host."""
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    N, D, K = 3001, 24, 40
    X = mixture(N, D, 3)
    Y0 = (1e-4 * np.random.default_rng(0).standard_normal((2, N))).astype(np.float32)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_late, args=(r, 2, port, X, Y0, K, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
    assert [r[3] for r in res] == [2, 2]
    for rank, status, dt, _ in res:
        assert "status -5" in status and "did not arrive" in status, (rank, status)
        assert dt < 5.0, (rank, dt)          # 60 iterations x 2 meetings x 0.3 s would be 36 s
