"""CPU suite for the point-sharded (multi-GPU) path: row partitioning, and the exchange steps of the
sharded pipeline modelled with the CPU oracle over a world_size-2 gloo group."""
import os
import socket

import numpy as np
import pytest

from conftest import mixture, rel_l2
from tsne_cuda_b200.distributed import shard_rows


@pytest.mark.parametrize("n,world", [(10, 1), (10, 2), (11, 2), (7, 8), (1000000, 8), (5, 16), (1, 4)])
def test_shards_cover_all_rows_once(n, world):
    covered = []
    chunk = (n + world - 1) // world
    for r in range(world):
        lo, hi = shard_rows(n, world, r)
        assert 0 <= lo <= hi <= n and hi - lo <= chunk
        assert lo == min(n, r * chunk)          # what the in-place all-gather relies on
        covered += list(range(lo, hi))
    assert covered == list(range(n))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import cpu
    from tsne_cuda_b200 import distributed
    try:
        N, D, K = 301, 7, 10
        X = mixture(N, D, 11)
        lo, hi = shard_rows(N, world, rank)
        chunk = (N + world - 1) // world
        # unique-id plumbing: rank 0's bytes reach everybody
        uid = distributed.share_unique_id(lambda: bytes(range(128)), rank, world)
        assert uid == bytes(range(128))
        # database-sharded search: all queries against my rows, all-gather of the partial lists, merge
        ids_p, d2_p = cpu.knn(X, K, db_lo=lo, db_hi=hi)
        gi = [torch.zeros((N, K), dtype=torch.int32) for _ in range(world)]
        gd = [torch.zeros((N, K), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gi, torch.from_numpy(ids_p))
        dist.all_gather(gd, torch.from_numpy(d2_p))
        ids, d2 = cpu.knn_merge(np.stack([t.numpy() for t in gi]), np.stack([t.numpy() for t in gd]))
        ids_full, d2_full = cpu.knn(X, K)
        assert np.array_equal(ids, ids_full) and np.array_equal(d2, d2_full)
        # global max-normalisation = all-reduce(max) of the shard maxima
        m = torch.tensor([float(d2_full[lo:hi].max()) if hi > lo else 0.0])
        dist.all_reduce(m, op=dist.ReduceOp.MAX)
        assert float(m) == float(d2_full.max())
        dh, _ = cpu.max_normalize(d2_full)
        P = cpu.symmetrize(cpu.perplexity(dh, 5.0, 1e-4), ids_full)
        # one sharded iteration: partial spread -> all-reduce, redundant convolution, partial gather ->
        # all-reduce of sum Z_i, attractive rows, update rows, all-gather of Y
        rng = np.random.default_rng(3)
        Y = rng.normal(0, 2, (2, N)).astype(np.float32)
        mn, mx = cpu.minmax(Y)
        w = torch.from_numpy(cpu.spread(Y, mn, mx, lo, hi))
        dist.all_reduce(w)
        assert rel_l2(w.numpy(), cpu.spread(Y, mn, mx)) < 1e-5
        # the same sum by slice owners (the peer-memory form from four ranks on): every rank sums its slice of the
        # nodes over all ranks' partial grids in rank order and hands the slice to everybody; all ranks then hold
        # bit-identical grids, and the normalisation follows from the summed grid without an exchange
        part = cpu.spread(Y, mn, mx, lo, hi).reshape(-1, 4)
        parts_w = [torch.zeros(part.shape, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(parts_w, torch.from_numpy(part))
        n_nodes = part.shape[0]
        slice_len = (n_nodes + world - 1) // world
        s_lo, s_hi = min(n_nodes, rank * slice_len), min(n_nodes, (rank + 1) * slice_len)
        mine_w = np.zeros((slice_len, 4), np.float32)
        acc = parts_w[0].numpy()[s_lo:s_hi].copy()
        for r in range(1, world):
            acc += parts_w[r].numpy()[s_lo:s_hi]
        mine_w[:s_hi - s_lo] = acc
        slices = [torch.zeros((slice_len, 4), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(slices, torch.from_numpy(mine_w))
        w_slices = np.concatenate([t.numpy() for t in slices])[:n_nodes]
        by_rank_order = parts_w[0].numpy().copy()
        for r in range(1, world):
            by_rank_order += parts_w[r].numpy()
        assert np.array_equal(w_slices, by_rank_order)
        assert rel_l2(w_slices, w.numpy().reshape(-1, 4)) < 1e-6
        yt = cpu.convolve(w.numpy(), mn, mx)
        Fr, zs, _ = cpu.gather(Y, mn, mx, yt, lo, hi)
        z = torch.tensor([zs], dtype=torch.float64)
        dist.all_reduce(z)
        Fr_full, Z_full = cpu.repulsive(Y)
        assert abs((float(z) - N) - Z_full) / abs(Z_full) < 1e-5
        assert rel_l2(Fr[:, lo:hi], Fr_full[:, lo:hi]) < 1e-5
        Fa = cpu.attractive(P, ids_full, Y, lo, hi)
        g = np.ones((2, N), np.float32)
        u = np.zeros((2, N), np.float32)
        Ynew, _, _ = cpu.apply_forces(Y, Fa, Fr, g, u, 100.0, float(z) - N, 0.5, 12.0)
        mine = np.zeros((2, chunk), np.float32)
        mine[:, :hi - lo] = Ynew[:, lo:hi]
        parts = [torch.zeros((2, chunk)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        Yg = np.concatenate([p.numpy() for p in parts], 1)[:, :N]
        Yref, _, _ = cpu.apply_forces(Y, cpu.attractive(P, ids_full, Y), Fr_full, g, u, 100.0, Z_full, 0.5, 12.0)
        assert rel_l2(Yg, Yref) < 1e-5
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peer
        q.put((rank, "FAILED: %r" % (e,)))
    finally:
        dist.destroy_process_group()


def test_sharded_pipeline_world_size_2_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
