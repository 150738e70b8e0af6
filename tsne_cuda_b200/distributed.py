"""One-process-per-GPU driver for a point-sharded run (torch.distributed is used for rendezvous
only; the data-path collectives are NCCL calls issued by libtsnecuda.so on its own stream).

Sharding: rank r owns the contiguous rows [r*ceil(N/W), min(N, (r+1)*ceil(N/W))) of the points,
of the fixed-width P, of gains and momentum, and produces those rows of the new embedding.  The
embedding and the 390x390x4 grid are replicated.  Per iteration: all-reduce of the grid after the
spread, all-reduce of sum Z_i after the gather, all-gather of the updated rows.  Set-up: exact kNN of the
owned rows against all points (queries sharded, no exchange; B200TSNE_KNN_SHARD=database shards
the database instead: every rank searches all queries against its own rows, then an all-to-all
of the partial lists and a merge), max-distance all-reduce, all-gather of ids and conditional p
for the symmetrisation.
"""
import os


def shard_rows(n, world, rank):
    """Rows owned by `rank`: equal chunks of ceil(n/world), the last ones may be short or empty."""
    chunk = (n + world - 1) // world
    lo = min(n, rank * chunk)
    return lo, min(n, lo + chunk)


def env_rank():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def share_unique_id(make_id, rank, world):
    """Rank 0 calls make_id() (-> 128 bytes); everyone gets the same bytes through torch.distributed."""
    import torch
    import torch.distributed as dist
    if world == 1:
        return make_id()
    t = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        t = torch.frombuffer(bytearray(make_id()), dtype=torch.uint8).clone()
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.broadcast(t, 0)
    return bytes(t.cpu().numpy().tobytes())


_unique_ids = {}   # (rank, world) -> the id this process already built a communicator from


def open_session(n, k, rank, local_rank, world):
    """Session owning this rank's rows, with the NCCL communicator attached when world > 1.  The
    first call of a process creates the communicator (seconds, collective over all ranks); later
    calls with the same rank and world size reuse it, as the library caches it by unique id."""
    from . import _lib
    lo, hi = shard_rows(n, world, rank)
    s = _lib.Session(n, k, lo, hi, device=local_rank)
    if world > 1:
        key = (rank, world)
        if key not in _unique_ids:
            _unique_ids[key] = share_unique_id(_lib.comm_unique_id, rank, world)
        s.attach_comm(_unique_ids[key], rank, world)
    return s


def release_communicators():
    """Destroy the cached communicators (call once all sessions are closed, before the process
    group is torn down)."""
    from . import _lib
    _unique_ids.clear()
    _lib.comm_release_all()
