#!/usr/bin/env python
"""Benchmark of the FIt-SNE hot path: gradient iterations/s and fit_transform seconds.

  python bench.py --gpus 1 --steps K --warmup W            # this engine, 1 GPU
  torchrun ... bench.py --gpus N --steps K --warmup W      # one rank per GPU, points sharded
  python bench.py --impl reference ...                     # the reference's own CUDA build (oracle/_ref)

A "step" is one gradient iteration (spread, FFT convolution, gather, attractive force, update) on
the N = 1,000,000, D = 50 synthetic Gaussian mixture with exact 90-NN affinities (config c3).
`value` is iterations/s with P, ids and Y resident in HBM, timed with CUDA events on the stream the
kernels are launched on (inside libtsnecuda.so); `e2e` is a complete fit_transform through the
drop-in symbol pymodule_tsne from host X to host Y.  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

G2 = 390 * 390


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def load_tensor_peak():
    """Measured cuBLAS bf16 TFLOP/s (burst: the search is timed alone), else the recipe's fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


class ClockSampler(object):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()   # the exact process started above
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for k, nm in enumerate(names):
                if len(r) > 3 + k and r[3 + k].lower().startswith("active"):
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def workload(args):
    from tsne_cuda_b200 import datasets
    X, hp = datasets.make(args.config, n=args.n)
    Y0 = datasets.initial_embedding(X.shape[0])
    return X, hp, Y0


def iter_bytes(n, k):
    """Algorithmic bytes of one gradient iteration: 8NK + 104N + 48G^2 (P value + id per stored entry,
    Y / force / gains / momentum traffic per point, three passes over the four-term grid)."""
    return 8.0 * n * k + 104.0 * n + 48.0 * G2


def run_ours(args):
    from tsne_cuda_b200 import _lib, distributed
    rank, local_rank, world = distributed.env_rank()
    multi = world > 1
    if multi:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl")
    X, hp, Y0 = workload(args)
    N, D = X.shape
    K = hp["num_neighbors"]
    lo, hi = distributed.shard_rows(N, world, rank)
    t0 = time.time()
    s = distributed.open_session(N, K, rank, local_rank, world)
    open_s = time.time() - t0
    t0 = time.time()
    s.affinities_from_points(X, hp["perplexity"], 1e-3)
    setup_s = time.time() - t0                  # the process's first call: kernels load, the memory pool grows
    s.enable_stage_timers(True)                 # once more, warm, for the device time of the search (CUDA events)
    t0 = time.time()
    s.affinities_from_points(X, hp["perplexity"], 1e-3)
    setup_warm_s = time.time() - t0
    setup_stages = s.stage_times()
    s.enable_stage_timers(False)
    s.set_schedule(hp["learning_rate"], hp["early_exaggeration"], 250, 0.5, 0.8)
    s.set_embedding(Y0)
    s.run(args.warmup)
    attr_mode, entries_per_group = s.attractive_mode()
    sharded_check = sharded_parity(s, X, K, lo, hi, rank, world) if multi else None

    def barrier():
        if multi:
            dist.barrier()
            torch.cuda.synchronize()

    barrier()
    l0 = s.launch_count()
    with ClockSampler(local_rank) as clk:
        ms, done = s.run(args.steps)
    barrier()
    launches = s.launch_count() - l0
    if multi:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = args.steps / (ms * 1e-3)

    # per-kernel durations of the same loop, stages serialised on one stream, CUDA events per stage
    s.enable_stage_timers(True)
    n_prof = max(5, min(50, args.steps))
    s.run(n_prof)
    stages = s.stage_times()
    s.enable_stage_timers(False)
    stage_us = {k: v[0] / n_prof * 1e3 for k, v in stages.items() if v[1] > 0 and k not in ("knn", "affinities")}
    # the attractive stage of one iteration: the row-major kernel alone, or the blocked kernel - alone on one GPU, where
    # the update kernel converts between point order and cell order, else with its two small companions (gather of the
    # embedding into the cell order, scatter of the forces back), timed together
    attr_s = stages["attractive"][0] / n_prof * 1e-3
    rows = hi - lo
    attr_bytes = 8.0 * rows * K + 16.0 * rows
    peak, peak_kind = load_peaks()
    # dram__bytes_read + dram__bytes_write of one launch from the committed ncu captures, scaled by the units
    # processed: row-major kernel 296.3 MB for 294.4 MB algorithmic (profiles/attractive_kernel_n400k.md);
    # blocked kernel: its stream of 6-byte entries padded to whole lanes (profiles/attractive_blocked_kernel_n400k.md)
    traffic_ratio = TRAFFIC_RATIO_BLOCKED if attr_mode else 296.3 / 294.4
    roof = {"bound": "hbm", "kernel": "attractive_blocked_kernel" if attr_mode else "attractive_kernel",
            "achieved": attr_bytes / attr_s / 1e9 if attr_s > 0 else None,
            "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
            "traffic": attr_bytes * traffic_ratio, "entries_per_row_and_tile": entries_per_group,
            "algorithmic_bytes_per_launch": attr_bytes, "avg_launch_us": attr_s * 1e6,
            "launches_timed_together": int(round(stages["attractive"][1] / n_prof))}
    roof["frac"] = roof["achieved"] / peak if roof["achieved"] else None
    it_bytes = iter_bytes(N, K) / world
    roof["iteration"] = {"achieved": it_bytes / (ms * 1e-3 / args.steps) / 1e9, "frac": it_bytes / (ms * 1e-3 / args.steps) / 1e9 / peak,
                         "algorithmic_bytes": it_bytes}
    # the neighbour search of the set-up: the tensor-core filter with its selection, exact re-rank and proof, timed on
    # the device in this process.  Algorithmic flops = one exact pass, 2 * queries * N * D; the filter executes three
    # bf16 products per key over an inner dimension padded to 64 (3.84x the algorithmic flops per tile pair it visits)
    # and skips the Voronoi cells no query of a block can reach (about 3/4 of the tile pairs on this mixture).
    knn_s = setup_stages.get("knn", (0.0, 0))[0] * 1e-3
    tpeak, tpeak_kind = load_tensor_peak()
    knn_flops = 2.0 * rows * N * D
    roof_knn = {"bound": "tensor", "kernel": "knn_tc_filter_kernel (with selection, re-rank and proof)",
                "achieved": knn_flops / knn_s / 1e12 if knn_s > 0 else None, "peak": tpeak, "peak_kind": tpeak_kind,
                "unit": "TFLOP/s", "algorithmic_flops": knn_flops, "seconds": knn_s, "setup_warm_s": setup_warm_s,
                "tensor_pipe_active_in_profile": 0.347, "profile": "profiles/knn_tc_filter_kernel_n400k.md"}
    roof_knn["frac"] = roof_knn["achieved"] / tpeak if roof_knn["achieved"] else None
    s.close()

    out = {"metric": "gradient_iterations_per_s", "value": value, "unit": "iterations/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": "%s: N=%d D=%d K=%d perplexity=%g, 4-component Gaussian mixture, exact kNN" %
                                  (args.config, N, D, K, hp["perplexity"]),
                      "l2_policy": "inputs larger than L2 (P+ids = %.0f MB per iteration)" % (8.0 * N * K / 1e6),
                      "parallelism": "points sharded over %d GPU(s)" % world},
           "gpu_launches": int(launches), "setup_s": setup_s, "open_session_s": open_s, "stage_us_per_iteration": stage_us,
           "roofline": roof, "roofline_knn": roof_knn, "clocks": clk.summary()}
    if sharded_check is not None:
        out["sharded_check"] = sharded_check

    if rank == 0 and not multi and not args.no_e2e:
        out["e2e"] = e2e_ours(X, hp, Y0, args)
    elif multi and not args.no_e2e:
        out["e2e"] = e2e_sharded(X, hp, Y0, args, rank, local_rank, world)
    if rank == 0 and not multi and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(X, hp, Y0, args)
    if multi:
        distributed.release_communicators()
        dist.destroy_process_group()
    return out if rank == 0 else None


TRAFFIC_RATIO_BLOCKED = 245.5 / 294.4   # dram__bytes_read + dram__bytes_write over algorithmic bytes, profiles/attractive_blocked_kernel_n400k.md


def sharded_parity(s, X, K, lo, hi, rank, world):
    """Evidence that N ranks compute what one does, printed with the bench line: 64 of this rank's neighbour
    rows against the CPU oracle's exact search, and the largest difference between this rank's embedding and
    rank 0's after the warm-up iterations (every rank must hold the same embedding)."""
    import torch
    import torch.distributed as dist
    from oracle import cpu
    _, ids = s.get_affinities()
    q0 = lo + (hi - lo) // 2
    q1 = min(hi, q0 + 64)
    ids_o, _ = cpu.knn(X, K, q_lo=q0, q_hi=q1)
    knn_ok = bool(np.array_equal(ids[q0 - lo:q1 - lo], ids_o))
    Y = torch.from_numpy(s.get_embedding()).cuda()
    Y0 = Y.clone()
    dist.broadcast(Y0, 0)
    diff = (Y - Y0).abs().max().reshape(1)
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    ok = torch.tensor([1 if knn_ok else 0], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return {"knn_rows_checked_per_rank": int(q1 - q0), "knn_rows_equal_cpu_oracle_on_all_ranks": bool(ok.item()),
            "max_abs_embedding_difference_to_rank0": float(diff.item()), "exchange_mode": s.exchange_mode()}


def e2e_ours(X, hp, Y0, args):
    """fit_transform through the drop-in symbol: host X -> host Y, everything inside the timed region."""
    from tsne_cuda_b200 import TSNE
    n_iter = args.e2e_iters
    t = TSNE(perplexity=hp["perplexity"], num_neighbors=hp["num_neighbors"], learning_rate=hp["learning_rate"],
             early_exaggeration=hp["early_exaggeration"], n_iter=n_iter, perplexity_epsilon=1e-3)
    y0 = np.asfortranarray(Y0.T)
    # one untimed call first (20 iterations): the first call of a process pays the lazy loading of every
    # kernel it uses and the first large device allocations
    warm = TSNE(perplexity=hp["perplexity"], num_neighbors=hp["num_neighbors"], learning_rate=hp["learning_rate"],
                early_exaggeration=hp["early_exaggeration"], n_iter=20, perplexity_epsilon=1e-3)
    warm.fit_transform(X, y0)
    times = []
    for _ in range(3):   # median of three calls: allocation and page-fault noise of a call is +-10 %
        t0 = time.time()
        Y = t.fit_transform(X, y0)
        times.append(time.time() - t0)
        assert np.isfinite(Y).all()
    T = sorted(times)[1]
    # where the time goes: the same fit through the session entry points, phases timed on the host
    from tsne_cuda_b200 import _lib
    ph = [time.time()]
    with _lib.Session(X.shape[0], hp["num_neighbors"]) as s:
        ph.append(time.time())
        s.affinities_from_points(X, hp["perplexity"], 1e-3)
        ph.append(time.time())
        s.set_schedule(hp["learning_rate"], hp["early_exaggeration"], 250, 0.5, 0.8)
        s.set_embedding(Y0)
        ph.append(time.time())
        loop_ms, _ = s.run(n_iter)
        ph.append(time.time())
        s.get_embedding()
        ph.append(time.time())
    ph.append(time.time())
    phases = {"open_session_s": ph[1] - ph[0], "h2d_points_knn_affinities_s": ph[2] - ph[1], "h2d_embedding_s": ph[3] - ph[2],
              "iterations_s": ph[4] - ph[3], "iterations_device_s": loop_ms * 1e-3, "d2h_embedding_s": ph[5] - ph[4],
              "close_s": ph[6] - ph[5]}
    return {"value": n_iter / T, "unit": "iterations/s", "fit_transform_s": T, "fit_transform_s_calls": times,
            "iterations": n_iter, "warmup_calls": 1, "phases_session_api": phases,
            "h2d_bytes_per_step": (X.nbytes + Y0.nbytes) / n_iter, "d2h_bytes_per_step": Y0.nbytes / n_iter,
            "api": "tsne_cuda_b200.TSNE.fit_transform -> pymodule_tsne"}


def e2e_sharded(X, hp, Y0, args, rank, local_rank, world):
    """Host X -> host Y through the session C ABI on every rank (the 31-argument symbol carries one device)."""
    import torch
    import torch.distributed as dist
    from tsne_cuda_b200 import distributed
    n_iter = args.e2e_iters

    phases = {}

    def fit(iters):
        t = [time.time()]
        s = distributed.open_session(X.shape[0], hp["num_neighbors"], rank, local_rank, world)
        t.append(time.time())
        s.affinities_from_points(X, hp["perplexity"], 1e-3)
        t.append(time.time())
        s.set_schedule(hp["learning_rate"], hp["early_exaggeration"], 250, 0.5, 0.8)
        s.set_embedding(Y0)
        s.run(iters)
        t.append(time.time())
        y = s.get_embedding()
        dist.barrier()
        s.close()
        t.append(time.time())
        phases.update(open_s=t[1] - t[0], affinities_s=t[2] - t[1], iterations_s=t[3] - t[2], fetch_close_s=t[4] - t[3])
        return y

    fit(20)   # one untimed call, as on a single GPU
    times = []
    for _ in range(3):   # median of three calls, as on a single GPU
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.time()
        Y = fit(n_iter)
        times.append(time.time() - t0)
    T = sorted(times)[1]
    t = torch.tensor([T], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    T = float(t.item())
    assert np.isfinite(Y).all()
    return {"value": n_iter / T, "unit": "iterations/s", "fit_transform_s": T, "iterations": n_iter,
            "h2d_bytes_per_step": (X.nbytes + Y0.nbytes) / n_iter, "d2h_bytes_per_step": Y0.nbytes / n_iter,
            "warmup_calls": 1, "phases_rank0": phases, "api": "b200tsne_session_* on every rank"}


def cpu_baseline(X, hp, Y0, args, budget_s=20.0):
    """The OpenMP restatement of the same iteration (oracle/), timed on a bounded sample: random
    fixed-width affinities of the workload's shape (the iteration's cost does not depend on their
    values) and as many iterations as fit in ~20 s."""
    from oracle import cpu
    N, K = X.shape[0], hp["num_neighbors"]
    rng = np.random.default_rng(1)
    ids = rng.integers(0, N, (N, K), dtype=np.int32)
    P = np.full((N, K), 1.0 / (N * K), np.float32)
    Y = (rng.standard_normal((2, N)) * 10).astype(np.float32)
    t0 = time.time()
    cpu.iterate(P, ids, Y, 1, hp["learning_rate"])
    one = time.time() - t0
    n = int(max(1, min(50, budget_s / max(one, 1e-3))))
    t0 = time.time()
    cpu.iterate(P, ids, Y, n, hp["learning_rate"])
    T = time.time() - t0
    return {"value": n / T, "unit": "iterations/s", "cores": cpu.num_threads(), "kind": "port",
            "sample": "%d full gradient iterations at N=%d K=%d on random affinities of the workload's shape" % (n, N, K)}


def knn_in_child_process(X, K, config, n):
    """The exact neighbour list the reference arm injects, computed by a CHILD python process so that the
    process that times the reference never maps this repository's CUDA library.  The child regenerates the
    seeded workload itself and leaves two .npy files in a temporary directory."""
    import tempfile
    tmp = tempfile.mkdtemp(prefix="b200tsne_knn_")
    code = ("import sys, numpy as np; sys.path.insert(0, %r); from tsne_cuda_b200 import _lib, datasets; "
            "X, hp = datasets.make(%r, n=%r); ids, d2 = _lib.knn(X, %d); "
            "np.save(%r, ids); np.save(%r, d2)" %
            (ROOT, config, n, K, os.path.join(tmp, "ids.npy"), os.path.join(tmp, "d2.npy")))
    subprocess.check_call([sys.executable, "-c", code], stdout=sys.stderr)
    ids, d2 = np.load(os.path.join(tmp, "ids.npy")), np.load(os.path.join(tmp, "d2.npy"))
    for f in ("ids.npy", "d2.npy"):
        os.remove(os.path.join(tmp, f))
    os.rmdir(tmp)
    assert ids.shape == (X.shape[0], K)
    return ids, d2


def run_reference(args):
    """The reference's own CUDA kernels (oracle/_ref, compiled from the reference tree for sm_100) through
    its own pymodule_tsne.  The reference's neighbour search is FAISS, which is not installed; the exact
    neighbour list is computed beforehand, outside the timed region and in another process, and injected.
    `value` comes from the reference's own loop timers: median over five pairs of runs of
    (loop time of warmup + steps iterations) - (loop time of warmup iterations).  When the reference build
    is absent the OpenMP port is timed instead."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from oracle import ref
    X, hp, Y0 = workload(args)
    N, D = X.shape
    K = hp["num_neighbors"]
    base = {"impl": "reference", "metric": "gradient_iterations_per_s", "unit": "iterations/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s: N=%d D=%d K=%d perplexity=%g, 4-component Gaussian mixture, exact kNN" %
                                   (args.config, N, D, K, hp["perplexity"])}}
    if not ref.available():
        cb = cpu_baseline(X, hp, Y0, args, budget_s=60.0)
        base.update({"value": cb["value"], "ms_per_step": 1e3 / cb["value"], "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "iterations/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return base
    ids, d2 = knn_in_child_process(X, K, args.config, args.n)
    ref.set_knn(ids, d2)
    kw = dict(perplexity=hp["perplexity"], learning_rate=hp["learning_rate"], num_neighbors=K,
              early_exaggeration=hp["early_exaggeration"], perplexity_search_epsilon=1e-3)

    def loop_seconds(n_iter):
        Y, tm = ref.fit_transform_timed(X, Y0, iterations=n_iter, **kw)
        return tm["loop_s"], tm, Y

    loop_seconds(max(args.warmup, 3))                      # context, plans, first-use costs
    pairs = []
    with ClockSampler(0) as clk:
        for _ in range(5):
            t_a, _, _ = loop_seconds(args.warmup)
            t_b, tm, Y = loop_seconds(args.warmup + args.steps)
            pairs.append(max(t_b - t_a, 1e-9))
    loop = float(np.median(pairs))
    value = args.steps / loop
    e2e = {"value": value, "unit": "iterations/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
           "note": "same as value: the full-length fit was skipped (--no-e2e)"}
    if not args.no_e2e:
        t0 = time.time()
        Yf = ref.fit_transform(X, Y0, iterations=args.e2e_iters, **kw)
        T = time.time() - t0
        e2e = {"value": args.e2e_iters / T, "unit": "iterations/s", "fit_transform_s": T, "iterations": args.e2e_iters,
               "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
               "note": "one fit of the same length as this engine's e2e, host X -> host Y, wall clock; EXCLUDES the "
                       "neighbour search (injected), which this engine's e2e includes",
               "finite": bool(np.isfinite(Yf).all())}
    base.update({"value": value, "ms_per_step": loop / args.steps * 1e3, "clocks": clk.summary(),
                 "iterations_per_s_pairs": [args.steps / p for p in pairs],
                 "reference_timers_last_run": {k: v for k, v in tm.items()},
                 "cpu_baseline": {"value": value, "unit": "iterations/s", "cores": 1, "kind": "reference",
                                  "sample": "reference CUDA kernels on the GPU driven by one host thread; median of 5 "
                                            "differences of the reference's own loop timers between runs of %d and %d "
                                            "iterations, neighbour list injected" % (args.warmup, args.warmup + args.steps)},
                 "e2e": e2e, "finite": bool(np.isfinite(Y).all())})
    return base


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c3")
    ap.add_argument("--n", type=int, default=None, help="override the number of points (debugging)")
    ap.add_argument("--e2e-iters", type=int, default=1000)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # Libraries (NCCL's version banner for one) write to file descriptor 1; the contract is ONE JSON
    # line on stdout, so everything written during the run goes to stderr instead.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        out = run_reference(args) if args.impl == "reference" else run_ours(args)
    finally:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
