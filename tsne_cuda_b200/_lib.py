"""ctypes binding of libtsnecuda.so (the C ABI declared in include/tsnecuda_b200.h).

The library is the product: there is no Python or CPU fallback.  Importing this module without a
built libtsnecuda.so raises ImportError with the build command.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtsnecuda.so")
N_STAGES = 9
G = 390

if not os.path.exists(LIB_PATH):
    raise ImportError("libtsnecuda.so is not built (%s); run `python -m tsne_cuda_b200.build`" % LIB_PATH)

lib = C.CDLL(LIB_PATH)

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int32)
_i64 = C.c_int64


class Options(C.Structure):
    """b200tsne_options of include/tsnecuda_b200.h."""
    _fields_ = [
        ("perplexity", C.c_float), ("learning_rate", C.c_float), ("early_exaggeration", C.c_float),
        ("num_neighbors", C.c_int), ("iterations", C.c_int), ("force_magnify_iters", C.c_int),
        ("perplexity_search_epsilon", C.c_float), ("pre_exaggeration_momentum", C.c_float),
        ("post_exaggeration_momentum", C.c_float), ("min_gradient_norm", C.c_float),
        ("initialization_type", C.c_int), ("preinit_data", _fp), ("random_seed", C.c_int),
        ("verbosity", C.c_int), ("print_interval", C.c_int), ("gpu_device", C.c_int),
        ("return_style", C.c_int), ("num_snapshots", C.c_int), ("dump_file", C.c_char_p),
        ("dump_interval", C.c_int),
    ]


# name -> (restype, argtypes); every symbol the header declares is listed here
SIGNATURES = {
    "b200tsne_last_error": (C.c_char_p, []),
    "b200tsne_version": (C.c_int, []),
    "pymodule_tsne": (None, None),  # bound by TSNE.py with the reference's own argtypes
    "b200tsne_default_options": (None, [C.POINTER(Options)]),
    "b200tsne_fit": (C.c_int, [_fp, _i64, C.c_int, C.POINTER(Options), _fp, _fp]),
    "b200tsne_fit_with_frames": (C.c_int, [_fp, _i64, C.c_int, C.POINTER(Options), _fp, _fp, C.c_void_p, C.c_void_p, C.c_int]),
    "b200tsne_knn": (C.c_int, [_fp, _i64, C.c_int, C.c_int, _i64, _i64, _i64, _i64, _ip, _fp, C.c_int]),
    "b200tsne_knn_last_stats": (C.c_int, [C.POINTER(C.c_int), C.POINTER(C.c_int), _fp]),
    "b200tsne_knn_noalloc": (C.c_int, [C.c_void_p, _i64, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tsne_knn_noalloc_max_elements": (_i64, []),
    "b200tsne_perplexity": (C.c_int, [_fp, _i64, C.c_int, C.c_float, C.c_float, C.c_float, _fp, _fp, _fp, C.c_int]),
    "b200tsne_symmetrize": (C.c_int, [_fp, _ip, _i64, C.c_int, _fp, C.c_int]),
    "b200tsne_attractive": (C.c_int, [_fp, _ip, _fp, _i64, C.c_int, _i64, _i64, _fp, C.c_int]),
    "b200tsne_attractive_blocked": (C.c_int, [_fp, _ip, _fp, _i64, C.c_int, _i64, _i64, _fp, C.c_int, _fp, _fp, C.c_int]),
    "b200tsne_attractive_symmetric": (C.c_int, [_fp, _ip, _fp, _i64, C.c_int, _fp, C.c_int, _fp, _fp, C.POINTER(_i64), _fp,
                                                 C.POINTER(C.c_int), C.c_int]),
    "b200tsne_session_set_symmetric": (C.c_int, [C.c_void_p, C.c_int]),
    "b200tsne_session_attractive_mode": (C.c_int, [C.c_void_p, _fp]),
    "b200tsne_repulsive": (C.c_int, [_fp, _i64, _fp, _fp, _fp, _fp, C.c_int]),
    "b200tsne_apply_forces": (C.c_int, [_fp, _fp, _fp, _fp, _fp, C.c_float, C.c_float, C.c_float, C.c_float, _i64, C.c_int]),
    "b200tsne_session_create": (C.c_int, [C.POINTER(C.c_void_p), _i64, C.c_int, _i64, _i64, C.c_int]),
    "b200tsne_session_destroy": (None, [C.c_void_p]),
    "b200tsne_session_set_affinities": (C.c_int, [C.c_void_p, _fp, _ip]),
    "b200tsne_session_affinities_from_points": (C.c_int, [C.c_void_p, _fp, C.c_int, C.c_float, C.c_float]),
    "b200tsne_session_set_embedding": (C.c_int, [C.c_void_p, _fp, C.c_int]),
    "b200tsne_session_get_embedding": (C.c_int, [C.c_void_p, _fp]),
    "b200tsne_session_get_affinities": (C.c_int, [C.c_void_p, _fp, _ip]),
    "b200tsne_session_get_state": (C.c_int, [C.c_void_p, _fp, _fp, _fp, C.POINTER(C.c_int)]),
    "b200tsne_session_set_state": (C.c_int, [C.c_void_p, _fp, _fp, _fp, C.c_int]),
    "b200tsne_session_set_schedule": (C.c_int, [C.c_void_p, C.c_float, C.c_float, C.c_int, C.c_float, C.c_float]),
    "b200tsne_session_run": (C.c_int, [C.c_void_p, C.c_int, C.c_float, _fp, C.POINTER(C.c_int)]),
    "b200tsne_session_stats": (C.c_int, [C.c_void_p, _fp, _fp, C.POINTER(C.c_int)]),
    "b200tsne_session_enable_stage_timers": (C.c_int, [C.c_void_p, C.c_int]),
    "b200tsne_session_stage_times": (C.c_int, [C.c_void_p, _fp, C.POINTER(_i64)]),
    "b200tsne_stage_name": (C.c_char_p, [C.c_int]),
    "b200tsne_session_launch_count": (_i64, [C.c_void_p]),
    "b200tsne_comm_unique_id": (C.c_int, [C.c_void_p]),
    "b200tsne_session_attach_comm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "b200tsne_comm_release_all": (None, []),
    "b200tsne_session_exchange_mode": (C.c_int, [C.c_void_p]),
    "b200tsne_release_cached_memory": (C.c_int, [C.c_int]),
    "b200tsne_session_set_peer_timeout_ms": (C.c_int, [C.c_void_p, C.c_int]),
    "b200tsne_selftest_bounded_waits": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_int), _fp, C.POINTER(C.c_int), _fp]),
}
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    if _args is not None:
        _fn.restype = _res
        _fn.argtypes = _args


class TsneError(RuntimeError):
    pass


def check(rc):
    if rc != 0:
        raise TsneError("libtsnecuda status %d: %s" % (rc, lib.b200tsne_last_error().decode()))


def _f(a):
    return a.ctypes.data_as(_fp) if a is not None else None


def _i(a):
    return a.ctypes.data_as(_ip) if a is not None else None


def _c(a, dt):
    return np.ascontiguousarray(a, dt)


# ---- stage entry points (host buffers) ---------------------------------------------------------
def knn(X, K, q_lo=0, q_hi=None, db_lo=0, db_hi=None, device=0):
    X = _c(X, np.float32)
    N, D = X.shape
    q_hi = N if q_hi is None else q_hi
    db_hi = N if db_hi is None else db_hi
    ids = np.empty((q_hi - q_lo, K), np.int32)
    d2 = np.empty((q_hi - q_lo, K), np.float32)
    check(lib.b200tsne_knn(_f(X), N, D, K, q_lo, q_hi, db_lo, db_hi, _i(ids), _f(d2), device))
    return ids, d2


def knn_last_stats():
    tc, rows, ratio = C.c_int(), C.c_int(), C.c_float()
    lib.b200tsne_knn_last_stats(C.byref(tc), C.byref(rows), C.byref(ratio))
    return {"tensor_core": tc.value, "rows_recomputed": rows.value, "filter_error_ratio": ratio.value}


def perplexity(d2, perp, eps, max_override=0.0, device=0):
    """Returns (p, betas, max)."""
    d2 = _c(d2, np.float32)
    N, K = d2.shape
    p = np.empty((N, K), np.float32)
    betas = np.empty(N, np.float32)
    mx = C.c_float()
    check(lib.b200tsne_perplexity(_f(d2), N, K, perp, eps, max_override, _f(p), _f(betas), C.byref(mx), device))
    return p, betas, mx.value


def symmetrize(p, ids, device=0):
    p = _c(p, np.float32)
    ids = _c(ids, np.int32)
    N, K = p.shape
    P = np.empty((N, K), np.float32)
    check(lib.b200tsne_symmetrize(_f(p), _i(ids), N, K, _f(P), device))
    return P


def attractive(P, ids, Y, row_lo=0, row_hi=None, device=0):
    """Y: (2,N) SoA. Returns F (2,N)."""
    P = _c(P, np.float32)
    ids = _c(ids, np.int32)
    Y = _c(Y, np.float32)
    N, K = P.shape
    row_hi = N if row_hi is None else row_hi
    F = np.empty((2, N), np.float32)
    check(lib.b200tsne_attractive(_f(P), _i(ids), _f(Y), N, K, row_lo, row_hi, _f(F), device))
    return F


def attractive_blocked(P, ids, Y, X=None, row_lo=0, row_hi=None, device=0):
    """The attractive force through the column-blocked copy of P. Returns (F (2,N), entries per row and tile)."""
    P = _c(P, np.float32)
    ids = _c(ids, np.int32)
    Y = _c(Y, np.float32)
    N, K = P.shape
    row_hi = N if row_hi is None else row_hi
    F = np.zeros((2, N), np.float32)
    epg = C.c_float()
    D = 0
    if X is not None:
        X = _c(X, np.float32)
        D = X.shape[1]
    check(lib.b200tsne_attractive_blocked(_f(P), _i(ids), _f(Y), N, K, row_lo, row_hi, _f(X), D, _f(F), C.byref(epg), device))
    return F, epg.value


def attractive_symmetric(p, ids, Y, X=None, device=0):
    """Force under the truly symmetric P = (p + p^T) / 2N.  Returns (F (2,N), P_fixed (N,K), number of extra entries,
    their sum, 1 if the blocked kernel ran)."""
    p = _c(p, np.float32)
    ids = _c(ids, np.int32)
    Y = _c(Y, np.float32)
    N, K = p.shape
    F = np.zeros((2, N), np.float32)
    P = np.zeros((N, K), np.float32)
    n_extra, s_extra, blocked = _i64(), C.c_float(), C.c_int()
    D = 0
    if X is not None:
        X = _c(X, np.float32)
        D = X.shape[1]
    check(lib.b200tsne_attractive_symmetric(_f(p), _i(ids), _f(Y), N, K, _f(X), D, _f(F), _f(P), C.byref(n_extra), C.byref(s_extra),
                                            C.byref(blocked), device))
    return F, P, n_extra.value, s_extra.value, blocked.value


def repulsive(Y, want_grids=False, device=0):
    """Y: (2,N) SoA. Returns (Frep, Z) or (Frep, Z, w, ytilde)."""
    Y = _c(Y, np.float32)
    N = Y.shape[1]
    F = np.empty((2, N), np.float32)
    Z = C.c_float()
    w = np.empty((G, G, 4), np.float32) if want_grids else None
    yt = np.empty((G, G, 4), np.float32) if want_grids else None
    check(lib.b200tsne_repulsive(_f(Y), N, _f(F), C.byref(Z), _f(w), _f(yt), device))
    return (F, Z.value, w, yt) if want_grids else (F, Z.value)


def apply_forces(Y, attr, rep, gains, old, eta, Z, momentum, exag, device=0):
    Y, attr, rep, gains, old = [np.array(a, np.float32, copy=True, order="C") for a in (Y, attr, rep, gains, old)]
    check(lib.b200tsne_apply_forces(_f(Y), _f(attr), _f(rep), _f(gains), _f(old), eta, Z, momentum, exag,
                                    Y.shape[1], device))
    return Y, gains, old


def fit(X, **kw):
    """b200tsne_fit; keyword names are the fields of b200tsne_options. Returns (Y (2,N) SoA, Z)."""
    X = _c(X, np.float32)
    N, D = X.shape
    o = Options()
    lib.b200tsne_default_options(C.byref(o))
    keep = []
    for k, v in kw.items():
        if k == "preinit_data":
            v = _c(v, np.float32)
            keep.append(v)
            o.preinit_data = _f(v)
        elif k == "dump_file":
            o.dump_file = v.encode() if isinstance(v, str) else v
        else:
            setattr(o, k, v)
    blocks = o.num_snapshots if o.return_style == 1 else 1
    Y = np.zeros((max(blocks, 1), 2, N), np.float32)
    Z = C.c_float()
    check(lib.b200tsne_fit(_f(X), N, D, C.byref(o), _f(Y), C.byref(Z)))
    return (Y[0] if blocks <= 1 else Y), Z.value


FRAME_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t)


def fit_with_frames(X, on_frame, every=1, **kw):
    """b200tsne_fit_with_frames: on_frame(bytes) is called with the text frame (number of points) and then with
    one raw float32 frame (2N values) after every `every`-th iteration; it returns True/None to go on, False for
    "gone".  Returns (Y (2,N) SoA, Z)."""
    X = _c(X, np.float32)
    N, D = X.shape
    o = Options()
    lib.b200tsne_default_options(C.byref(o))
    keep = []
    for k, v in kw.items():
        if k == "preinit_data":
            v = _c(v, np.float32)
            keep.append(v)
            o.preinit_data = _f(v)
        else:
            setattr(o, k, v)

    def trampoline(user, data, nbytes):
        ok = on_frame(C.string_at(data, nbytes))
        return 0 if (ok is None or ok) else 1

    cb = FRAME_FN(trampoline)
    Y = np.zeros((2, N), np.float32)
    Z = C.c_float()
    check(lib.b200tsne_fit_with_frames(_f(X), N, D, C.byref(o), _f(Y), C.byref(Z), C.cast(cb, C.c_void_p), None, int(every)))
    return Y, Z.value


# ---- device-resident session -------------------------------------------------------------------
class Session(object):
    """The gradient loop with everything resident in HBM (b200tsne_session_*)."""

    def __init__(self, N, K, row_lo=0, row_hi=None, device=0):
        self.N, self.K = int(N), int(K)
        self.row_lo = int(row_lo)
        self.row_hi = self.N if row_hi is None else int(row_hi)
        self._h = C.c_void_p()
        check(lib.b200tsne_session_create(C.byref(self._h), self.N, self.K, self.row_lo, self.row_hi, device))

    def close(self):
        if self._h:
            lib.b200tsne_session_destroy(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def set_affinities(self, P_rows, ids_rows):
        P_rows = _c(P_rows, np.float32)
        ids_rows = _c(ids_rows, np.int32)
        assert P_rows.shape == (self.row_hi - self.row_lo, self.K) == ids_rows.shape
        check(lib.b200tsne_session_set_affinities(self._h, _f(P_rows), _i(ids_rows)))

    def affinities_from_points(self, X, perplexity, epsilon):
        X = _c(X, np.float32)
        assert X.shape[0] == self.N
        check(lib.b200tsne_session_affinities_from_points(self._h, _f(X), X.shape[1], perplexity, epsilon))

    def get_affinities(self):
        r = self.row_hi - self.row_lo
        P = np.empty((r, self.K), np.float32)
        ids = np.empty((r, self.K), np.int32)
        check(lib.b200tsne_session_get_affinities(self._h, _f(P), _i(ids)))
        return P, ids

    def set_embedding(self, Y, reset=True):
        Y = _c(Y, np.float32)
        assert Y.shape == (2, self.N)
        check(lib.b200tsne_session_set_embedding(self._h, _f(Y), 1 if reset else 0))

    def get_embedding(self):
        Y = np.empty((2, self.N), np.float32)
        check(lib.b200tsne_session_get_embedding(self._h, _f(Y)))
        return Y

    def get_state(self):
        """(Y (2,N), momentum (2,rows), gains (2,rows), step): everything a later session needs to continue."""
        r = self.row_hi - self.row_lo
        Y = np.empty((2, self.N), np.float32)
        mom = np.empty((2, r), np.float32)
        gains = np.empty((2, r), np.float32)
        step = C.c_int()
        check(lib.b200tsne_session_get_state(self._h, _f(Y), _f(mom), _f(gains), C.byref(step)))
        return Y, mom, gains, step.value

    def set_state(self, Y, momentum, gains, step):
        Y, momentum, gains = _c(Y, np.float32), _c(momentum, np.float32), _c(gains, np.float32)
        check(lib.b200tsne_session_set_state(self._h, _f(Y), _f(momentum), _f(gains), int(step)))

    def set_schedule(self, learning_rate=200.0, early_exaggeration=12.0, force_magnify_iters=250,
                     pre_momentum=0.5, post_momentum=0.8):
        check(lib.b200tsne_session_set_schedule(self._h, learning_rate, early_exaggeration, force_magnify_iters,
                                                pre_momentum, post_momentum))

    def run(self, n_iters, min_gradient_norm=0.0):
        """Returns (device milliseconds of the loop, iterations done)."""
        ms = C.c_float()
        done = C.c_int()
        check(lib.b200tsne_session_run(self._h, n_iters, min_gradient_norm, C.byref(ms), C.byref(done)))
        return ms.value, done.value

    def stats(self):
        Z, un, st = C.c_float(), C.c_float(), C.c_int()
        check(lib.b200tsne_session_stats(self._h, C.byref(Z), C.byref(un), C.byref(st)))
        return {"Z": Z.value, "update_norm": un.value, "step": st.value}

    def enable_stage_timers(self, on=True):
        check(lib.b200tsne_session_enable_stage_timers(self._h, 1 if on else 0))

    def stage_times(self):
        ms = (C.c_float * N_STAGES)()
        n = (_i64 * N_STAGES)()
        check(lib.b200tsne_session_stage_times(self._h, ms, n))
        return {lib.b200tsne_stage_name(k).decode(): (ms[k], n[k]) for k in range(N_STAGES)}

    def launch_count(self):
        return lib.b200tsne_session_launch_count(self._h)

    def exchange_mode(self):
        """0 single GPU, 1 NCCL collectives, 2 peer memory (see include/tsnecuda_b200.h)."""
        return lib.b200tsne_session_exchange_mode(self._h)

    def set_symmetric(self, on=True):
        """Before affinities_from_points: P truly symmetric, (p + p^T) / 2N, instead of the reference's fixed-width form."""
        check(lib.b200tsne_session_set_symmetric(self._h, 1 if on else 0))

    def attractive_mode(self):
        """(1 if the loop uses the column-blocked copy of P else 0, sampled entries per row and tile)."""
        epg = C.c_float()
        m = lib.b200tsne_session_attractive_mode(self._h, C.byref(epg))
        return m, epg.value

    def set_peer_timeout_ms(self, ms):
        """Limit of one meeting of the ranks (peer-memory exchange only)."""
        check(lib.b200tsne_session_set_peer_timeout_ms(self._h, int(ms)))

    def attach_comm(self, unique_id, rank, world_size):
        buf = C.create_string_buffer(bytes(unique_id), 128)
        check(lib.b200tsne_session_attach_comm(self._h, buf, rank, world_size))


def selftest_bounded_waits(timeout_ms=20, device=0):
    """Makes the two bounded device-side waits run out on purpose (nothing faults or hangs); returns
    {"peer": (status, ms), "barrier": (status, ms)} where status -5 means the wait gave up as designed."""
    ps, bs, pm, bm = C.c_int(), C.c_int(), C.c_float(), C.c_float()
    check(lib.b200tsne_selftest_bounded_waits(device, int(timeout_ms), C.byref(ps), C.byref(pm), C.byref(bs), C.byref(bm)))
    return {"peer": (ps.value, pm.value), "barrier": (bs.value, bm.value)}


def comm_unique_id():
    buf = C.create_string_buffer(128)
    check(lib.b200tsne_comm_unique_id(buf))
    return buf.raw


def release_cached_memory(device=0):
    """Return the device memory the library keeps for reuse to the driver."""
    check(lib.b200tsne_release_cached_memory(device))


def comm_release_all():
    """Destroy the communicators the library cached (every session that used one must be closed)."""
    lib.b200tsne_comm_release_all()
