"""Loader for oracle/_ref/libtsnecuda_ref.so: the reference's own CUDA sources compiled for sm_100
(see oracle/ref_build/).  Test infrastructure; needs a GPU.  `available()` is False when the library
has not been built (it cannot be built without the reference tree)."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libtsnecuda_ref.so")
_lib = None
_keep = []
_fp, _ip = C.POINTER(C.c_float), C.POINTER(C.c_int32)


def available():
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH)
        L.ref_max_normalize.argtypes = [_fp, C.c_longlong]
        L.ref_perplexity.argtypes = [_fp, C.c_int, C.c_int, C.c_float, C.c_float, _fp]
        L.ref_symmetrize.argtypes = [_fp, _ip, C.c_int, C.c_int, _fp]
        L.ref_attractive.argtypes = [_fp, _ip, _fp, C.c_int, C.c_int, _fp]
        L.ref_repulsive.argtypes = [_fp, C.c_int, _fp, _fp, _fp, _fp, _fp]
        L.ref_apply_forces.argtypes = [_fp, _fp, _fp, _fp, _fp, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]
        L.ref_set_knn.argtypes = [C.POINTER(C.c_int64), _fp, C.c_longlong, C.c_int]
        L.ref_run_seeded.argtypes = [_fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _fp]
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(_fp) if a is not None else None


def _i(a):
    return a.ctypes.data_as(_ip)


def max_normalize(d2):
    out = np.array(d2, np.float32, copy=True, order="C")
    lib().ref_max_normalize(_f(out), out.size)
    return out


def perplexity(dhat, perp, eps):
    dhat = np.ascontiguousarray(dhat, np.float32)
    p = np.empty_like(dhat)
    lib().ref_perplexity(_f(dhat), dhat.shape[0], dhat.shape[1], perp, eps, _f(p))
    return p


def symmetrize(p, ids):
    p = np.ascontiguousarray(p, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    P = np.empty_like(p)
    lib().ref_symmetrize(_f(p), _i(ids), p.shape[0], p.shape[1], _f(P))
    return P


def attractive(P, ids, Y):
    P = np.ascontiguousarray(P, np.float32)
    ids = np.ascontiguousarray(ids, np.int32)
    Y = np.ascontiguousarray(Y, np.float32)
    F = np.empty((2, P.shape[0]), np.float32)
    lib().ref_attractive(_f(P), _i(ids), _f(Y), P.shape[0], P.shape[1], _f(F))
    return F


def repulsive(Y, want_grids=False):
    Y = np.ascontiguousarray(Y, np.float32)
    N = Y.shape[1]
    F = np.empty((2, N), np.float32)
    Z = C.c_float()
    w = np.empty((390, 390, 4), np.float32) if want_grids else None
    yt = np.empty((390, 390, 4), np.float32) if want_grids else None
    phi = np.empty((N, 4), np.float32) if want_grids else None
    lib().ref_repulsive(_f(Y), N, _f(F), C.byref(Z), _f(w), _f(yt), _f(phi))
    return (F, Z.value, w, yt, phi) if want_grids else (F, Z.value)


def apply_forces(Y, attr, rep, gains, old, eta, Z, momentum, exag):
    Y, attr, rep, gains, old = [np.array(a, np.float32, copy=True, order="C") for a in (Y, attr, rep, gains, old)]
    lib().ref_apply_forces(_f(Y), _f(attr), _f(rep), _f(gains), _f(old), eta, Z, momentum, exag, Y.shape[1])
    return Y, gains, old


def set_knn(ids, d2):
    """Inject a neighbour list that the next pymodule_tsne call of the reference build will use
    instead of searching (ids (N,K) any int dtype, d2 (N,K) float32 unnormalised squared distances)."""
    ids64 = np.ascontiguousarray(ids, np.int64)
    d2 = np.ascontiguousarray(d2, np.float32)
    _keep[:] = [ids64, d2]
    lib().ref_set_knn(ids64.ctypes.data_as(C.POINTER(C.c_int64)), _f(d2), ids64.shape[0], ids64.shape[1])


def clear_knn():
    _keep[:] = []
    lib().ref_set_knn(None, None, 0, 0)


def run_seeded(X, init_type, seed, iterations=0, num_neighbors=30, perplexity=10.0):
    """tsnecuda::RunTsne of the reference with Options::random_seed = seed; init_type 0 UNIFORM, 1 GAUSSIAN.
    Returns Y (2,N) SoA; with iterations = 0 that is the initial embedding the reference draws."""
    X = np.ascontiguousarray(X, np.float32)
    N, D = X.shape
    Y = np.zeros((2, N), np.float32)
    lib().ref_run_seeded(_f(X), N, D, init_type, seed, iterations, num_neighbors, perplexity, _f(Y))
    return Y


LOOP_TIMERS = ("_time_other", "_time_compute_charges", "_time_precompute_2d", "_time_nbodyfft", "_time_norm",
               "_time_attr", "_time_apply_forces")


def fit_transform_timed(X, y0=None, **kw):
    """fit_transform with verbosity 1, returning (Y, timers): the reference's own `_time_*: <s>s` lines
    (src/fit_tsne.cu:586-601) parsed into a dict.  timers["loop_s"] is the sum of the seven timers the
    reference accumulates inside its gradient loop (src/fit_tsne.cu:402-544); they are host clocks around
    phases that each end in a host synchronisation or follow one, so their sum is the loop's wall time.
    print_interval is pushed out of reach so that verbosity adds one norm computation, at step 0."""
    import re
    import tempfile
    kw = dict(kw, verbosity=1, print_interval=1 << 30)
    with tempfile.TemporaryFile(mode="w+b") as tmp:
        saved = os.dup(1)
        os.dup2(tmp.fileno(), 1)
        try:
            Y = fit_transform(X, y0, **kw)
        finally:
            os.dup2(saved, 1)
            os.close(saved)
        tmp.seek(0)
        text = tmp.read().decode(errors="replace")
    timers = {m.group(1): float(m.group(2)) for m in re.finditer(r"^(_time_\w+|total_time): ([0-9.eE+-]+)s\s*$", text, re.M)}
    timers["loop_s"] = sum(timers.get(k, 0.0) for k in LOOP_TIMERS)
    return Y, timers


def fit_transform(X, y0=None, **kw):
    """The reference's pymodule_tsne through the reference's argument order (src/ext/pymodule_ext.cu:6-40).
    Returns Y as (2,N) SoA."""
    L = lib()
    X = np.ascontiguousarray(X, np.float32)
    N, D = X.shape
    res = np.zeros((2, N), np.float32)
    dims = (C.c_ssize_t * 2)(N, D)
    pre = np.ascontiguousarray(y0, np.float32) if y0 is not None else np.zeros((1, 1), np.float32)
    g = lambda k, d: kw.get(k, d)
    empty = np.zeros(1, np.uint8)
    L.pymodule_tsne.restype = None
    L.pymodule_tsne.argtypes = [_fp, _fp, C.POINTER(C.c_ssize_t)] + [C.c_float] * 4 + [C.c_int] * 4 + [C.c_float] * 6 + \
        [C.c_int, _fp, C.c_bool, C.c_char_p, C.c_int, C.c_bool, C.c_char_p] + [C.c_int] * 7
    L.pymodule_tsne(_f(res), _f(X), dims, g("perplexity", 50.0), g("learning_rate", 200.0),
                    g("early_exaggeration", 12.0), 5.0, g("num_neighbors", 32), g("iterations", 1000), 1000,
                    g("force_magnify_iters", 250), g("perplexity_search_epsilon", 1e-3), g("pre_momentum", 0.5),
                    g("post_momentum", 0.8), 0.5, 0.0025, 0.0, 3 if y0 is not None else 1, _f(pre), False, b"", 1,
                    False, b"", 10000, g("verbosity", 0), g("print_interval", 10), 0, 0, 0, 1)
    return res
