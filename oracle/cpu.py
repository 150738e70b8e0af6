"""ctypes wrapper over oracle/tsne_oracle.c (test infrastructure; see that file's header)."""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
F32 = np.float32
I32 = np.int32


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB if os.path.exists(_build.LIB) else _build.build_oracle()
        L = C.CDLL(path)
        fp, ip, dp = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_double)
        L.orc_num_threads.restype = C.c_int
        L.orc_knn.argtypes = [fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, ip, fp]
        L.orc_knn_merge.argtypes = [ip, fp, C.c_int, C.c_int, C.c_int, ip, fp]
        L.orc_max_normalize.argtypes = [fp, C.c_size_t]
        L.orc_max_normalize.restype = C.c_float
        L.orc_perplexity.argtypes = [fp, C.c_int, C.c_int, C.c_float, C.c_float, fp, fp]
        L.orc_symmetrize.argtypes = [fp, ip, C.c_int, C.c_int, fp]
        L.orc_attractive.argtypes = [fp, ip, fp, C.c_int, C.c_int, C.c_int, C.c_int, fp]
        L.orc_minmax.argtypes = [fp, C.c_int, fp, fp]
        L.orc_spread.argtypes = [fp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, fp]
        L.orc_convolve.argtypes = [fp, C.c_float, C.c_float, fp]
        L.orc_gather.argtypes = [fp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, fp, fp, fp]
        L.orc_gather.restype = C.c_double
        L.orc_repulsive.argtypes = [fp, C.c_int, fp, fp, fp, fp, fp]
        L.orc_repulsive_exact.argtypes = [fp, C.c_int, dp, dp]
        L.orc_apply_forces.argtypes = [fp, fp, fp, fp, fp, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int]
        L.orc_iterate.argtypes = [fp, ip, fp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                                  C.c_float, C.c_int, C.c_float, C.c_float]
        L.orc_iterate.restype = C.c_float
        L.orc_affinities.argtypes = [fp, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, ip, fp]
        L.orc_kl_divergence.argtypes = [fp, ip, fp, C.c_int, C.c_int]
        L.orc_kl_divergence.restype = C.c_double
        L.orc_nn_preservation.argtypes = [ip, C.c_int, fp, C.c_int, C.c_int]
        L.orc_nn_preservation.restype = C.c_double
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def _d(a):
    return a.ctypes.data_as(C.POINTER(C.c_double))


def G():
    return 390


def num_threads():
    return lib().orc_num_threads()


def knn(X, K, q_lo=0, q_hi=None, db_lo=0, db_hi=None):
    X = np.ascontiguousarray(X, F32)
    N, D = X.shape
    q_hi = N if q_hi is None else q_hi
    db_hi = N if db_hi is None else db_hi
    ids = np.empty((q_hi - q_lo, K), I32)
    d2 = np.empty((q_hi - q_lo, K), F32)
    lib().orc_knn(_f(X), N, D, K, q_lo, q_hi, db_lo, db_hi, _i(ids), _f(d2))
    return ids, d2


def knn_merge(ids_parts, d2_parts):
    ids_parts = np.ascontiguousarray(ids_parts, I32)
    d2_parts = np.ascontiguousarray(d2_parts, F32)
    parts, n, K = ids_parts.shape
    ids = np.empty((n, K), I32)
    d2 = np.empty((n, K), F32)
    lib().orc_knn_merge(_i(ids_parts), _f(d2_parts), parts, n, K, _i(ids), _f(d2))
    return ids, d2


def max_normalize(d2):
    out = np.array(d2, F32, copy=True, order="C")
    m = lib().orc_max_normalize(_f(out), out.size)
    return out, m


def perplexity(dhat, perp, eps, return_betas=False):
    dhat = np.ascontiguousarray(dhat, F32)
    N, K = dhat.shape
    p = np.empty((N, K), F32)
    betas = np.empty(N, F32)
    lib().orc_perplexity(_f(dhat), N, K, perp, eps, _f(p), _f(betas))
    return (p, betas) if return_betas else p


def symmetrize(p, ids):
    p = np.ascontiguousarray(p, F32)
    ids = np.ascontiguousarray(ids, I32)
    N, K = p.shape
    P = np.empty((N, K), F32)
    lib().orc_symmetrize(_f(p), _i(ids), N, K, _f(P))
    return P


def attractive(P, ids, Y, lo=0, hi=None):
    """Y: SoA array of shape (2, N). Returns F (2, N) (rows outside [lo,hi) are zero)."""
    P = np.ascontiguousarray(P, F32)
    ids = np.ascontiguousarray(ids, I32)
    Y = np.ascontiguousarray(Y, F32)
    N, K = P.shape
    hi = N if hi is None else hi
    F = np.zeros((2, N), F32)
    lib().orc_attractive(_f(P), _i(ids), _f(Y), N, K, lo, hi, _f(F))
    return F


def minmax(Y):
    Y = np.ascontiguousarray(Y, F32)
    a, b = C.c_float(), C.c_float()
    lib().orc_minmax(_f(Y), Y.shape[1], C.byref(a), C.byref(b))
    return a.value, b.value


def spread(Y, cmin, cmax, lo=0, hi=None):
    Y = np.ascontiguousarray(Y, F32)
    N = Y.shape[1]
    hi = N if hi is None else hi
    w = np.empty((390, 390, 4), F32)
    lib().orc_spread(_f(Y), N, lo, hi, cmin, cmax, _f(w))
    return w


def convolve(w, cmin, cmax):
    w = np.ascontiguousarray(w, F32)
    yt = np.empty((390, 390, 4), F32)
    lib().orc_convolve(_f(w), cmin, cmax, _f(yt))
    return yt


def gather(Y, cmin, cmax, ytilde, lo=0, hi=None):
    Y = np.ascontiguousarray(Y, F32)
    ytilde = np.ascontiguousarray(ytilde, F32)
    N = Y.shape[1]
    hi = N if hi is None else hi
    F = np.zeros((2, N), F32)
    phi = np.zeros((N, 4), F32)
    zs = lib().orc_gather(_f(Y), N, lo, hi, cmin, cmax, _f(ytilde), _f(F), _f(phi))
    return F, zs, phi


def repulsive(Y, want_grids=False):
    """Returns (Frep (2,N), Z) or (Frep, Z, w, ytilde, phi)."""
    Y = np.ascontiguousarray(Y, F32)
    N = Y.shape[1]
    F = np.empty((2, N), F32)
    Z = C.c_float()
    if want_grids:
        w = np.empty((390, 390, 4), F32)
        yt = np.empty((390, 390, 4), F32)
        phi = np.empty((N, 4), F32)
        lib().orc_repulsive(_f(Y), N, _f(F), C.byref(Z), _f(w), _f(yt), _f(phi))
        return F, Z.value, w, yt, phi
    lib().orc_repulsive(_f(Y), N, _f(F), C.byref(Z), None, None, None)
    return F, Z.value


def repulsive_exact(Y):
    Y = np.ascontiguousarray(Y, F32)
    N = Y.shape[1]
    F = np.empty((2, N), np.float64)
    Z = C.c_double()
    lib().orc_repulsive_exact(_f(Y), N, _d(F), C.byref(Z))
    return F, Z.value


def apply_forces(Y, attr, rep, gains, old, eta, Z, momentum, exag):
    """All arrays (2,N) float32; returns updated copies (Y, gains, old)."""
    Y, attr, rep, gains, old = [np.array(a, F32, copy=True, order="C") for a in (Y, attr, rep, gains, old)]
    lib().orc_apply_forces(_f(Y), _f(attr), _f(rep), _f(gains), _f(old), eta, Z, momentum, exag, Y.shape[1])
    return Y, gains, old


def iterate(P, ids, Y, n_steps, eta, exag=12.0, force_magnify_iters=250, pre_m=0.5, post_m=0.8,
            first_step=0, gains=None, old=None):
    P = np.ascontiguousarray(P, F32)
    ids = np.ascontiguousarray(ids, I32)
    Y = np.array(Y, F32, copy=True, order="C")
    N, K = P.shape
    gains = np.ones((2, N), F32) if gains is None else np.array(gains, F32, copy=True, order="C")
    old = np.zeros((2, N), F32) if old is None else np.array(old, F32, copy=True, order="C")
    Z = lib().orc_iterate(_f(P), _i(ids), _f(Y), _f(gains), _f(old), N, K, first_step, n_steps, eta, exag,
                          force_magnify_iters, pre_m, post_m)
    return Y, gains, old, Z


def affinities(X, K, perp, eps):
    X = np.ascontiguousarray(X, F32)
    N, D = X.shape
    ids = np.empty((N, K), I32)
    P = np.empty((N, K), F32)
    lib().orc_affinities(_f(X), N, D, K, perp, eps, _i(ids), _f(P))
    return ids, P


def kl_divergence(P, ids, Y):
    P = np.ascontiguousarray(P, F32)
    ids = np.ascontiguousarray(ids, I32)
    Y = np.ascontiguousarray(Y, F32)
    return lib().orc_kl_divergence(_f(P), _i(ids), _f(Y), P.shape[0], P.shape[1])


def nn_preservation(ids_hi, Y, k=10):
    ids_hi = np.ascontiguousarray(ids_hi, I32)
    Y = np.ascontiguousarray(Y, F32)
    return lib().orc_nn_preservation(_i(ids_hi), ids_hi.shape[1], _f(Y), Y.shape[1], k)
