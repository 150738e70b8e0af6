"""float64 NumPy restatement of the FIt-SNE stages (test infrastructure).

Independent of oracle/tsne_oracle.c: used to cross-check it on small inputs.  Citations are to the
reference project (paths relative to its root).
"""
import numpy as np

N_BOXES, N_INTERP, G = 130, 3, 390


def knn(X, K):
    """Exact kNN in float64, ties by index (self included)."""
    X = np.asarray(X, np.float64)
    d = ((X[:, None, :] - X[None, :, :]) ** 2).sum(-1)
    order = np.lexsort((np.broadcast_to(np.arange(len(X)), d.shape), d), axis=1)[:, :K]
    return order.astype(np.int32), np.take_along_axis(d, order, 1)


def perplexity(dhat, perp, eps, max_iter=200):
    """src/kernels/perplexity_search.cu:35-79 in float64."""
    dhat = np.asarray(dhat, np.float64)
    N, K = dhat.shape
    out = np.empty((N, K))
    big = float(np.finfo(np.float32).max)
    for i in range(N):
        beta, lo, hi = 1.0, -big, big
        for _ in range(max_iter):
            p = np.exp(-beta * dhat[i])
            if dhat[i, 0] == 0:
                p[0] = 0.0
            S = p.sum()
            with np.errstate(divide="ignore", invalid="ignore"):
                e = p * np.log(p)
            e[~np.isfinite(e)] = 0.0
            diff = -e.sum() / S + np.log(S) - np.log(perp)
            if abs(diff) < eps:
                break
            if diff > 0:
                lo = beta
                beta = beta * 2 if abs(hi) == big else (beta + hi) / 2
            else:
                hi = beta
                beta = beta / 2 if abs(lo) == big else (beta + lo) / 2
        out[i] = p / S
    return out


def symmetrize(p, ids):
    """src/util/math_utils.cu:269-291."""
    N, K = p.shape
    P = np.array(p, np.float64)
    for i in range(N):
        for s in range(K):
            j = ids[i, s]
            m = ids[j] == i
            P[i, s] += p[j][m].sum()
    return P / (2.0 * N)


def attractive(P, ids, Y):
    """src/kernels/attr_forces.cu:129-184; Y is (2,N)."""
    Y = np.asarray(Y, np.float64)
    dx = Y[0][:, None] - Y[0][ids]
    dy = Y[1][:, None] - Y[1][ids]
    pq = np.asarray(P, np.float64) / (1 + dx * dx + dy * dy)
    return np.stack([(pq * dx).sum(1), (pq * dy).sum(1)])


def _weights(c, cmin, bw):
    idx = np.clip(((c - cmin) / bw).astype(np.int64), 0, N_BOXES - 1)
    xin = (c - (idx * bw + cmin)) / bw
    sp = (np.arange(N_INTERP) + 0.5) / N_INTERP
    L = np.empty((N_INTERP, len(c)))
    for j in range(N_INTERP):
        v = np.ones(len(c))
        den = 1.0
        for k in range(N_INTERP):
            if k != j:
                v *= xin - sp[k]
                den *= sp[j] - sp[k]
        L[j] = v / den
    return idx, L


def repulsive(Y):
    """One evaluation of src/fit_tsne.cu:425-469 in float64, with the 780-point zero-padded
    convolution of src/kernels/nbodyfft.cu (kernel centred at index G, quadrant [G,2G) read back).
    Returns Frep (2,N), Z, w (G,G,4), ytilde (G,G,4)."""
    Y = np.asarray(Y, np.float64)
    x, y = Y
    N = len(x)
    cmin, cmax = Y.min(), Y.max()
    bw = (cmax - cmin) / N_BOXES
    h = bw / N_INTERP
    bx, Lx = _weights(x, cmin, bw)
    by, Ly = _weights(y, cmin, bw)
    ch = np.stack([np.ones(N), x, y, x * x + y * y], 1)
    w = np.zeros((G, G, 4))
    for a in range(3):
        for b in range(3):
            np.add.at(w, (bx * 3 + a, by * 3 + b), (Lx[a] * Ly[b])[:, None] * ch)
    M = 2 * G
    r = np.arange(G) * h
    kq = (1.0 + r[:, None] ** 2 + r[None, :] ** 2) ** -2
    kt = np.zeros((M, M))
    ii = np.arange(G)
    kt[np.ix_(G + ii, G + ii)] = kq
    kt[np.ix_(G - ii, G + ii)] = kq
    kt[np.ix_(G + ii, G - ii)] = kq
    kt[np.ix_(G - ii, G - ii)] = kq
    fk = np.fft.rfft2(kt)
    yt = np.empty((G, G, 4))
    for t in range(4):
        pad = np.zeros((M, M))
        pad[:G, :G] = w[:, :, t]
        yt[:, :, t] = np.fft.irfft2(np.fft.rfft2(pad) * fk, s=(M, M))[G:, G:]
    phi = np.zeros((N, 4))
    for a in range(3):
        for b in range(3):
            phi += (Lx[a] * Ly[b])[:, None] * yt[bx * 3 + a, by * 3 + b]
    Zi = (1 + x * x + y * y) * phi[:, 0] - 2 * (x * phi[:, 1] + y * phi[:, 2]) + phi[:, 3]
    F = np.stack([x * phi[:, 0] - phi[:, 1], y * phi[:, 0] - phi[:, 2]])
    return F, Zi.sum() - N, w, yt


def repulsive_exact(Y):
    Y = np.asarray(Y, np.float64)
    dx = Y[0][:, None] - Y[0][None, :]
    dy = Y[1][:, None] - Y[1][None, :]
    q = 1.0 / (1.0 + dx * dx + dy * dy)
    np.fill_diagonal(q, 0.0)
    return np.stack([(q * q * dx).sum(1), (q * q * dy).sum(1)]), q.sum()


def apply_forces(Y, attr, rep, gains, old, eta, Z, momentum, exag):
    """src/kernels/apply_forces.cu:34-55 in float64."""
    g = exag * attr - rep / Z
    gains = np.where(np.signbit(g) != np.signbit(old), gains + 0.2, gains * 0.8)
    gains = np.maximum(gains, 0.01)
    old = momentum * old - eta * gains * g
    return Y + old, gains, old
