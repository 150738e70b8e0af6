"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The public datasets the reference quotes numbers on (MNIST, CIFAR-10 features) are not available
offline; these generators stand in for them.  Every generator is deterministic in its seed.
"""
import numpy as np


def gaussian_mixture(n, d=50, components=4, seed=20240, chunk=1 << 18):
    """Isotropic unit-variance mixture, equal weights, component means ~ N(0, 10^2 I)."""
    rng = np.random.default_rng(seed)
    mu = rng.normal(0.0, 10.0, (components, d)).astype(np.float32)
    X = np.empty((n, d), np.float32)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        X[lo:hi] = mu[np.arange(lo, hi) % components] + rng.standard_normal((hi - lo, d), dtype=np.float32)
    return X


def mnist_shaped(n=60000, d=784, classes=10, seed=20241):
    """[0,1] pixels: per-class prototype with ~80 % exact zeros, Gaussian noise 0.1, zero mask kept."""
    rng = np.random.default_rng(seed)
    mask = rng.random((classes, d)) >= 0.8
    proto = (rng.random((classes, d)) * mask).astype(np.float32)
    lab = np.arange(n) % classes
    X = proto[lab] + rng.normal(0.0, 0.1, (n, d)).astype(np.float32)
    np.clip(X, 0.0, 1.0, out=X)
    X *= mask[lab]
    return np.ascontiguousarray(X, np.float32)


def feature_shaped(n=50000, d=1024, classes=10, seed=20242):
    """ReLU-like classifier features: max(0, mu_c + N(0,1)), mu_c ~ N(0, I)."""
    rng = np.random.default_rng(seed)
    mu = rng.standard_normal((classes, d)).astype(np.float32)
    X = mu[np.arange(n) % classes] + rng.standard_normal((n, d), dtype=np.float32)
    np.maximum(X, 0.0, out=X)
    return X


def initial_embedding(n, seed=7):
    """Y0 ~ N(0, 1e-4^2) as a (2, n) array, injected so that two engines start identically."""
    rng = np.random.default_rng(seed)
    return (1e-4 * rng.standard_normal((2, n))).astype(np.float32)


CONFIGS = {
    # name: (generator, kwargs, perplexity, K, learning_rate (None = N/12), early_exaggeration)
    "c0": (gaussian_mixture, dict(n=5000, d=50, seed=20240), 30.0, 90, 200.0, 12.0),
    "c1": (mnist_shaped, dict(n=60000, d=784), 30.0, 90, 200.0, 12.0),
    "c2": (feature_shaped, dict(n=50000, d=1024), 50.0, 150, 10.0, 12.0),
    "c3": (gaussian_mixture, dict(n=1000000, d=50, seed=20243), 30.0, 90, None, 12.0),
    "c4": (gaussian_mixture, dict(n=10000000, d=50, seed=20244), 30.0, 90, None, 12.0),
}


def make(name, n=None):
    gen, kw, perp, K, lr, exag = CONFIGS[name]
    kw = dict(kw)
    if n is not None:
        kw["n"] = int(n)
    X = gen(**kw)
    if lr is None:
        lr = X.shape[0] / 12.0
    return X, dict(perplexity=perp, num_neighbors=K, learning_rate=float(lr), early_exaggeration=exag)
