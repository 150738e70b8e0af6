"""GPU suite: the reference's own, unmodified Python wrapper driving this library.

INTEGRATION.md's supported drop-in is "put libtsnecuda.so into the tsnecuda package directory": the reference's
TSNE.py loads `libtsnecuda` from its own directory and binds the one symbol pymodule_tsne
(src/python/tsnecuda/TSNE.py:138-183).  The reference's package files are staged, unmodified, under
oracle/_ref/python/ by the reference build recipe (they are not part of this repository); the test copies
them to a scratch directory, puts this repository's library beside them, and runs the reference's own
smoke call (src/python/tsnecuda/__init__.py:4-7: 5 000 x 50 uniform points) plus a seeded mixture."""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "oracle", "_ref", "python", "tsnecuda")

SCRIPT = r"""
import sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import tsnecuda                                  # the reference's package, unmodified
assert tsnecuda.__file__.startswith(sys.argv[1])
tsnecuda.test()                                  # the reference's own smoke call
rng = np.random.default_rng(0)
mu = rng.normal(0, 10, (4, 50))
X = (mu[np.arange(5000) % 4] + rng.normal(0, 1, (5000, 50))).astype(np.float32)
Y = tsnecuda.TSNE(perplexity=30, num_neighbors=90, n_iter=500).fit_transform(X)
assert Y.shape == (5000, 2) and np.isfinite(Y).all()
lab = np.arange(5000) % 4
cent = np.stack([Y[lab == c].mean(0) for c in range(4)])
near = np.linalg.norm(Y[:, None] - cent[None], axis=2).argmin(1)
assert (near == lab).mean() > 0.99, (near == lab).mean()
for bad in (dict(n_components=3), dict(metric="cosine"), dict(init="pca")):
    try:
        tsnecuda.TSNE(**bad)
    except NotImplementedError:
        pass
    else:
        raise AssertionError(bad)
print("drop-in ok")
"""


def test_unmodified_reference_wrapper_runs_on_this_library(tmp_path):
    if not os.path.exists(os.path.join(STAGED, "TSNE.py")):
        pytest.skip("the reference's Python package was not staged (oracle/_ref is built where the reference tree is)")
    from tsne_cuda_b200 import _lib
    pkg = tmp_path / "tsnecuda"
    shutil.copytree(STAGED, pkg)
    shutil.copyfile(_lib.LIB_PATH, pkg / "libtsnecuda.so")
    r = subprocess.run([sys.executable, "-c", SCRIPT, str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "drop-in ok" in r.stdout
