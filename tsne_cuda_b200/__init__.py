"""B200-native FIt-SNE engine behind the tsnecuda API.

`TSNE` mirrors the reference's `tsnecuda.TSNE`; `_lib` binds the C ABI of libtsnecuda.so
(stage entry points and the device-resident session).  There is no CPU fallback: the CUDA
library must be built (`python -m tsne_cuda_b200.build`).
"""
from .TSNE import TSNE  # noqa: F401


def test():
    """Smoke run with the reference's own smoke input (src/python/tsnecuda/__init__.py:4-7)."""
    import numpy as np
    return TSNE(verbose=1).fit_transform(np.random.random((5000, 50)))
