"""CPU suite: the C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments with status codes before touching CUDA."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tsnecuda_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(b200tsne_\w+|pymodule_tsne)\s*\(", text))
    return sorted(n for n in names)


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for must in ("pymodule_tsne", "b200tsne_fit", "b200tsne_knn", "b200tsne_perplexity", "b200tsne_symmetrize",
                 "b200tsne_attractive", "b200tsne_repulsive", "b200tsne_apply_forces", "b200tsne_session_run"):
        assert must in syms


def test_library_exports_every_declared_symbol(engine):
    for name in declared_symbols():
        assert hasattr(engine.lib, name), "libtsnecuda.so does not export %s" % name
    # and the Python binding lists every one of them
    assert set(declared_symbols()) <= set(engine.SIGNATURES)


def test_cpp_entry_point_is_exported(engine):
    import subprocess
    out = subprocess.check_output(["nm", "-DC", engine.LIB_PATH], text=True)
    assert "tsnecuda::RunTsne(tsnecuda::Options&, tsnecuda::GpuOptions&)" in out
    assert "tsnecuda::GpuOptions::GpuOptions(int)" in out


def test_invalid_arguments_return_status_without_a_gpu(engine):
    lib = engine.lib
    x = np.zeros((4, 3), np.float32)
    ids = np.zeros((4, 2), np.int32)
    d2 = np.zeros((4, 2), np.float32)
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    i = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    assert lib.b200tsne_knn(None, 4, 3, 2, 0, 4, 0, 4, i(ids), f(d2), 0) == -1
    assert lib.b200tsne_knn(f(x), 4, 3, 0, 0, 4, 0, 4, i(ids), f(d2), 0) == -1
    assert lib.b200tsne_knn(f(x), 4, 3, 2, 3, 2, 0, 4, i(ids), f(d2), 0) == -1
    assert b"invalid" in lib.b200tsne_last_error()
    assert lib.b200tsne_perplexity(f(d2), 4, 2, -1.0, 1e-3, 0.0, f(d2), None, None, 0) == -1
    assert lib.b200tsne_symmetrize(f(d2), i(ids), 0, 2, f(d2), 0) == -1
    assert lib.b200tsne_attractive(f(d2), i(ids), f(d2), 4, 2, 3, 2, f(d2), 0) == -1
    assert lib.b200tsne_session_run(None, 1, 0.0, None, None) == -1
    o = engine.Options()
    lib.b200tsne_default_options(C.byref(o))
    assert (o.perplexity, o.num_neighbors, o.iterations, o.force_magnify_iters) == (50.0, 1023, 1000, 250)
    res = np.zeros((2, 4), np.float32)
    o.initialization_type = 7
    assert lib.b200tsne_fit(f(x), 4, 3, C.byref(o), f(res), None) == -1
    o.initialization_type = 1
    o.return_style = 5
    assert lib.b200tsne_fit(f(x), 4, 3, C.byref(o), f(res), None) == -1
    assert lib.b200tsne_fit(None, 4, 3, C.byref(o), f(res), None) == -1


def test_python_front_end_validates_like_the_reference():
    from tsne_cuda_b200 import TSNE
    # exception types of the reference's wrapper (src/python/tsnecuda/TSNE.py:73-94, :129-130)
    with pytest.raises(NotImplementedError):
        TSNE(n_components=3)
    with pytest.raises(NotImplementedError):
        TSNE(metric="cosine")
    with pytest.raises(NotImplementedError):
        TSNE(init="pca")
    with pytest.raises(ValueError):
        TSNE(return_style="sometimes")
    t = TSNE(perplexity=30, num_neighbors=90, metric="innerproduct", return_style="snapshots", num_snapshots=4)
    assert (t.metric, t.return_style, t.num_snapshots, t.perplexity_epsilon) == (0, 1, 4, 1e-3)
    args = t._lib.pymodule_tsne.argtypes
    assert len(args) == 31


def test_no_gpu_means_a_loud_error_not_a_fallback(engine):
    """Without a CUDA device the product reports a CUDA error; it never computes on the CPU."""
    import ctypes.util  # noqa: F401
    x = np.random.default_rng(0).normal(size=(64, 5)).astype(np.float32)
    try:
        engine.knn(x, 4)
    except engine.TsneError as e:
        assert "CUDA" in str(e) or "device" in str(e)
    else:
        # a GPU is present: then the answer must be the CUDA library's (exactness is tested in the gpu suite)
        pass
