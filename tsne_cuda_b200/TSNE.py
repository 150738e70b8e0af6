"""sklearn-style front end, mirroring the reference's tsnecuda.TSNE.

Replaces src/python/tsnecuda/TSNE.py:36-258 of the reference: same constructor keywords and
defaults, same validation errors, same `fit_transform(X, y=None)` contract (X -> float32
C-contiguous, result (N, 2) float32 Fortran-ordered, `y` used as the initial embedding), and the
same single ctypes symbol `pymodule_tsne` with the same 31 argument types, loaded from
`libtsnecuda` in this package's directory.
"""
import os
from collections import namedtuple
from ctypes import POINTER, c_bool, c_float, c_int

import numpy as N

_ARG_NAMES = [
    "result", "points", "dims", "perplexity", "learning_rate", "early_exaggeration", "magnitude_factor",
    "num_neighbors", "iterations", "iterations_no_progress", "force_magnify_iters", "perplexity_search_epsilon",
    "pre_exaggeration_momentum", "post_exaggeration_momentum", "theta", "epssq", "min_gradient_norm",
    "initialization_type", "preinit_data", "dump_points", "dump_file", "dump_interval", "use_interactive",
    "viz_server", "viz_timeout", "verbosity", "print_interval", "gpu_device", "return_style", "num_snapshots",
    "distance_metric",
]
TsneConfig = namedtuple("TsneConfig", _ARG_NAMES)


def _c_string(text):
    """NUL-terminated uint8 array of an ASCII string (how the reference passes file names)."""
    return N.require(N.array([ord(ch) for ch in text] + [0]), N.uint8, ["CONTIGUOUS", "ALIGNED"])


class TSNE(object):
    def __init__(self, n_components=2, perplexity=50.0, early_exaggeration=12.0, learning_rate=200.0,
                 num_neighbors=32, force_magnify_iters=250, pre_momentum=0.5, post_momentum=0.8, theta=0.5,
                 epssq=0.0025, n_iter=1000, n_iter_without_progress=1000, min_grad_norm=0.0,
                 perplexity_epsilon=1e-3, metric="euclidean", init="random", return_style="once", num_snapshots=5,
                 verbose=0, random_seed=None, use_interactive=False, viz_timeout=10000,
                 viz_server="tcp://localhost:5556", dump_points=False, dump_file="dump.txt", dump_interval=1,
                 print_interval=10, device=0, magnitude_factor=5):
        if n_components != 2:
            raise NotImplementedError("Only projection into 2 dimensions is supported.")
        self.n_components = int(n_components)
        self.perplexity = float(perplexity)
        self.early_exaggeration = float(early_exaggeration)
        self.learning_rate = float(learning_rate)
        self.n_iter = int(n_iter)
        self.n_iter_without_progress = int(n_iter_without_progress)
        self.min_grad_norm = float(min_grad_norm)
        if metric in ("euclidean", "L2"):
            self.metric = 1
        elif metric == "innerproduct":
            self.metric = 0
        else:
            raise NotImplementedError("Only the 'euclidean' ('L2') and 'innerproduct' metrics are supported.")
        if init not in ("random",):
            raise NotImplementedError("Only init='random' is supported (pass an initial embedding as fit_transform's y).")
        self.init = init
        self.verbose = int(verbose)
        self.device_id = int(device)
        self.print_interval = int(print_interval)
        self.num_neighbors = int(num_neighbors)
        self.force_magnify_iters = int(force_magnify_iters)
        self.pre_momentum = float(pre_momentum)
        self.post_momentum = float(post_momentum)
        self.theta = float(theta)
        self.epssq = float(epssq)
        self.perplexity_epsilon = float(perplexity_epsilon)
        self.magnitude_factor = float(magnitude_factor)
        self.dump_file = str(dump_file)
        self.dump_points = bool(dump_points)
        self.dump_interval = int(dump_interval)
        self.use_interactive = bool(use_interactive)
        self.viz_server = str(viz_server)
        self.viz_timeout = int(viz_timeout)
        if return_style == "once":
            self.return_style = 0
        elif return_style == "snapshots":
            self.return_style = 1
        else:
            raise ValueError("Invalid return style...")
        self.num_snapshots = int(num_snapshots)

        self._path = os.path.dirname(os.path.abspath(__file__))
        self._lib = N.ctypeslib.load_library("libtsnecuda", self._path)
        self._lib.pymodule_tsne.restype = None
        f32 = N.float32
        self._lib.pymodule_tsne.argtypes = list(TsneConfig(
            result=N.ctypeslib.ndpointer(f32, ndim=2, flags="ALIGNED, F_CONTIGUOUS, WRITEABLE"),
            points=N.ctypeslib.ndpointer(f32, ndim=2, flags="ALIGNED, CONTIGUOUS"),
            dims=POINTER(N.ctypeslib.c_intp),
            perplexity=c_float, learning_rate=c_float, early_exaggeration=c_float, magnitude_factor=c_float,
            num_neighbors=c_int, iterations=c_int, iterations_no_progress=c_int, force_magnify_iters=c_int,
            perplexity_search_epsilon=c_float, pre_exaggeration_momentum=c_float, post_exaggeration_momentum=c_float,
            theta=c_float, epssq=c_float, min_gradient_norm=c_float, initialization_type=c_int,
            preinit_data=N.ctypeslib.ndpointer(f32, ndim=2, flags="ALIGNED, F_CONTIGUOUS"),
            dump_points=c_bool, dump_file=N.ctypeslib.ndpointer(N.uint8, flags="ALIGNED, CONTIGUOUS"),
            dump_interval=c_int, use_interactive=c_bool,
            viz_server=N.ctypeslib.ndpointer(N.uint8, flags="ALIGNED, CONTIGUOUS"), viz_timeout=c_int,
            verbosity=c_int, print_interval=c_int, gpu_device=c_int, return_style=c_int, num_snapshots=c_int,
            distance_metric=c_int))

    def fit_transform(self, X, y=None):
        """Embed X (n_points, n_dims); `y` (n_points, 2), if given, is the initial embedding."""
        self.points = N.require(X, N.float32, ["CONTIGUOUS", "ALIGNED"])
        blocks = self.num_snapshots if self.return_style == 1 else 1
        # One (N,2) Fortran-ordered block per returned embedding.  (The reference allocates a single
        # block even for snapshots and lets the library write past it.)
        out = N.zeros((self.points.shape[0], self.n_components * blocks), N.float32, order="F")
        self.embedding = N.require(out, N.float32, ["F_CONTIGUOUS", "ALIGNED", "WRITEABLE"])
        if y is None:
            self.initialization_type = 1
            self.preinit_data = N.require(N.zeros((1, 1)), N.float32, ["F_CONTIGUOUS", "ALIGNED"])
        else:
            self.initialization_type = 3
            self.preinit_data = N.require(y, N.float32, ["F_CONTIGUOUS", "ALIGNED"])
        self.dump_file_ = _c_string(self.dump_file)
        self.viz_server_ = _c_string(self.viz_server)
        self._lib.pymodule_tsne(*self._construct_tsne_args(self.embedding, self.points))
        if blocks > 1:
            return N.stack([self.embedding[:, 2 * b:2 * b + 2] for b in range(blocks)])
        return self.embedding

    def _construct_tsne_args(self, result_array, input_array):
        return TsneConfig(
            result=result_array, points=input_array, dims=input_array.ctypes.shape, perplexity=self.perplexity,
            learning_rate=self.learning_rate, early_exaggeration=self.early_exaggeration,
            magnitude_factor=self.magnitude_factor, num_neighbors=self.num_neighbors, iterations=self.n_iter,
            iterations_no_progress=self.n_iter_without_progress, force_magnify_iters=self.force_magnify_iters,
            perplexity_search_epsilon=self.perplexity_epsilon, pre_exaggeration_momentum=self.pre_momentum,
            post_exaggeration_momentum=self.post_momentum, theta=self.theta, epssq=self.epssq,
            min_gradient_norm=self.min_grad_norm, initialization_type=self.initialization_type,
            preinit_data=self.preinit_data, dump_points=self.dump_points, dump_file=self.dump_file_,
            dump_interval=self.dump_interval, use_interactive=self.use_interactive, viz_server=self.viz_server_,
            viz_timeout=self.viz_timeout, verbosity=self.verbose, print_interval=self.print_interval,
            gpu_device=self.device_id, return_style=self.return_style, num_snapshots=self.num_snapshots,
            distance_metric=self.metric)
