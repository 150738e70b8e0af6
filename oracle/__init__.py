"""CPU oracle for the FIt-SNE hot path: test infrastructure only.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs may import this
package.  `oracle.cpu` wraps the OpenMP C restatement, `oracle.np64` is a float64 NumPy restatement
used to cross-check it, `oracle.ref` loads the reference's own CUDA build when it is present.
"""
