"""CPU oracle for the k-means path.  TEST INFRASTRUCTURE, not product code.

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; the shipped engine (``h2o4gpu_b200``) never does and
has no CPU fallback.

Contents
--------
``sklearn_oracle``  the reference's CPU path itself: ``h2o4gpu.KMeans(n_gpus=0)``
                    resolves to scikit-learn's Lloyd solver
                    (src/interface_py/h2o4gpu/solvers/kmeans.py:539-541, 738-750,
                    768-770), so the oracle calls ``sklearn.cluster.KMeans`` with
                    the keyword arguments that wrapper forwards.
``lloyd``           a numpy restatement of that solver (one Lloyd step at a time,
                    any float dtype) used for teacher-forced per-step parity and
                    for the conventions of the GPU reference's ABI (squared,
                    column-major transform).
``lloyd_ref.c``     the same step in plain C with fp64 accumulation, built by
                    ``oracle/Makefile`` into ``oracle/_build/``.

Parity pin: the reference holds no numeric k-means test at the Python boundary
(tests/python/open_data/kmeans/test_kmeans.py is named by Makefile:503 but is
absent from the checkout).  The restatement is pinned (a) against the literal
arrays of the reference's kernel tests (tests/cpp/gpu/kmeans/*.cu) and the
README example (README.md:115-133), and (b) against scikit-learn itself, the
library the reference's CPU path runs, through fixtures under tests/golden/.
scikit-learn is a third-party dependency of the reference (pinned 1.3.2 in
src/interface_py/requirements_buildonly.txt:17-18); the copy importable here is
1.9.0, the same chunked dense Lloyd algorithm.
"""
