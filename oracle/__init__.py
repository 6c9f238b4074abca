"""CPU oracle for the tensor-permutation path (test infrastructure, not product code).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package.  See oracle/host_transpose.c for the statement of the algorithm and the
reference lines it follows.
"""
from .oracle import (  # noqa: F401
    build,
    load,
    transpose_numpy,
    transpose_formula,
    transpose_blocked,
    source_index_formula_py,
    index_pattern,
    num_threads,
    use_all_cores,
)
