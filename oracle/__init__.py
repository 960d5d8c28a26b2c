"""CPU oracle for the chunked delta-rule backward (DeltaNet, GDN, KDA, GDN2).

TEST INFRASTRUCTURE ONLY.  Nothing in ``rewy_b200`` imports this package; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py`` as the checker / baseline, never as the product path.

Parity pin: the functions here are checked (tests/test_oracle.py) against
  * gradients produced by the reference's own FP64 token recurrence
    (src/fast_delta_rule/validation.py:23-38) run in the build container and
    committed as tests/golden/recurrence_*.npz,
  * the reference's closed-form chunk backward
    (benchmarks/plotting/check_manuscript_math.py:21-54) on its own seed, committed
    as tests/golden/closed_form_seed79.npz,
  * the reference's matrix-intra FP64 oracle
    (scripts/npu950_intra_regression.py:25-46) on the reference's captured
    fixtures validation/npu950_intra/{kda,gdn2}.npz.
"""
from .recurrence import recurrence, recurrence_grads
from .chunked import chunk_forward, chunk_backward, FAMILIES
from .matrix_intra import matrix_intra_pairwise, matrix_intra_centered
from .naive_chunk import naive_chunk_forward, naive_chunk_backward_fp32

__all__ = [
    "recurrence", "recurrence_grads", "chunk_forward", "chunk_backward", "FAMILIES",
    "matrix_intra_pairwise", "matrix_intra_centered",
    "naive_chunk_forward", "naive_chunk_backward_fp32",
]
