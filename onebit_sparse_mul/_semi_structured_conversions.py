"""Drop-in module name of the reference's onebit_sparse_mul/_semi_structured_conversions.py."""
from onebitsparsemul_b200._semi_structured_conversions import (  # noqa: F401
    mask_creator, sparse_semi_structured_from_dense_cutlass, sparse_semi_structured_to_dense_cutlass)
