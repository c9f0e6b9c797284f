"""Drop-in import name of the reference package: ``import onebit_sparse_mul`` keeps working and
resolves to the B200 implementation in ``onebitsparsemul_b200`` (same names as the reference's
onebit_sparse_mul/__init__.py:6-145)."""
from onebitsparsemul_b200 import *  # noqa: F401,F403
from onebitsparsemul_b200 import __all__  # noqa: F401
