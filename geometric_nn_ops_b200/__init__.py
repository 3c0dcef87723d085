"""B200-native triangle attention and triangle multiplicative update.

Public API: :mod:`geometric_nn_ops_b200.triangle`.  All arithmetic runs in the
in-tree CUDA library ``libtri_b200.so`` (see ``include/tri_b200.h``).
"""

from . import _precision, triangle  # noqa: F401

__version__ = "0.1.0"
