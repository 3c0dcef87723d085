"""Drop-in ``geometric_nn_ops_torch`` namespace served by the B200 library.

Put this directory's parent (``dropin/``) ahead of the reference package on ``sys.path`` (or install it in its
place) and every importer of the reference -- user code, and the unmodified ``cuequivariance_ops_torch`` shim,
which imports ``geometric_nn_ops_torch.triangle.{triangle_attention, triangle_multiplicative_update,
attention_pair_bias}`` and ``geometric_nn_ops_torch._precision`` -- lands in ``geometric_nn_ops_b200``.
Only the public surface is provided: the reference's private ``_kernels`` / ``_reference`` packages have no
counterpart here.
"""

import os
import sys

try:
    import geometric_nn_ops_b200  # noqa: F401
except ImportError:  # running from a source checkout: the library sits two directories up
    _root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if _root not in sys.path:
        sys.path.append(_root)
    import geometric_nn_ops_b200  # noqa: F401

from . import _precision, triangle  # noqa: E402,F401
