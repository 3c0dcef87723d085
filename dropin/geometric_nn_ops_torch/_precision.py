"""``geometric_nn_ops_torch._precision`` as importers of the reference see it (the cuequivariance shim reads
``torch_precision()`` and ``IEEE`` from here): the B200 library's precision module under the reference's name."""

from geometric_nn_ops_b200._precision import IEEE, TF32, matmul_precision, torch_precision

__all__ = ["IEEE", "TF32", "matmul_precision", "torch_precision"]
