"""fp32 matmul precision, read from torch's global setting at call time.

Mirrors ``geometric_nn_ops_torch/_precision.py:34-44,74-83`` of the reference:
``"tf32"`` only when ``torch.backends.cuda.matmul.fp32_precision == "tf32"`` (or the
legacy ``allow_tf32`` on torch builds without that attribute); 16-bit operands are
pinned to ``"ieee"`` because the setting cannot change them.
"""

import torch

IEEE = "ieee"
TF32 = "tf32"


def torch_precision() -> str:
    matmul = torch.backends.cuda.matmul
    if hasattr(matmul, "fp32_precision"):
        return TF32 if matmul.fp32_precision == TF32 else IEEE
    return TF32 if matmul.allow_tf32 else IEEE


def matmul_precision(*, fp32_operands: bool) -> str:
    if not fp32_operands:
        return IEEE
    return torch_precision()
