"""Key-mask sentinel and bool-mask -> additive-bias helper.

Same values as ``geometric_nn_ops_torch/triangle/_masking.py:13-42``.  The CUDA
kernels take the bool mask directly and form the bias on the fly; these helpers
exist for callers (and the cuequivariance shim) that import them.
"""

import torch


def mask_val(dtype: torch.dtype) -> float:
    if dtype == torch.float64:
        return 1e18
    if dtype in (torch.float32, torch.bfloat16):
        return 1e9
    if dtype == torch.float16:
        return torch.finfo(dtype).max / 2
    raise ValueError(f"Unsupported dtype {dtype}")


def masked_key_bias(mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    # val * (float(mask) - 1): +0.0 on kept keys (not -0.0), -val on masked ones.
    return mask_val(dtype) * (mask.to(torch.float32) - 1)
