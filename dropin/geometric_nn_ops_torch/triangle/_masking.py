"""``geometric_nn_ops_torch.triangle._masking`` for importers that use the key-mask helpers."""

from geometric_nn_ops_b200.triangle._masking import mask_val, masked_key_bias

__all__ = ["mask_val", "masked_key_bias"]
