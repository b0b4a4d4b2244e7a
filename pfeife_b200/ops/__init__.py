"""Differentiable ops on the sm_100a kernels (see functional.py) and raw kernel wrappers
(kernels.py)."""
from .functional import (  # noqa: F401
    ParamSlot, attention, conv2d, group_norm, upsample_nearest2x, attention_qkv, compute_dtype, cross_entropy, embedding, geglu, gelu, layer_norm, linear, mlp,
    mse_loss, register_param, rms_norm, rope, rope_tables, silu, swiglu, unregister_params,
)
