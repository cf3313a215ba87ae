"""lrqk_b200 -- the LRQK decode-time selection and attention path as sm_100a CUDA kernels.

The public names mirror the reference's ``lrqk_attention`` module; see
``lrqk_b200/lrqk_attention.py``.  The compute library ``liblrqk_sm100.so`` is built in-tree by
``python -m lrqk_b200.build``; importing this package does not require a GPU, using it does.
"""
from .lrqk_attention import (  # noqa: F401
    AutoIncreaseTensor,
    AutoIncreaseTensorSharedKV,
    DynamicLRQKCache,
    InitAQAK,
    LightAttentionIndicesFactory,
    LightAttentionIndicesNoHitMiss,
    PreAllocatedTensor,
    repeat_kv,
)

__all__ = [
    "AutoIncreaseTensor", "AutoIncreaseTensorSharedKV", "DynamicLRQKCache", "InitAQAK",
    "LightAttentionIndicesFactory", "LightAttentionIndicesNoHitMiss", "PreAllocatedTensor", "repeat_kv",
]
