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
    cast_lrqk_decode,
    cast_lrqk_prefill,
    repeat_kv,
)

from .hf_models import (  # noqa: F401,E402
    load_lrqk_model,
    load_model,
    load_model_hack,
    load_tokenizer,
    lrqk_attention_forward,
    lrqk_decoder_layer_forward,
    patch_model,
)

from .extras import (  # noqa: F401,E402
    FullOffloadCache,
    HitRateCounter,
    LightAttentionIndicesOffloadPrefill,
    WrapForwardTimer,
    run_task,
    tps_estimate,
)

__all__ = [
    "FullOffloadCache", "HitRateCounter", "LightAttentionIndicesOffloadPrefill", "WrapForwardTimer", "run_task",
    "tps_estimate",
    "load_lrqk_model", "load_model", "load_model_hack", "load_tokenizer", "lrqk_attention_forward", "lrqk_decoder_layer_forward", "patch_model",
    "AutoIncreaseTensor", "AutoIncreaseTensorSharedKV", "DynamicLRQKCache", "InitAQAK",
    "LightAttentionIndicesFactory", "LightAttentionIndicesNoHitMiss", "PreAllocatedTensor", "cast_lrqk_decode", "cast_lrqk_prefill", "repeat_kv",
]
