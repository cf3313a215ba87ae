"""The Python surface mirrors the reference's: class names, constructor arguments in the reference's order and
with its defaults (lrqk_attention.py:1031-1046 for the per-layer factory, :1785-1798 for the cache -- the two
differ on purpose there: tol 1e-4 vs 1e-2, attn_topk 128 vs num_active_tokens 512, one lite token vs 16), the
growth containers, the throughput table's rows.  Import-only: no GPU is touched."""
import inspect

import pytest

import lrqk_b200
from lrqk_b200 import (DynamicLRQKCache, InitAQAK, LightAttentionIndicesFactory, LightAttentionIndicesNoHitMiss)
from lrqk_b200.extras import task_dict


def _defaults(fn):
    return {k: v.default for k, v in inspect.signature(fn).parameters.items() if k != "self"}


def test_factory_constructor_matches_the_reference():
    d = _defaults(LightAttentionIndicesFactory.__init__)
    assert list(d) == ["num_lite_tokens", "attn_topk", "num_key_value_groups", "r", "max_iter", "tol", "weights",
                       "capacity", "init_aq_ak_method", "scaling_ratio", "device", "dtype"]
    assert (d["num_lite_tokens"], d["attn_topk"], d["num_key_value_groups"], d["r"], d["max_iter"], d["tol"]) == \
        (1, 128, 1, 16, 2, 1e-4)
    assert d["weights"] == (1.0, 1.0, 1.0, 1.0) and d["capacity"] == 4096 and d["scaling_ratio"] == 1.5
    assert d["init_aq_ak_method"] == InitAQAK.randn and d["device"] is None and d["dtype"] is None


def test_cache_constructor_matches_the_reference():
    d = _defaults(DynamicLRQKCache.__init__)
    assert list(d) == ["r", "num_active_tokens", "lambda_Q", "lambda_K", "max_iter", "lite_tokens", "tol",
                       "max_sequence_length", "num_key_value_groups", "lwattn_factory", "init_aq_ak_method"]
    assert (d["r"], d["num_active_tokens"], d["lambda_Q"], d["lambda_K"], d["max_iter"], d["lite_tokens"], d["tol"],
            d["max_sequence_length"], d["num_key_value_groups"]) == (16, 512, 1.0, 1.0, 2, 16, 1e-2, 4096, 1)
    assert d["lwattn_factory"] is LightAttentionIndicesFactory and d["init_aq_ak_method"] == InitAQAK.randn


def test_weights_argument_like_the_reference():
    f = LightAttentionIndicesFactory(weights=2.0)                    # a float means all four (:1066-1067)
    assert f.weights == (2.0, 2.0, 2.0, 2.0)
    assert LightAttentionIndicesFactory(weights=(0.5, 1.0, 2.0, 1.0)).weights == (0.5, 1.0, 2.0, 1.0)
    with pytest.raises(ValueError):
        LightAttentionIndicesFactory(weights=[1.0, 1.0, 1.0, 1.0])   # neither float nor tuple (:1072)
    with pytest.raises(ValueError):
        LightAttentionIndicesFactory(weights=(1.0, 1.0, 1.0))
    with pytest.raises(ValueError):
        LightAttentionIndicesFactory(weights=(1.0, -1.0, 1.0, 1.0))  # (a negative weight loses positive definiteness)


def test_init_methods_and_pairs():
    assert {m.name for m in InitAQAK} == {"randn", "top", "topcol"}
    f = LightAttentionIndicesFactory(max_iter=3, tol=1e-3)
    assert f.max_iter == (3, 3) and f.tol == (1e-3, 1e-3)            # _ensure_tuple2, :1057-1058
    f = LightAttentionIndicesFactory(max_iter=(1, 4), tol=(1e-2, 1e-5), num_lite_tokens=8, attn_topk=64)
    assert f.max_iter == (1, 4) and f.tol == (1e-2, 1e-5) and f.gpu_capacity == 72
    assert len(f) == 0 and f.lite_indices == [-1] * 8


def test_decode_before_prefill_is_an_error_not_a_fallback():
    f = LightAttentionIndicesFactory()
    with pytest.raises(RuntimeError):
        f.decode(None, None, None)
    c = DynamicLRQKCache()
    with pytest.raises(NotImplementedError):
        c[0]                                                          # no indexing, as in the reference (:1834-1839)


def test_throughput_table_rows_and_exports():
    assert list(task_dict) == ["lrqk_default", "lrqk_offload", "lrqk_no_hitmiss", "gpu_only", "cpu_offload"]
    assert issubclass(LightAttentionIndicesNoHitMiss, LightAttentionIndicesFactory)
    for name in ("AutoIncreaseTensor", "AutoIncreaseTensorSharedKV", "PreAllocatedTensor", "repeat_kv", "FullOffloadCache",
                 "HitRateCounter", "LightAttentionIndicesOffloadPrefill", "WrapForwardTimer", "load_model", "load_model_hack",
                 "load_lrqk_model", "load_tokenizer", "cast_lrqk_decode", "cast_lrqk_prefill", "tps_estimate", "run_task"):
        assert hasattr(lrqk_b200, name), name
