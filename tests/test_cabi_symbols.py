"""The shared library loads on a machine without a GPU and exports every function that
include/lrqk_sm100.h declares; compute entries refuse to run without an sm_100 device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "lrqk_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lrqk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from lrqk_b200 import _lib
    names = _declared()
    assert len(names) >= 20
    handle = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert sorted(_lib.exported_names()) == names, "ctypes binding and header disagree"
    lib = _lib.lib()
    assert lib.lrqk_version().startswith(b"lrqk_sm100")
    assert lib.lrqk_strerror(_lib.ENODEVICE) and lib.lrqk_strerror(-99)


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from lrqk_b200 import _lib
    lib = _lib.lib()
    assert lib.lrqk_device_supported() == 0
    layer = _lib.Layer()
    assert lib.lrqk_score_topk(C.byref(layer), None, 10, None, None, 0, None, 0, None) == _lib.ENODEVICE
    assert lib.lrqk_layer_step(None, None, None) == _lib.EINVAL
    from lrqk_b200 import LightAttentionIndicesFactory
    fac = LightAttentionIndicesFactory(num_lite_tokens=4, attn_topk=8, r=8)
    with pytest.raises((RuntimeError, AssertionError)):
        fac.prefill(torch.zeros(1, 1, 64, 128), torch.zeros(1, 1, 64, 128), torch.zeros(1, 1, 64, 128))


def test_host_containers_match_reference_growth_rule():
    # lrqk_attention_test.py:8-66 (append / getitem / growth) on the CPU containers
    import random
    import torch
    from lrqk_b200 import AutoIncreaseTensor, PreAllocatedTensor
    random.seed(0)
    ait = AutoIncreaseTensor(capacity=16, dim=0)
    target = torch.randn(512, 128)
    ll = 0
    while ll < 512:
        rr = min(ll + random.randint(1, 16), 512)
        ait.append(target[ll:rr])
        ll = rr
        s = random.randint(1, rr - 1) if rr > 1 else 0
        assert len(ait) == rr and torch.equal(ait[:s], target[:s]) and torch.equal(ait[s], target[s])
    assert not ait.data[len(ait):].any()                      # new space is zeroed
    a2 = AutoIncreaseTensor(capacity=16, dim=2)
    t4 = torch.randn(2, 8, 200, 16)
    a2.append(t4[:, :, :128])
    assert a2.capacity == max(16, int(128 * 1.5))             # first allocation rule
    for i in range(128, 200):
        a2.append(t4[:, :, i:i + 1])
        assert torch.equal(a2[:, :, :i + 1], t4[:, :, :i + 1])
    p = PreAllocatedTensor(8, 0)
    p.append(torch.ones(5, 2))
    with pytest.raises(ValueError):
        p.append(torch.ones(4, 2))
