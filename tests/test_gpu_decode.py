"""Parity of the CUDA decode-path kernels (called through the C ABI) with the CPU oracle.

Tolerances: integer outputs (selected positions, slot table, masks, gathered rows) must be
bit-exact.  Proxy scores are fp32 in either dtype: within 1e-5 (fp32 operands) / 1e-3 (bf16 operands)
of the oracle's, relative to the largest magnitude of the tensor, and bit-exact against the oracle's
emulation of the kernel's summation order.  Results that are STORED in bf16 (attention rows, projected
query / key, right factors) are held to the fp32 tolerance of the same quantity -- 1e-5 for attention,
2e-4 for the r x r solves, whose round-off the solves amplify -- plus one rounding of the element to
bf16 (``gpu_util.bf16_excess``): a bound of 1e-3 of the largest magnitude cannot hold for a stored bf16
value, whose rounding alone is up to 2^-9 = 1.95e-3 of it.
"""
import json
import os

import numpy as np
import pytest
import torch

import lrqk_oracle as orc
from gpu_util import bf16_excess

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _state(**kw):
    from lrqk_b200.state import LayerState
    return LayerState(**kw)


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


# --------------------------------------------------------------------------------------------
# score + top-k
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,r,bsz,hq,cand,k", [
    (torch.bfloat16, 32, 1, 8, 20000, 512),
    (torch.bfloat16, 32, 2, 4, 4099, 2048),     # k close to the candidate count, ragged length
    (torch.bfloat16, 16, 1, 3, 70001, 1024),    # several CTAs per head needed for the keys to fit
    (torch.bfloat16, 64, 1, 2, 9000, 64),
    (torch.bfloat16, 8, 1, 2, 5000, 100),       # 16-byte rows
    (torch.float32, 16, 1, 8, 4079, 256),       # BASELINE config 0 shape
    (torch.float32, 8, 2, 4, 635, 64),
    (torch.float32, 64, 1, 2, 3000, 17),
])
def test_score_topk_matches_oracle(dtype, r, bsz, hq, cand, k):
    g = torch.Generator().manual_seed(cand + r)
    cap = cand + 37
    A = torch.randn(bsz, hq, cap, r, generator=g).to(dtype)
    qh = torch.randn(bsz, hq, r, generator=g).to(dtype)
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hq, head_dim=128, r=r, k=k, m=4, a_capacity=cap,
                host_capacity=16, dtype=dtype, with_host=False)
    st.A_K.copy_(A)
    scores = torch.full((bsz, hq, cand), float("nan"), device="cuda")
    wanted = st.score_topk(qh.cuda(), cand, scores_out=scores).cpu().numpy()
    scores = scores.cpu()
    ref = orc.proxy_scores(A[:, :, :cand], qh[:, :, None, :])
    tol = 1e-5 if dtype == torch.float32 else 1e-3
    assert _rel(scores, ref) < tol
    # identical fp32 scores -> identical selection, ties to the lower position
    assert np.array_equal(wanted, orc.topk_sorted(scores, k))
    if dtype == torch.bfloat16:
        lanes = max(1, r * 2 // 64)
        canon = orc.proxy_scores_lane_order(A[:, :, :cand], qh[:, :, None, :], lanes)
        assert np.array_equal(scores.numpy().view(np.uint32), canon.view(np.uint32)), "summation order drifted"


@pytest.mark.parametrize("r,hq,cand,k", [(32, 2, 131007, 2048), (16, 2, 70001, 1024), (64, 2, 9000, 64), (32, 4, 20000, 512)])
def test_score_topk_one_and_two_kernel_plans_agree(r, hq, cand, k):
    """With few heads the keys are formed by a separate all-SM kernel into a workspace (the state sizes one
    when that plan applies); without a workspace the clusters score their own segments.  Same scores, same
    selection, bit for bit."""
    g = torch.Generator().manual_seed(cand)
    st = _state(bsz=1, q_heads=hq, kv_heads=hq, head_dim=128, r=r, k=k, m=4, a_capacity=cand + 5,
                host_capacity=16, dtype=torch.bfloat16, with_host=False)
    assert st.score_ws is not None, "this shape is meant to take the two-kernel plan"
    st.A_K.copy_(torch.randn(1, hq, cand + 5, r, generator=g).to(torch.bfloat16))
    st.A_K[:, 0].copy_((st.A_K[:, 0].float() * 2).round() / 2)            # a head with ties at the cut
    qh = torch.randn(1, hq, r, generator=g).to(torch.bfloat16).cuda()
    s2 = torch.full((1, hq, cand), float("nan"), device="cuda")
    two = st.score_topk(qh, cand, scores_out=s2).clone()
    ws, st.score_ws = st.score_ws, None
    s1 = torch.full((1, hq, cand), float("nan"), device="cuda")
    one = st.score_topk(qh, cand, scores_out=s1).clone()
    st.score_ws = ws
    assert torch.equal(s1.view(torch.int32), s2.view(torch.int32)) and torch.equal(one, two)
    assert np.array_equal(two.cpu().numpy(), orc.topk_sorted(s2.cpu(), k))


def test_score_topk_heavy_ties():
    # scores restricted to a handful of values: the tie rule decides almost every pick
    g = torch.Generator().manual_seed(5)
    bsz, hq, r, cand, k = 1, 4, 32, 30011, 1000
    A = torch.zeros(bsz, hq, cand, r)
    A[..., 0] = torch.randint(-3, 4, (bsz, hq, cand), generator=g).float()
    A[0, 0, :, 0] = 1.0                          # one head with every score equal
    A[0, 1, ::2, 0] = -0.0                       # signed zeros compare equal
    A[0, 1, 1::2, 0] = 0.0
    qh = torch.zeros(bsz, hq, r)
    qh[..., 0] = 1.0
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hq, head_dim=128, r=r, k=k, m=4, a_capacity=cand,
                host_capacity=16, dtype=torch.bfloat16, with_host=False)
    st.A_K.copy_(A.to(torch.bfloat16))
    scores = torch.zeros((bsz, hq, cand), device="cuda")
    wanted = st.score_topk(qh.to(torch.bfloat16).cuda(), cand, scores_out=scores).cpu().numpy()
    assert np.array_equal(wanted, orc.topk_sorted(scores.cpu(), k))
    assert wanted[0, 0].tolist() == list(range(k))
    assert wanted[0, 1].tolist() == list(range(k))


def test_score_topk_rejects_bad_arguments():
    from lrqk_b200._lib import LrqkError
    st = _state(bsz=1, q_heads=2, kv_heads=2, head_dim=128, r=16, k=64, m=4, a_capacity=1000,
                host_capacity=16, dtype=torch.bfloat16, with_host=False)
    qh = torch.zeros(1, 2, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(LrqkError):
        st.score_topk(qh, 64)          # not more candidates than k
    with pytest.raises(LrqkError):
        st.score_topk(qh, 1001)        # beyond the capacity


# --------------------------------------------------------------------------------------------
# hit/miss difference and the miss fetch
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("k,l,heads", [(5, 8, 1), (64, 100, 6), (257, 300, 3), (2048, 30000, 8), (4096, 4096, 2)])
def test_slot_diff_matches_oracle(k, l, heads):
    rng = np.random.default_rng(k)
    if k == 5:
        now = np.array([[0, 1, 2, 6, 7]], dtype=np.int32)     # the reference's docstring example
        new = np.array([[0, 2, 4, 5, 6]], dtype=np.int32)
    else:
        now = np.stack([rng.permutation(l)[:k] for _ in range(heads)]).astype(np.int32)
        new = np.stack([np.sort(rng.permutation(l)[:k]) for _ in range(heads)]).astype(np.int32)
        if heads > 1:
            new[1] = np.sort(now[1])                              # a head with no miss at all
    st = _state(bsz=1, q_heads=heads, kv_heads=heads, head_dim=128, r=16, k=k, m=4, a_capacity=64,
                host_capacity=16, dtype=torch.bfloat16, with_host=False)
    st.table.copy_(torch.from_numpy(now).view(1, heads, k))
    st.slot_diff(torch.from_numpy(new).view(1, heads, k).cuda())
    upd, mask, cnt = orc.slot_diff(now, new)
    assert np.array_equal(st.table.cpu().numpy()[0], upd)
    assert np.array_equal(st.mask.cpu().numpy()[0], mask)
    assert np.array_equal(st.miss_count.cpu().numpy()[0], cnt)
    counters = st.counters.cpu().numpy()
    assert counters[0] == cnt.sum() and counters[1] == 0
    lst = st.miss_list.cpu().numpy()[:counters[0]]
    want = sorted((h, s, int(upd[h, s])) for h in range(heads) for s in range(k) if mask[h, s])
    assert sorted(map(tuple, lst.tolist())) == want
    if k == 5:
        assert upd.tolist() == [[0, 4, 2, 6, 5]] and mask.tolist() == [[0, 1, 0, 0, 1]]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_miss_gather_fills_exactly_the_missed_slots(dtype):
    g = torch.Generator().manual_seed(9)
    bsz, hq, hkv, d, k, m, cap = 2, 8, 2, 128, 96, 4, 700
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hkv, head_dim=d, r=16, k=k, m=m, a_capacity=64,
                host_capacity=cap, dtype=dtype)
    st.host.data.copy_(torch.randn(bsz, hkv, cap, 2 * d, generator=g).to(dtype))
    rng = np.random.default_rng(3)
    now = np.stack([rng.permutation(600)[:k] for _ in range(bsz * hq)]).astype(np.int32).reshape(bsz, hq, k)
    new = np.sort(np.stack([rng.permutation(600)[:k] for _ in range(bsz * hq)]), axis=-1).astype(np.int32).reshape(bsz, hq, k)
    st.table.copy_(torch.from_numpy(now))
    K0 = torch.randn(bsz, hq, k + m, d, generator=g).to(dtype)
    V0 = torch.randn(bsz, hq, k + m, d, generator=g).to(dtype)
    st.K_res.copy_(K0)
    st.V_res.copy_(V0)
    st.slot_diff(torch.from_numpy(new).cuda())
    st.miss_gather()
    torch.cuda.synchronize()
    upd, mask, _ = orc.slot_diff(now, new)
    rows = orc.miss_rows(upd, mask, hkv, hq // hkv, cap)
    fetched = st.host.data.view(-1, 2 * d)[torch.from_numpy(rows)]
    Kexp, Vexp = K0.clone(), V0.clone()
    bm = torch.from_numpy(mask.astype(bool))
    Kexp[:, :, :k][bm] = fetched[:, :d]
    Vexp[:, :, :k][bm] = fetched[:, d:]
    assert torch.equal(st.K_res.cpu(), Kexp) and torch.equal(st.V_res.cpu(), Vexp)
    st.close()


def test_native_gather_entry_points():
    import ctypes as C
    from lrqk_b200 import _lib
    from lrqk_b200.state import HostStore
    lib = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(11)
    # d0_indices_select against index_select (cpp_kernel/main_test.py:11-23), source in pinned host memory
    hs = HostStore(1, 1, 64000, 96, torch.float32)          # rows of 192 floats
    src = hs.data.view(64000, 192)
    src.copy_(torch.from_numpy(rng.standard_normal((64000, 192)).astype(np.float32)))
    for n in (1, 37, 512):
        rows = torch.from_numpy(rng.integers(0, 64000, n))
        dst = torch.empty(n, 192, device="cuda")
        _lib.check(lib.lrqk_d0_indices_select(C.c_void_p(dst.data_ptr()), C.c_void_p(hs.device_ptr),
                                              C.c_void_p(rows.cuda().data_ptr()), n, 192 * 4, 64000, stream), "select")
        assert torch.equal(dst.cpu(), src[rows])
    _lib.check(lib.lrqk_d0_indices_select(None, None, None, 0, 768, 64000, stream), "empty select")
    # take_along_dim_with_mask invariants (cpp_kernel/main_demo.py:150-196)
    b, h, grp, s, w, k = 2, 8, 4, 32, 64, 8
    srcm = rng.standard_normal((b, h, s, w)).astype(np.float16)
    idx = np.stack([rng.permutation(s)[:k] for _ in range(b * h * grp)]).reshape(b, h, grp, k).astype(np.int64)
    mask = rng.random((b, h, grp, k)) < 0.4
    exp = orc.take_along_dim_with_mask(srcm, idx, mask)
    d_src = torch.from_numpy(srcm).cuda()
    d_idx, d_mask = torch.from_numpy(idx).cuda(), torch.from_numpy(mask.astype(np.uint8)).cuda()
    dst = torch.zeros(b * h * grp * k, w, dtype=torch.float16, device="cuda")
    n_out = torch.zeros(1, dtype=torch.int64, device="cuda")
    ws = torch.zeros(lib.lrqk_take_along_dim_with_mask_workspace_bytes(b, h, grp, k), dtype=torch.uint8, device="cuda")
    _lib.check(lib.lrqk_take_along_dim_with_mask(
        C.c_void_p(dst.data_ptr()), C.c_void_p(d_src.data_ptr()), C.c_void_p(d_idx.data_ptr()),
        C.c_void_p(d_mask.data_ptr()), b, h, s, grp, k, w * 2, C.c_void_p(n_out.data_ptr()),
        C.c_void_p(ws.data_ptr()), stream), "masked gather")
    n = int(n_out.item())
    assert n == exp.shape[0] and np.array_equal(dst[:n].cpu().numpy(), exp)
    hs.close()


# --------------------------------------------------------------------------------------------
# lite ring, projection/update, attention
# --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_lite_append_and_flush(dtype):
    g = torch.Generator().manual_seed(2)
    bsz, hq, hkv, d, k, m, cap = 2, 8, 2, 128, 16, 4, 64
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hkv, head_dim=d, r=16, k=k, m=m, a_capacity=64,
                host_capacity=cap, dtype=dtype)
    K0 = torch.randn(bsz, hq, k + m, d, generator=g).to(dtype)
    st.K_res.copy_(K0)
    st.V_res.copy_(K0 * 2)
    grp = hq // hkv
    rows = []
    for slot in range(m):
        kn = torch.randn(bsz, hkv, d, generator=g).to(dtype)
        vn = torch.randn(bsz, hkv, d, generator=g).to(dtype)
        rows.append(torch.cat([kn, vn], dim=-1))
        flush = m if slot == m - 1 else 0
        st.lite_append(kn.cuda(), vn.cuda(), slot, 100 + slot, flush, 10)
        Kc = st.K_res.cpu()
        assert torch.equal(Kc[:, :, k + slot], kn.repeat_interleave(grp, dim=1))
        assert torch.equal(st.V_res.cpu()[:, :, k + slot], vn.repeat_interleave(grp, dim=1))
        assert torch.equal(Kc[:, :, :k], K0[:, :, :k])
    torch.cuda.synchronize()
    assert st.lite_pos.cpu().tolist() == [100, 101, 102, 103]
    assert torch.equal(st.host.data[:, :, 10:10 + m], torch.stack(rows, dim=2))
    assert not st.host.data[:, :, :10].any() and not st.host.data[:, :, 10 + m:].any()
    st.close()


@pytest.mark.parametrize("dtype,d,rows,bsz,hq", [
    (torch.bfloat16, 128, 2112, 1, 32), (torch.bfloat16, 128, 272, 2, 8), (torch.float32, 128, 272, 1, 8),
    (torch.bfloat16, 64, 100, 1, 3), (torch.float32, 64, 33, 2, 2), (torch.bfloat16, 128, 5, 1, 2),
    (torch.bfloat16, 128, 9000, 1, 2), (torch.float32, 128, 5000, 1, 1),   # more rows than 64 splits of one staging round
])
def test_flash_decode_matches_oracle(dtype, d, rows, bsz, hq):
    g = torch.Generator().manual_seed(rows)
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hq, head_dim=d, r=16, k=rows - 4, m=4, a_capacity=64,
                host_capacity=16, dtype=dtype, with_host=False) if rows > 4 else \
        _state(bsz=bsz, q_heads=hq, kv_heads=hq, head_dim=d, r=16, k=1, m=4, a_capacity=64,
               host_capacity=16, dtype=dtype, with_host=False)
    K = (torch.randn(bsz, hq, st.k + st.m, d, generator=g) * 2).to(dtype)
    V = torch.randn(bsz, hq, st.k + st.m, d, generator=g).to(dtype)
    q = torch.randn(bsz, hq, d, generator=g).to(dtype)
    st.K_res.copy_(K)
    st.V_res.copy_(V)
    tol = 1e-5 if dtype == torch.float32 else 1e-3
    for use_rows in (st.k + st.m, max(1, (st.k + st.m) // 2)):
        out = st.flash_decode(q.cuda(), rows=use_rows).float().cpu()
        ref = orc.attention(q[:, :, None], K[:, :, :use_rows], V[:, :, :use_rows])[:, :, 0]
        if dtype == torch.bfloat16:
            assert bf16_excess(out, ref, 1e-5) <= 1.0
        else:
            assert _rel(out, ref) < tol
    # calling twice gives the same bits (the ticket is re-armed, the fold order is fixed)
    a = st.flash_decode(q.cuda()).clone()
    b = st.flash_decode(q.cuda()).clone()
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,r,k,m,bsz,hq,hkv,max_iter,d", [
    (torch.float32, 16, 256, 16, 1, 8, 2, 2, 128), (torch.bfloat16, 32, 512, 64, 2, 8, 2, 2, 128),
    (torch.float32, 8, 64, 4, 2, 4, 2, 3, 128), (torch.bfloat16, 64, 300, 20, 1, 4, 4, 1, 128),
    (torch.float32, 32, 100, 7, 1, 2, 1, 0, 128),
    (torch.bfloat16, 16, 1024, 32, 2, 4, 2, 1, 128),   # rank and ring of the Qwen2.5-7B configuration (tensor-core Grams at r=16)
    (torch.bfloat16, 8, 200, 8, 1, 3, 1, 2, 128),
    (torch.bfloat16, 16, 300, 12, 1, 4, 2, 2, 64),     # head_dim 64: one operand tile per right factor, 128-row key stages
    (torch.float32, 8, 150, 6, 1, 2, 2, 2, 64),
    (torch.bfloat16, 64, 4096, 128, 1, 2, 1, 4, 128),  # rank, set size and alternations of the 256K configuration
])
def test_project_update_matches_oracle(dtype, r, k, m, bsz, hq, hkv, max_iter, d):
    _check_project_update(dtype, r, k, m, bsz, hq, hkv, max_iter, d, (1.0, 1.0))


@pytest.mark.parametrize("dtype,r,k,m,bsz,hq,hkv,max_iter,d,lam", [
    (torch.float32, 16, 256, 16, 1, 4, 2, 2, 128, (0.75, 1.5)),     # lambda_dec_q, lambda_dec_k
    (torch.bfloat16, 32, 512, 64, 1, 8, 2, 3, 128, (2.5, 0.4)),
    (torch.float32, 8, 64, 4, 2, 2, 2, 2, 64, (1.0, 0.3)),          # one weight at 1 still takes the general form
    (torch.bfloat16, 64, 300, 20, 1, 2, 2, 2, 128, (0.0, 2.0)),     # no q k^T term of the new token at all
    (torch.bfloat16, 16, 1024, 32, 1, 4, 2, 2, 128, (4.0, 1.0)),
])
def test_project_update_with_weights_matches_oracle(dtype, r, k, m, bsz, hq, hkv, max_iter, d, lam):
    _check_project_update(dtype, r, k, m, bsz, hq, hkv, max_iter, d, lam)


@pytest.mark.parametrize("dtype,lam", [(torch.float32, (1.0, 1.0)), (torch.bfloat16, (1.0, 1.0)), (torch.float32, (0.5, 2.0))])
def test_cast_lrqk_decode_functional_form(dtype, lam):
    """The reference's function signature (lrqk_attention.py:803-839) on the projection kernel, against the oracle."""
    from lrqk_b200 import cast_lrqk_decode
    g = torch.Generator().manual_seed(17)
    b, h, n, r, d = 2, 4, 300, 16, 128
    A = (torch.randn(b, h, n, r, generator=g) * 0.5).to(dtype)
    K = torch.randn(b, h, n, d, generator=g).to(dtype)
    BQ = (torch.randn(b, h, r, d, generator=g) * 0.3).to(dtype)
    BK = (torch.randn(b, h, r, d, generator=g) * 0.3).to(dtype)
    q = torch.randn(b, h, 1, d, generator=g).to(dtype)
    k = torch.randn(b, h, 1, d, generator=g).to(dtype)
    oBQ, oBK, oq, ok = cast_lrqk_decode(BQ.cuda(), A.cuda(), BK.cuda(), K.cuda(), q.cuda(), k.cuda(),
                                        lambda_dec_q=lam[0], lambda_dec_k=lam[1], max_iter=3, tol=1e-12)
    assert oq.shape == (b, h, 1, r) and ok.shape == (b, h, 1, r) and oBQ.dtype == dtype
    eBQ, eBK, eq, ek = orc.cast_decode(BQ, A, BK, K, q, k, 3, 1e-12, lam[0], lam[1])
    if dtype == torch.float32:
        for x, y in ((oBQ, eBQ), (oBK, eBK), (oq, eq), (ok, ek)):
            assert _rel(x.float().cpu(), y.float()) < 2e-4
    else:
        f = torch.float32
        rBQ, rBK, rq, rk = orc.decode_project_update(BQ.to(f), A.to(f), BK.to(f), K.to(f), q.to(f), k.to(f), 3, 1e-12)
        for x, y in ((oBQ, rBQ), (oBK, rBK), (oq, rq), (ok, rk)):
            assert bf16_excess(x, y, 2e-4) <= 1.0


def test_project_then_update_equals_project_update():
    """lrqk_decode_project followed by lrqk_decode_update (how the fused step splits the stage) against the one call."""
    from gpu_util import synthetic_state
    st = synthetic_state(1, 8, 2, 128, 32, 512, 64, 9000, seed=4)
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(1, 8, 128, generator=g, device="cuda").to(torch.bfloat16)
    kn = torch.randn(1, 2, 128, generator=g, device="cuda").to(torch.bfloat16)
    BQ, BK, A = st.B_Q.clone(), st.B_K.clone(), st.A_K.clone()
    qa = st.project_update(q, kn, 2, 1e-2, 9000).clone()
    one = (st.B_Q.clone(), st.B_K.clone(), st.A_K[:, :, 9000].clone(), int(st.counters[2]))
    st.B_Q.copy_(BQ); st.B_K.copy_(BK); st.A_K.copy_(A)
    st.project(q, kn, 2, 9000)
    torch.cuda.synchronize()
    assert torch.equal(st.B_Q, BQ) and torch.equal(st.A_K, A)          # the first half writes only its workspace
    qb = st.update(q, kn, 2, 1e-2, 9000).clone()
    torch.cuda.synchronize()
    assert torch.equal(qa, qb) and torch.equal(st.B_Q, one[0]) and torch.equal(st.B_K, one[1])
    assert torch.equal(st.A_K[:, :, 9000], one[2]) and int(st.counters[2]) == one[3]
    st.check_status()
    st.close()


def _check_project_update(dtype, r, k, m, bsz, hq, hkv, max_iter, d, lam):
    g = torch.Generator().manual_seed(r * k)
    cap = 3000 if k < 2000 else 6000
    grp = hq // hkv
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hkv, head_dim=d, r=r, k=k, m=m, a_capacity=cap,
                host_capacity=16, dtype=dtype, with_host=False, max_iter=max(1, max_iter),
                weights=(1.0, 1.0) + tuple(lam))
    A = torch.randn(bsz, hq, cap, r, generator=g).to(dtype)
    append_row = cap - 500
    A[:, :, append_row:] = 0                     # the row being appended still reads as zero
    BQ = (torch.randn(bsz, hq, r, d, generator=g) * 0.3).to(dtype)
    BK = (torch.randn(bsz, hq, r, d, generator=g) * 0.3).to(dtype)
    Kres = torch.randn(bsz, hq, k + m, d, generator=g).to(dtype)
    table = torch.stack([torch.randperm(append_row - m - 5, generator=g)[:k] for _ in range(bsz * hq)]).view(bsz, hq, k).int()
    lite = torch.arange(append_row - m + 1, append_row + 1, dtype=torch.int32)
    q = torch.randn(bsz, hq, d, generator=g).to(dtype)
    kn = torch.randn(bsz, hkv, d, generator=g).to(dtype)
    for t, s in ((st.A_K, A), (st.B_Q, BQ), (st.B_K, BK), (st.K_res, Kres), (st.table, table), (st.lite_pos, lite)):
        t.copy_(s)
    for tol_exit in (1e-12, 1e3):                # never leave early / leave after the first alternation
        st.B_Q.copy_(BQ)
        st.B_K.copy_(BK)
        st.A_K.copy_(A)
        qh = st.project_update(q.cuda(), kn.cuda(), max_iter, tol_exit, append_row).float().cpu()
        act = torch.cat([table.long(), lite.long().view(1, 1, m).expand(bsz, hq, m)], dim=-1)
        A_act = torch.gather(A, 2, act[..., None].expand(-1, -1, -1, r))
        krep = kn.repeat_interleave(grp, dim=1)[:, :, None]
        f = torch.float32
        ops = (BQ.to(f), A_act.to(f), BK.to(f), Kres.to(f), q[:, :, None].to(f), krep.to(f))
        if tuple(lam) == (1.0, 1.0):
            eBQ, eBK, eq, ek, iters = orc.decode_project_update(*ops, max_iter, tol_exit, return_iters=True)
        else:
            eBQ, eBK, eq, ek, iters = orc.decode_project_update_weighted(*ops, lam[0], lam[1], max_iter, tol_exit,
                                                                         return_iters=True)
        assert int(st.counters[2].item()) == iters
        tol = 2e-4                                   # the solves amplify fp32 round-off
        if dtype == torch.float32:
            assert _rel(qh, eq[:, :, 0]) < tol
            assert _rel(st.A_K[:, :, append_row].float(), ek[:, :, 0]) < tol
            assert _rel(st.B_Q.float(), eBQ) < tol and _rel(st.B_K.float(), eBK) < tol
        else:                                        # the same bound, plus the rounding of the stored value
            assert bf16_excess(qh, eq[:, :, 0], tol) <= 1.0
            assert bf16_excess(st.A_K[:, :, append_row], ek[:, :, 0], tol) <= 1.0
            assert bf16_excess(st.B_Q, eBQ, tol) <= 1.0 and bf16_excess(st.B_K, eBK, tol) <= 1.0
        assert torch.equal(st.A_K[:, :, :append_row].cpu(), A[:, :, :append_row])


@pytest.mark.parametrize("dtype,d,k,m,bsz,hq,hkv,miss", [
    (torch.bfloat16, 128, 512, 64, 1, 8, 2, 0.9), (torch.bfloat16, 128, 2048, 64, 1, 4, 2, 0.1),
    (torch.float32, 128, 300, 20, 2, 4, 4, 0.5), (torch.bfloat16, 64, 257, 8, 1, 6, 3, 1.0),
    (torch.float32, 64, 64, 4, 1, 2, 1, 0.0),
    (torch.bfloat16, 128, 9000, 16, 1, 2, 1, 0.6),   # more rows than 64 splits of one staging round: two rounds per CTA
    (torch.float32, 128, 4990, 10, 1, 1, 1, 0.3),
])
def test_fetch_attend_equals_miss_gather_then_attention(dtype, d, k, m, bsz, hq, hkv, miss):
    """One kernel that refills the missed slots from the host store while it attends to them, against the two
    kernels it replaces in the fused step: resident rows and attention output identical bit for bit; a slot
    whose table entry points outside the host store is left alone by both."""
    ctx = max(5000, 2 * k)
    g = torch.Generator().manual_seed(k + d)
    st = _state(bsz=bsz, q_heads=hq, kv_heads=hkv, head_dim=d, r=16, k=k, m=m, a_capacity=ctx + 64,
                host_capacity=ctx + 64, dtype=dtype)
    st.host.data[:, :, :ctx].copy_(torch.randn(bsz, hkv, ctx, 2 * d, generator=g).to(dtype))
    st.K_res.copy_(torch.randn(bsz, hq, k + m, d, generator=g).to(dtype))
    st.V_res.copy_(torch.randn(bsz, hq, k + m, d, generator=g).to(dtype))
    table = torch.stack([torch.randperm(ctx, generator=g)[:k] for _ in range(bsz * hq)]).view(bsz, hq, k).int()
    mask = (torch.rand(bsz, hq, k, generator=g) < miss).to(torch.uint8)
    if miss > 0:
        table[0, 0, 3] = ctx + 64 + 7          # malformed: outside the store
        table[0, hq - 1, 5] = -2
        mask[0, 0, 3] = mask[0, hq - 1, 5] = 1
    st.table.copy_(table)
    st.mask.copy_(mask)
    # the miss list the stand-alone fetch kernel takes: (head, slot, position) of every set mask byte
    hh, ss = np.nonzero(mask.view(bsz * hq, k).numpy())
    entries = np.stack([hh, ss, table.view(bsz * hq, k).numpy()[hh, ss]], axis=1).astype(np.int32)
    st.miss_list[:len(entries)].copy_(torch.from_numpy(entries))
    st.counters.zero_()
    st.counters[0] = len(entries)
    q = torch.randn(bsz, hq, d, generator=g).to(dtype).cuda()
    K0, V0 = st.K_res.clone(), st.V_res.clone()
    st.miss_gather()
    out_a = st.flash_decode(q).clone()
    Ka, Va = st.K_res.clone(), st.V_res.clone()
    st.K_res.copy_(K0)
    st.V_res.copy_(V0)
    out_b = st.fetch_attend(q).clone()
    torch.cuda.synchronize()
    assert torch.equal(st.K_res, Ka) and torch.equal(st.V_res, Va)
    assert torch.equal(out_a.view(torch.uint8), out_b.view(torch.uint8))
    # and the refilled slots hold the host rows
    grp = hq // hkv
    ok = (table >= 0) & (table < ctx + 64) & (mask != 0)
    for b in range(bsz):
        for h in range(hq):
            sel = ok[b, h].nonzero()[:, 0]
            rows = st.host.data[b, h // grp][table[b, h][sel].long()]
            assert torch.equal(st.K_res[b, h, sel.cuda()].cpu(), rows[:, :d])
            assert torch.equal(st.V_res[b, h, sel.cuda()].cpu(), rows[:, d:])
    untouched = ~ok
    assert torch.equal(st.K_res[:, :, :k][untouched.cuda()], K0[:, :, :k][untouched.cuda()])
    st.check_status()
    st.close()


# --------------------------------------------------------------------------------------------
# whole decode steps against the oracle and against the reference's recorded trace
# --------------------------------------------------------------------------------------------
def _load_case(name):
    z = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    return z, json.loads(str(z["config"]))


@pytest.mark.parametrize("name", ["cfg0", "wrap_top", "topcol_g1", "weighted", "weighted_decode_only"])
def test_layer_step_replay_against_oracle_and_golden(name):
    """Every step starts from the oracle's state, so one stage's round-off cannot cascade:
    integer outputs must then equal the oracle's exactly whenever the device scores rank the
    candidates the way the oracle's do; attention is compared with the reference's trace."""
    from gpu_util import bookkeeping, squeeze_step, state_from_oracle, sync_state
    z, c = _load_case(name)
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    lay = orc.OracleLayer(c["r"], c["k"], c["m"], c["hq"] // c["hkv"], c["max_iter"], c["tol"],
                          capacity=c["seq"] + 64, init=c["init"], weights=tuple(c.get("weights", (1.0, 1.0, 1.0, 1.0))))
    torch.manual_seed(c["init_seed"])
    lay.prefill(Q, K, V)
    st = state_from_oracle(lay, c["hkv"], max_iter=c["max_iter"][1])
    exact_steps = 0
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        sync_state(st, lay)
        bk = bookkeeping(lay)
        dq, dk, dv = squeeze_step(q, k, v)
        args = st.make_step_args(dq, dk, dv, max_iter=c["max_iter"][1], tol=c["tol"], **bk)
        st.layer_step(args)
        torch.cuda.synchronize()
        lay.decode(q, k, v)
        tr = lay.trace[-1]
        assert bk["candidates"] == tr.candidates
        assert st.lite_pos.cpu().tolist() == lay.lite_indices
        assert _rel(st.q_hat.cpu(), tr.q_hat[:, :, 0]) < 2e-4
        # selection from the device's own q_hat, judged with the oracle's tie rule
        dev_scores = orc.proxy_scores(st.A_K[:, :, :tr.candidates].cpu(), st.q_hat.cpu()[:, :, None])
        wanted = st.wanted.cpu().numpy()
        overlap = np.mean([len(np.intersect1d(wanted[b, h], tr.wanted[b, h])) / c["k"]
                           for b in range(c["bsz"]) for h in range(c["hq"])])
        assert overlap > 0.99
        counters = st.counters.cpu().numpy()
        assert counters[1] == 0
        if np.array_equal(wanted, tr.wanted):
            exact_steps += 1
            assert np.array_equal(st.table.cpu().numpy(), tr.table)
            assert np.array_equal(st.mask.cpu().numpy(), tr.mask)
            assert counters[0] == tr.mask.sum()
            assert torch.equal(st.K_res.cpu(), lay.Kres) and torch.equal(st.V_res.cpu(), lay.Vres)
            assert torch.equal(st.host.data, lay.host)
            assert _rel(st.attn_out.cpu(), torch.from_numpy(z[f"s{s}_attn"])[:, :, 0]) < 1e-4
        del dev_scores
    assert exact_steps >= c["steps"] - 1
    st.close()


@pytest.mark.parametrize("c", [
    dict(seed=3, bsz=2, hq=8, hkv=2, seq=3000, d=128, r=32, k=256, m=8, steps=20, max_iter=2),
    # head structure, rank and ring length of the Qwen2.5-7B configuration (28/4 heads, r=16, m=32, one alternation)
    dict(seed=4, bsz=2, hq=14, hkv=2, seq=2500, d=128, r=16, k=128, m=32, steps=36, max_iter=1),
    # ... and of the Qwen2.5-32B configuration (40/8 heads, r=64, m=128, four alternations)
    dict(seed=5, bsz=1, hq=10, hkv=2, seq=6000, d=128, r=64, k=512, m=128, steps=10, max_iter=4),
], ids=["llama-like", "qwen7b-like", "qwen32b-like"])
def test_layer_step_free_running_bf16(c):
    """bf16, many steps without resynchronising from the oracle.  After each step the oracle
    adopts the device's rounded factors, so both sides start every step from the same bits: the
    projected query must agree within tolerance, and the integer stages -- recomputed by the
    oracle from the device's own q_hat -- must agree exactly."""
    from gpu_util import bookkeeping, squeeze_step, state_from_oracle
    grp = c["hq"] // c["hkv"]
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"], dtype=torch.bfloat16)
    lay = orc.OracleLayer(c["r"], c["k"], c["m"], grp, (2, c["max_iter"]), (1e-2, 1e-2), capacity=c["seq"] + 64, init="top")
    lay.prefill(Q, K, V)
    st = state_from_oracle(lay, c["hkv"], max_iter=c["max_iter"])
    total_miss = 0
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"], dtype=torch.bfloat16)
        bk = bookkeeping(lay)
        dq, dk, dv = squeeze_step(q, k, v)
        st.layer_step(st.make_step_args(dq, dk, dv, max_iter=c["max_iter"], tol=1e-2, **bk))
        torch.cuda.synchronize()
        table_before = lay.table.copy()
        lay.decode(q, k, v, want_attention=False)
        tr = lay.trace[-1]
        assert bk["candidates"] == tr.candidates
        assert bf16_excess(st.q_hat, tr.q_hat[:, :, 0].float(), 5e-4, roundings=2) <= 1.0   # the oracle's is rounded too
        wanted = orc.topk_sorted(orc.proxy_scores(lay.A_K[:, :, :tr.candidates], st.q_hat.cpu()[:, :, None]), c["k"])
        assert np.array_equal(st.wanted.cpu().numpy(), wanted), f"step {s}"
        table, mask, cnt = orc.slot_diff(table_before, wanted)
        assert np.array_equal(st.table.cpu().numpy(), table) and np.array_equal(st.mask.cpu().numpy(), mask)
        assert np.array_equal(st.miss_count.cpu().numpy(), cnt)
        total_miss += int(cnt.sum())
        assert torch.equal(st.host.data, lay.host)
        # every selected slot holds the host row of its table entry; lite slots hold the ring
        Kres, Vres = st.K_res.cpu(), st.V_res.cpu()
        idx = torch.from_numpy(table.astype(np.int64))
        for b in range(c["bsz"]):
            for h in range(c["hq"]):
                rows = st.host.data[b, h // grp][idx[b, h]]
                assert torch.equal(Kres[b, h, :c["k"]], rows[:, :c["d"]])
                assert torch.equal(Vres[b, h, :c["k"]], rows[:, c["d"]:])
        assert torch.equal(Kres[:, :, c["k"]:], lay.Kres[:, :, c["k"]:])
        assert torch.equal(Vres[:, :, c["k"]:], lay.Vres[:, :, c["k"]:])
        assert bf16_excess(st.attn_out, orc.attention(q, Kres, Vres)[:, :, 0], 1e-5) <= 1.0
        # the oracle adopts the device's state for the next step
        lay.table = table
        lay.B_Q, lay.B_K = st.B_Q.cpu(), st.B_K.cpu()
        lay.A_K[:, :, lay.a_len - 1] = st.A_K[:, :, lay.a_len - 1].cpu()
        lay.Kres, lay.Vres = Kres.clone(), Vres.clone()
    assert total_miss > 0
    st.close()
