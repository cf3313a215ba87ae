"""The CPU oracle replayed against traces recorded from the reference project itself
(tests/golden/*.npz, written by tests/golden/make_golden.py)."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import lrqk_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["cfg0", "wrap_top", "topcol_g1", "short_k3", "short_exact_k", "weighted", "weighted_prompt_only",
         "weighted_decode_only"]


def _sha(t):
    a = t.numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _load(name):
    z = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    return z, json.loads(str(z["config"]))


def _run(c, faithful):
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    lay = orc.OracleLayer(c["r"], c["k"], c["m"], c["hq"] // c["hkv"], c["max_iter"], c["tol"],
                          capacity=c["seq"] + 64, init=c["init"], faithful=faithful,
                          weights=tuple(c.get("weights", (1.0, 1.0, 1.0, 1.0))))
    torch.manual_seed(c["init_seed"])
    lay.prefill(Q, K, V)
    return lay


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("faithful", [True, False])
def test_oracle_matches_reference_trace(name, faithful):
    z, c = _load(name)
    lay = _run(c, faithful)
    # prefill: factors within fp32 round-off of the reference's, selection identical
    np.testing.assert_allclose(lay.B_Q.numpy(), z["prefill_B_Q"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(lay.B_K.numpy(), z["prefill_B_K"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(lay.A_K[:, :, :c["seq"]:8].numpy(), z["prefill_A_K_every8"], rtol=2e-4, atol=2e-5)
    assert np.array_equal(lay.table, z["prefill_table"])
    assert lay.host.shape[2] == int(z["host_capacity"])
    assert _sha(lay.Kres) == str(z["prefill_Kres_sha256"])
    assert _sha(lay.Vres) == str(z["prefill_Vres_sha256"])
    prev = lay.table.copy()
    for s in range(c["steps"]):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        Kres, Vres = lay.decode(q, k, v)
        tr = lay.trace[-1]
        np.testing.assert_allclose(tr.k_hat.numpy(), z[f"s{s}_k_hat"], rtol=2e-4, atol=2e-5)
        if f"s{s}_wanted" in z:
            assert np.array_equal(tr.wanted, z[f"s{s}_wanted"]), f"step {s}: selection differs"
            assert np.array_equal(tr.mask.astype(bool), prev != z[f"s{s}_table"])
        else:                              # all-resident branch of a short prompt: nothing selected
            assert tr.wanted is None and tr.candidates == -1
        if f"s{s}_rows" in z:
            assert Kres.shape[2] == int(z[f"s{s}_rows"])
        assert np.array_equal(tr.table, z[f"s{s}_table"]), f"step {s}: slot table differs"
        lite = z[f"s{s}_lite"]
        assert list(lite[:c["m"]]) == lay.lite_indices
        assert (int(lite[-3]), int(lite[-2]), int(lite[-1])) == (lay.lite_len, lay.current_len, lay.host_len)
        assert _sha(Kres) == str(z[f"s{s}_Kres_sha256"]), f"step {s}: resident keys differ"
        assert _sha(Vres) == str(z[f"s{s}_Vres_sha256"]), f"step {s}: resident values differ"
        np.testing.assert_allclose(tr.attn.numpy(), z[f"s{s}_attn"], rtol=1e-5, atol=1e-6)
        prev = tr.table.copy()
    np.testing.assert_allclose(lay.B_Q.numpy(), z["final_B_Q"], rtol=5e-4, atol=5e-5)
    np.testing.assert_allclose(lay.B_K.numpy(), z["final_B_K"], rtol=5e-4, atol=5e-5)


def test_slot_diff_docstring_example():
    # worked example in the reference's docstring of only_indices_in_cpu
    upd, mask = orc.slot_diff_python([0, 1, 2, 6, 7], [0, 2, 4, 5, 6])
    assert upd == [0, 4, 2, 6, 5] and mask == [0, 1, 0, 0, 1]
    u, m, cnt = orc.slot_diff(np.array([[0, 1, 2, 6, 7]]), np.array([[0, 2, 4, 5, 6]]))
    assert u.tolist() == [[0, 4, 2, 6, 5]] and m.tolist() == [[0, 1, 0, 0, 1]] and cnt.tolist() == [2]
    tu, tm = orc.slot_diff_reference_ops(torch.tensor([0, 1, 2, 6, 7]).view(1, 1, 5, 1),
                                         torch.tensor([0, 2, 4, 5, 6]).view(1, 1, 5, 1))
    assert tu.view(-1).tolist() == [0, 4, 2, 6, 5] and tm.view(-1).tolist() == [False, True, False, False, True]


def test_slot_diff_forms_agree_random():
    rng = np.random.default_rng(0)
    for k, l in ((8, 32), (64, 100), (257, 300), (33, 33)):
        now = np.stack([rng.permutation(l)[:k] for _ in range(6)]).astype(np.int32)
        new = np.stack([np.sort(rng.permutation(l)[:k]) for _ in range(6)]).astype(np.int32)
        u, m, cnt = orc.slot_diff(now, new)
        tu, tm = orc.slot_diff_reference_ops(torch.from_numpy(now.astype(np.int64)).view(1, 6, k, 1),
                                             torch.from_numpy(new.astype(np.int64)).view(1, 6, k, 1))
        assert np.array_equal(u, tu.view(6, k).numpy()) and np.array_equal(m.astype(bool), tm.view(6, k).numpy())
        for i in range(6):
            pu, pm = orc.slot_diff_python(now[i], new[i])
            assert pu == u[i].tolist() and pm == m[i].tolist()
            assert sorted(pu) == new[i].tolist() and cnt[i] == sum(pm)


def test_topk_forms_agree_and_tie_rule():
    rng = np.random.default_rng(1)
    s = rng.standard_normal((5, 1000)).astype(np.float32)
    assert np.array_equal(orc.topk_sorted(s, 100), orc.topk_sorted_numpy(s, 100))
    ref = torch.sort(torch.topk(torch.from_numpy(s), 100, dim=-1).indices, dim=-1).values.numpy()
    assert np.array_equal(orc.topk_sorted(s, 100), ref)
    # heavy ties: lower position wins; -0.0 ties with +0.0
    t = np.array([[1.0, 0.0, -0.0, 1.0, 0.0, 1.0, -1.0, 0.0]], dtype=np.float32)
    assert orc.topk_sorted(t, 5).tolist() == [[0, 1, 2, 3, 5]]
    assert orc.topk_sorted_numpy(t, 5).tolist() == [[0, 1, 2, 3, 5]]
    q = np.round(rng.standard_normal((3, 4096)) * 4).astype(np.float32)
    assert np.array_equal(orc.topk_sorted(q, 512), orc.topk_sorted_numpy(q, 512))
    with pytest.raises(ValueError):
        orc.topk_sorted(s, 1001)


def test_gather_matches_index_select():
    # the reference's own unit test of its gather: cpp_kernel/main_test.py:11-23
    rng = np.random.default_rng(2)
    for _ in range(4):
        w, n = int(rng.integers(128, 512)), int(rng.integers(10, 512))
        src = rng.standard_normal((64000, w)).astype(np.float32)
        rows = rng.integers(0, 64000, n)
        assert np.array_equal(orc.gather_rows(src, rows), src[rows])
    assert orc.gather_rows(src, np.zeros(0, dtype=np.int64)).shape == (0, w)


def test_masked_gather_invariants():
    # cpp_kernel/main_demo.py:150-196: masked slots hold src[b,h,idx], the rest stay zero
    rng = np.random.default_rng(3)
    b, h, g, s, w, k = 2, 8, 4, 32, 64, 8
    src = rng.standard_normal((b, h, s, w)).astype(np.float16)
    idx = np.stack([rng.permutation(s)[:k] for _ in range(b * h * g)]).reshape(b, h, g, k).astype(np.int64)
    mask = rng.random((b, h, g, k)) < 0.4
    out = orc.take_along_dim_with_mask(src, idx, mask)
    full = np.zeros((b, h, g, k, w), dtype=np.float16)
    full[mask] = out
    for i, j, a, e in np.ndindex(b, h, g, k):
        if mask[i, j, a, e]:
            assert np.array_equal(full[i, j, a, e], src[i, j, idx[i, j, a, e]])
        else:
            assert not full[i, j, a, e].any()
    rows = orc.miss_rows(idx.reshape(b, h * g, k).astype(np.int32), mask.reshape(b, h * g, k), h, g, s)
    assert np.array_equal(orc.gather_rows(src.reshape(-1, w), rows), out)


def test_lane_order_scores_close_to_matmul():
    g = torch.Generator().manual_seed(4)
    A = torch.randn(2, 3, 500, 32, generator=g).to(torch.bfloat16)
    q = torch.randn(2, 3, 1, 32, generator=g).to(torch.bfloat16)
    a = orc.proxy_scores_lane_order(A, q, 4)
    b = orc.proxy_scores(A, q).numpy()
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)
