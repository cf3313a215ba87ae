"""The decode step at the benchmark's full shape (32/8 heads, 131072-token context, r=32, k=2048,
m=64, bf16), checked through properties that do not need the CPU oracle to repeat the work:

* selection: ascending, duplicate-free, inside the candidate range, and a threshold cut of the
  kernel's own fp32 scores (every selected score >= every unselected one; of equal scores at the
  cut the lower positions are the ones taken);
* hit/miss: the slot table after the step holds exactly the wanted set, untouched slots kept their
  position, the mask counts the misses, the miss list has one entry per refilled slot;
* miss fetch: every refilled slot holds the host store's row of its new position, byte for byte,
  and no other resident row changed (checksums before/after);
* attention: equals softmax(q K^T / sqrt(d)) V over the resident rows computed by torch on the
  same device within the tolerance the small-shape tests use (1e-5 plus one rounding to bf16).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_full_shape_step_properties():
    from lrqk_b200.state import LayerState
    bsz, hq, hkv, d, r, k, m, ctx = 1, 32, 8, 128, 32, 2048, 64, 131072
    grp = hq // hkv
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(77)
    st = LayerState(bsz, hq, hkv, d, r, k, m, a_capacity=ctx + 256, host_capacity=ctx + 256, dtype=torch.bfloat16)
    st.A_K[:, :, :ctx].copy_(torch.randn(bsz, hq, ctx, r, generator=g, device=dev) * 0.5)
    # quantise one head's factors coarsely so that equal scores occur at the cut
    st.A_K[:, 3, :ctx].copy_((st.A_K[:, 3, :ctx].float() * 2).round() / 2)
    host = torch.randn(bsz, hkv, ctx, 2 * d, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    st.host.data[:, :, :ctx].copy_(host)
    q_hat = torch.randn(bsz, hq, r, generator=g, device=dev).to(torch.bfloat16)
    q_hat[:, 3] = (q_hat[:, 3].float() * 2).round() / 2
    cand = ctx - m - 1
    # slot table: a random resident set per head; resident rows = the matching host rows
    rng = np.random.default_rng(1)
    table = np.stack([rng.permutation(cand)[:k] for _ in range(hq)]).astype(np.int32).reshape(bsz, hq, k)
    st.table.copy_(torch.from_numpy(table))
    idx = torch.from_numpy(table.astype(np.int64))
    for h in range(hq):
        rows = host[0, h // grp][idx[0, h]]
        st.K_res[0, h, :k].copy_(rows[:, :d])
        st.V_res[0, h, :k].copy_(rows[:, d:])
    lite = torch.randn(bsz, hq, m, 2 * d, generator=g, device=dev).to(torch.bfloat16)
    st.K_res[:, :, k:].copy_(lite[..., :d])
    st.V_res[:, :, k:].copy_(lite[..., d:])
    K_before, V_before = st.K_res.clone(), st.V_res.clone()

    scores = torch.full((bsz, hq, cand), float("nan"), device=dev)
    wanted = st.score_topk(q_hat, cand, scores_out=scores).clone()
    st.slot_diff()
    st.miss_gather()
    q = torch.randn(bsz, hq, d, generator=g, device=dev).to(torch.bfloat16)
    out = st.flash_decode(q).clone()
    torch.cuda.synchronize()

    # ---- selection ----
    w = wanted.long()
    assert bool((w[..., 1:] > w[..., :-1]).all()) and int(w.min()) >= 0 and int(w.max()) < cand
    assert not torch.isnan(scores).any()
    sel = torch.gather(scores, 2, w)
    cut = sel.min(dim=2, keepdim=True).values
    picked = torch.zeros_like(scores, dtype=torch.bool).scatter_(2, w, True)
    assert bool((scores[~picked].view(bsz, hq, -1) <= cut).all())          # nothing unselected beats the cut
    at_cut = scores == cut
    for h in range(hq):                                                      # ties: the lower positions are taken
        pos = at_cut[0, h].nonzero()[:, 0]
        taken = picked[0, h][pos]
        n_taken = int(taken.sum())
        assert bool(taken[:n_taken].all()) and not bool(taken[n_taken:].any())
    assert int(at_cut[0, 3].sum()) > 1                                       # the quantised head really has ties
    # ---- hit/miss ----
    new_table = st.table.cpu().numpy()
    mask = st.mask.cpu().numpy().astype(bool)
    wn = wanted.cpu().numpy()
    assert np.array_equal(np.sort(new_table, axis=-1), wn)
    assert np.array_equal(new_table[~mask], table[~mask])                    # untouched slots keep their position
    cnt = st.miss_count.cpu().numpy()
    assert np.array_equal(cnt, mask.sum(-1)) and int(st.counters[0]) == int(mask.sum()) and int(st.counters[1]) == 0
    for h in range(0, hq, 7):                                                # refilled slots were not resident before
        assert not np.isin(new_table[0, h][mask[0, h]], table[0, h]).any()
    # ---- miss fetch ----
    nt = torch.from_numpy(new_table.astype(np.int64))
    for h in range(hq):
        rows = host[0, h // grp][nt[0, h]].to(dev)
        assert torch.equal(st.K_res[0, h, :k], rows[:, :d]) and torch.equal(st.V_res[0, h, :k], rows[:, d:])
    keep = torch.from_numpy(~mask).to(dev)
    assert torch.equal(st.K_res[:, :, :k][keep], K_before[:, :, :k][keep])
    assert torch.equal(st.K_res[:, :, k:], K_before[:, :, k:]) and torch.equal(st.V_res[:, :, k:], V_before[:, :, k:])
    # ---- attention ----
    ref = torch.nn.functional.scaled_dot_product_attention(q[:, :, None].float(), st.K_res.float(), st.V_res.float())[:, :, 0]
    from gpu_util import bf16_excess
    assert bf16_excess(out, ref, 1e-5) <= 1.0     # fp32 tolerance plus the rounding of the stored bf16 row
    st.close()
