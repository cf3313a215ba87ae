"""The fused decode step (``lrqk_layer_step``) at shapes where a head's candidates span a CLUSTER of
CTAs -- 2, 4 and 8 -- which is how the benchmark's shape (32 heads x 131007 candidates: clusters of 4,
hit/miss difference as the tail of the scoring kernel behind a cluster barrier) runs.

Every case runs one step twice from the same state, stage by stage and fused, and requires every
output to be bit-identical (projected query, appended factor row, right factors, selection, slot
table, mask, miss counts, sorted miss list, resident rows, ring positions, flushed host rows,
attention).  The stage-by-stage result is then judged against the CPU oracle: the selection must be
the oracle's top-k (ties -> lower position) of the device's own fp32 scores, table / mask / counts the
oracle's set difference, every refilled slot must hold the host store's row, and the attention must
agree with the oracle's on the resident rows within the fp32 tolerance (1e-5) plus one rounding of the
result to bf16 (``gpu_util.bf16_excess``).
"""
import numpy as np
import pytest
import torch

import lrqk_oracle as orc

pytestmark = pytest.mark.gpu

CASES = [
    # hq, hkv, ctx, r, k, m, max_iter, expected cluster size of the scoring kernel
    dict(bsz=1, hq=8, hkv=2, ctx=20000 + 65, r=32, k=512, m=64, max_iter=2, cluster=4),
    dict(bsz=1, hq=3, hkv=1, ctx=70001 + 33, r=16, k=1024, m=32, max_iter=1, cluster=8),
    dict(bsz=2, hq=64, hkv=16, ctx=60000, r=32, k=1024, m=64, max_iter=2, cluster=2),
    dict(bsz=1, hq=32, hkv=8, ctx=131072, r=32, k=2048, m=64, max_iter=2, cluster=4),      # the benchmark's shape
    dict(bsz=1, hq=4, hkv=2, ctx=262144, r=64, k=4096, m=128, max_iter=4, cluster=8),      # 256K shape, fewer heads
]


def _ids(c):
    return f"{c['bsz']}x{c['hq']}h-ctx{c['ctx']}-r{c['r']}-k{c['k']}-cluster{c['cluster']}"


@pytest.mark.parametrize("c", CASES, ids=_ids)
@pytest.mark.parametrize("flush", [False, True], ids=["ring-write", "ring-flush"])
def test_fused_step_equals_staged_and_oracle(c, flush):
    from gpu_util import bf16_excess, synthetic_state
    from lrqk_b200 import selfcheck
    bsz, hq, hkv, d, r, k, m, ctx = c["bsz"], c["hq"], c["hkv"], 128, c["r"], c["k"], c["m"], c["ctx"]
    grp = hq // hkv
    st = synthetic_state(bsz, hq, hkv, d, r, k, m, ctx, seed=ctx % 97, max_iter=c["max_iter"], tie_head=1)
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn(bsz, hq, d, generator=g, device="cuda").to(torch.bfloat16)
    kn = torch.randn(bsz, hkv, d, generator=g, device="cuda").to(torch.bfloat16)
    vn = torch.randn(bsz, hkv, d, generator=g, device="cuda").to(torch.bfloat16)
    # host counters of the step, as LightAttentionIndicesFactory._step_counters derives them
    lite_slot = m - 1 if flush else 5
    lite = list(range(ctx - m, ctx))
    lite[lite_slot] = ctx
    flush_rows = m if flush else 0
    candidates = lite[0 if flush else lite_slot + 1] - 1
    table_before = st.table.cpu().numpy().copy()
    staged = {}
    bad = selfcheck.compare_step(st, q, kn, vn, lite_slot=lite_slot, position=ctx, flush_rows=flush_rows, host_row=ctx,
                                 candidates=candidates, max_iter=c["max_iter"], tol=1e-2, staged_out=staged)
    assert bad == [], f"fused and stage-by-stage steps differ in {bad}"
    # the scoring kernel really ran as a cluster of the expected size
    assert -(-candidates // c["cluster"]) <= 49152 and (c["cluster"] == 1 or candidates > 49152 or candidates // c["cluster"] >= 4096)

    # ---- the stage-by-stage result against the oracle ----
    scores = torch.full((bsz, hq, candidates), float("nan"), device="cuda")
    again = st.score_topk(staged["q_hat"], candidates, scores_out=scores).cpu().numpy()
    scores = scores.cpu()
    wanted = staged["wanted"].cpu().numpy()
    assert np.array_equal(again, wanted)
    assert np.array_equal(wanted, orc.topk_sorted(scores, k)), "selection is not the oracle's top-k of the device scores"
    ref_scores = orc.proxy_scores(st.A_K[:, :, :candidates].cpu(), staged["q_hat"].cpu()[:, :, None, :])
    assert float((scores - ref_scores).abs().max() / ref_scores.abs().max()) < 1e-3
    table, mask, cnt = orc.slot_diff(table_before, wanted)
    assert np.array_equal(staged["table"].cpu().numpy(), table)
    assert np.array_equal(staged["mask"].cpu().numpy(), mask)
    assert np.array_equal(staged["miss_count"].cpu().numpy(), cnt)
    ml = staged["miss_list"].cpu().numpy()
    heads, slots = np.nonzero(mask.reshape(bsz * hq, k))
    assert np.array_equal(ml[:, 0], heads) and np.array_equal(ml[:, 1], slots)
    assert np.array_equal(ml[:, 2], table.reshape(bsz * hq, k)[heads, slots])
    assert int(cnt.sum()) > 0
    # resident rows: every selected slot holds the host row of its table entry, the ring holds the step's k/v
    Kres, Vres = staged["K_res"].cpu(), staged["V_res"].cpu()
    idx = torch.from_numpy(table.astype(np.int64))
    for b in range(bsz):
        for h in range(0, hq, max(1, hq // 8)):
            rows = st.host.data[b, h // grp][idx[b, h]]
            assert torch.equal(Kres[b, h, :k], rows[:, :d]) and torch.equal(Vres[b, h, :k], rows[:, d:])
            assert torch.equal(Kres[b, h, k + lite_slot], kn[b, h // grp].cpu())
            assert torch.equal(Vres[b, h, k + lite_slot], vn[b, h // grp].cpu())
    assert staged["lite_pos"].cpu().tolist() == lite
    if flush:      # the ring went to host rows [ctx, ctx + m) as K|V, in slot order, from the first head of each group
        ring = torch.cat([Kres[:, ::grp, k:], Vres[:, ::grp, k:]], dim=-1)
        assert torch.equal(staged["host_rows"], ring)
    att = orc.attention(q.cpu()[:, :, None].float(), Kres.float(), Vres.float())[:, :, 0]
    assert bf16_excess(staged["attn_out"], att, 1e-5) <= 1.0     # fp32 tolerance + one rounding to bf16
    st.close()
