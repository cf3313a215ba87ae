"""Cross-check of the fused decode step against the stage-by-stage entry points, on the device.

``lrqk_layer_step`` enqueues the whole step as five dependent kernels in which two stages have no
kernel of their own: the ring write rides on the projection kernel and the hit/miss difference
runs as the tail of the scoring kernel, behind a cluster barrier when a head spans several CTAs.
The stage-by-stage entries (``lrqk_lite_append``, ``lrqk_decode_project_update``,
``lrqk_score_topk``, ``lrqk_slot_diff``, ``lrqk_miss_gather``, ``lrqk_flash_decode``) compute the
same step with one launch per stage.  Both must leave the same bits behind; :func:`compare_step`
runs one step both ways from the same starting state and reports every output that differs.  It
is what the GPU tests use at the shapes where a head needs a cluster of CTAs, and what ``bench.py``
runs once per layer state after its timed loops.

The function synchronises the device and copies a few tensors; it is a diagnostic, not part of
the decode path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .state import LayerState


def _miss_rows(st: LayerState) -> torch.Tensor:
    """The miss list of the last step as rows (head, slot, pos) sorted by head, then slot (the
    order of the entries across heads is unspecified)."""
    n = int(st.counters[0].item())
    rows = st.miss_list[:n].to(torch.int64)
    key = rows[:, 0] * (st.k + 1) + rows[:, 1]
    return rows[torch.argsort(key)]


class _Snapshot:
    """The tensors a step reads and overwrites."""

    def __init__(self, st: LayerState, position: int, flush_rows: int, host_row: int):
        self.position, self.flush_rows, self.host_row = position, flush_rows, host_row
        torch.cuda.synchronize()           # the host store below is read on the CPU
        self.B_Q, self.B_K = st.B_Q.clone(), st.B_K.clone()
        self.K_res, self.V_res = st.K_res.clone(), st.V_res.clone()
        self.table, self.lite_pos = st.table.clone(), st.lite_pos.clone()
        self.a_row = st.A_K[:, :, position].clone()
        self.host = st.host.data[:, :, host_row:host_row + flush_rows].clone() if flush_rows else None

    def restore(self, st: LayerState):
        st.B_Q.copy_(self.B_Q); st.B_K.copy_(self.B_K)
        st.K_res.copy_(self.K_res); st.V_res.copy_(self.V_res)
        st.table.copy_(self.table); st.lite_pos.copy_(self.lite_pos)
        st.A_K[:, :, self.position].copy_(self.a_row)
        if self.host is not None:
            st.host.data[:, :, self.host_row:self.host_row + self.flush_rows].copy_(self.host)


def _outputs(st: LayerState, position: int, flush_rows: int, host_row: int, attention: bool) -> Dict[str, torch.Tensor]:
    torch.cuda.synchronize()
    out = {
        "q_hat": st.q_hat.clone(), "k_hat_row": st.A_K[:, :, position].clone(),
        "B_Q": st.B_Q.clone(), "B_K": st.B_K.clone(),
        "wanted": st.wanted.clone(), "table": st.table.clone(), "mask": st.mask.clone(),
        "miss_count": st.miss_count.clone(), "miss_list": _miss_rows(st),
        "K_res": st.K_res.clone(), "V_res": st.V_res.clone(), "lite_pos": st.lite_pos.clone(),
        "list_len_status_iters": st.counters[:3].clone(),
    }
    if attention:
        out["attn_out"] = st.attn_out.clone()
    if flush_rows:
        out["host_rows"] = st.host.data[:, :, host_row:host_row + flush_rows].clone()
    return out


@torch.no_grad()
def compare_step(st: LayerState, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, *, lite_slot: int,
                 position: int, flush_rows: int, host_row: int, candidates: int, max_iter: int, tol: float,
                 attention: bool = True, staged_out: Optional[dict] = None) -> List[str]:
    """Run one decode step twice from the current state -- stage by stage, then (after restoring
    every tensor the step overwrites) through ``lrqk_layer_step`` -- and return the names of the
    outputs that are not bit-identical (an empty list when the two agree).  The state is left as
    the fused step wrote it.  q [B,Hq,d], k_new / v_new [B,Hkv,d]; the integer arguments are the
    host counters of the step, as ``lrqk_step_args`` takes them.  ``staged_out``: an optional dict
    that receives the stage-by-stage outputs (device tensors)."""
    snap = _Snapshot(st, position, flush_rows, host_row)
    st.lite_append(k_new, v_new, lite_slot, position, flush_rows, host_row)
    st.project_update(q, k_new, max_iter, tol, position)
    st.score_topk(st.q_hat, candidates)
    st.slot_diff()
    st.miss_gather()
    if attention:
        st.flash_decode(q)
    staged = _outputs(st, position, flush_rows, host_row, attention)
    if staged_out is not None:
        staged_out.update(staged)
    snap.restore(st)
    st.layer_step(st.make_step_args(q, k_new, v_new, lite_slot, position, flush_rows, host_row, candidates,
                                    max_iter, tol, attention=attention))
    fused = _outputs(st, position, flush_rows, host_row, attention)
    bad = [name for name in staged if staged[name].shape != fused[name].shape or not torch.equal(staged[name], fused[name])]
    if int(fused["list_len_status_iters"][1].item()) != 0:
        bad.append("diff_status")          # a head's evicted and missing counts differed
    return bad


@torch.no_grad()
def compare_factory_step(fac, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, attention: bool = True,
                         staged_out: Optional[dict] = None) -> List[str]:
    """:func:`compare_step` for a prefilled ``LightAttentionIndicesFactory``: advances the factory's
    host counters by one step exactly as ``decode`` would.  q [B,Hq,d] or [B,Hq,1,d]."""
    st = fac.state
    fac._reserve()
    q = fac._flat(q.to(st.dtype), st.q_heads)
    k_new = fac._flat(k_new.to(st.dtype), st.kv_heads)
    v_new = fac._flat(v_new.to(st.dtype), st.kv_heads)
    slot, position, flush_rows, host_row, candidates = fac._step_counters()
    return compare_step(st, q, k_new, v_new, lite_slot=slot, position=position, flush_rows=flush_rows,
                        host_row=host_row, candidates=candidates, max_iter=fac.max_iter[1], tol=fac.tol[1],
                        attention=attention, staged_out=staged_out)
