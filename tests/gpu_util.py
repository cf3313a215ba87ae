"""Helpers shared by the GPU parity tests: move an oracle layer's state onto the device."""
import numpy as np
import torch

import lrqk_oracle as orc
from lrqk_b200.state import LayerState


def state_from_oracle(lay: "orc.OracleLayer", kv_heads: int, max_iter: int = 2) -> LayerState:
    b, hq, a_cap, r = lay.A_K.shape
    d = lay.Kres.shape[-1]
    st = LayerState(b, hq, kv_heads, d, r, lay.k, lay.m, a_capacity=a_cap, host_capacity=lay.host.shape[2],
                    dtype=lay.A_K.dtype, max_iter=max_iter)
    sync_state(st, lay)
    return st


def sync_state(st: LayerState, lay: "orc.OracleLayer"):
    st.A_K.copy_(lay.A_K)
    st.B_Q.copy_(lay.B_Q)
    st.B_K.copy_(lay.B_K)
    st.K_res.copy_(lay.Kres)
    st.V_res.copy_(lay.Vres)
    st.table.copy_(torch.from_numpy(lay.table))
    st.lite_pos.copy_(torch.tensor(lay.lite_indices, dtype=torch.int32))
    st.host.data.copy_(lay.host)
    st.host.current_len = lay.host_len
    torch.cuda.synchronize()


def bookkeeping(lay: "orc.OracleLayer"):
    """Host counters of the NEXT decode step, derived the way the reference's Python
    attributes evolve (lrqk_attention.py:1174-1196, :1562-1568)."""
    lite_slot = lay.lite_len
    position = lay.current_len
    fills = lite_slot + 1 >= lay.m
    flush_rows = lay.m if fills else 0
    host_row = lay.host_len
    lite_after = list(lay.lite_indices)
    lite_after[lite_slot] = position
    next_len = 0 if fills else lite_slot + 1
    candidates = lite_after[next_len] - 1
    return dict(lite_slot=lite_slot, position=position, flush_rows=flush_rows, host_row=host_row,
                candidates=candidates)


def squeeze_step(q, k, v):
    """[B,H,1,d] -> contiguous [B,H,d] CUDA tensors."""
    return tuple(t[:, :, 0, :].contiguous().cuda() for t in (q, k, v))
