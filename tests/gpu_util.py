"""Helpers shared by the GPU parity tests: move an oracle layer's state onto the device."""
import numpy as np
import torch

import lrqk_oracle as orc
from lrqk_b200.state import LayerState


def state_from_oracle(lay: "orc.OracleLayer", kv_heads: int, max_iter: int = 2) -> LayerState:
    b, hq, a_cap, r = lay.A_K.shape
    d = lay.Kres.shape[-1]
    st = LayerState(b, hq, kv_heads, d, r, lay.k, lay.m, a_capacity=a_cap, host_capacity=lay.host.shape[2],
                    dtype=lay.A_K.dtype, max_iter=max_iter, weights=getattr(lay, "weights", (1.0, 1.0, 1.0, 1.0)))
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


def synthetic_state(bsz, hq, hkv, d, r, k, m, ctx, seed=0, dtype=torch.bfloat16, max_iter=2, tie_head=None):
    """A decode-ready layer state at context length `ctx` built from seeded random tensors instead of a
    prompt pass (full-size shapes would take the CPU oracle minutes): random rank-r factors, right
    factors of a well-conditioned size, a host store of random rows, a random ascending resident set
    whose slots hold the matching host rows, and a full lite ring over the last m positions.
    `tie_head`: query head whose factors are quantised coarsely so that equal scores occur."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    grp = hq // hkv
    cap = ctx + 2 * m + 64
    st = LayerState(bsz, hq, hkv, d, r, k, m, a_capacity=cap, host_capacity=cap, dtype=dtype, max_iter=max_iter)
    st.A_K[:, :, :ctx].copy_(torch.randn(bsz, hq, ctx, r, generator=g, device=dev) * 0.5)
    if tie_head is not None:
        st.A_K[:, tie_head, :ctx].copy_((st.A_K[:, tie_head, :ctx].float() * 2).round() / 2)
    st.B_Q.copy_(torch.randn(bsz, hq, r, d, generator=g, device=dev) * 0.3)
    st.B_K.copy_(torch.randn(bsz, hq, r, d, generator=g, device=dev) * 0.3)
    hostg = torch.Generator().manual_seed(seed + 1)
    for b in range(bsz):
        for h in range(hkv):
            st.host.data[b, h, :ctx].copy_(torch.randn(ctx, 2 * d, generator=hostg).to(dtype))
    st.host.current_len = ctx
    cand = ctx - m
    rng = np.random.default_rng(seed + 2)
    table = np.stack([np.sort(rng.permutation(cand)[:k]) for _ in range(bsz * hq)]).astype(np.int32).reshape(bsz, hq, k)
    st.table.copy_(torch.from_numpy(table))
    idx = torch.from_numpy(table.astype(np.int64))
    lite = torch.arange(ctx - m, ctx)
    for b in range(bsz):
        for h in range(hq):
            rows = st.host.data[b, h // grp][idx[b, h]]
            st.K_res[b, h, :k].copy_(rows[:, :d])
            st.V_res[b, h, :k].copy_(rows[:, d:])
            ring = st.host.data[b, h // grp][lite]
            st.K_res[b, h, k:].copy_(ring[:, :d])
            st.V_res[b, h, k:].copy_(ring[:, d:])
    st.lite_pos.copy_(lite.to(torch.int32))
    torch.cuda.synchronize()
    return st


def bf16_excess(dev: torch.Tensor, ref32: torch.Tensor, fp32_tol: float, roundings: int = 1) -> float:
    """How far a bf16 result `dev` lies from the fp32 oracle value `ref32`, in units of the allowed
    distance; <= 1 passes.  Allowed per element: the arithmetic tolerance the same kernel meets in
    fp32 (`fp32_tol`, relative to the largest magnitude of the tensor -- 1e-5 for scores and
    attention) plus ONE rounding to bf16 of that element (half a bf16 ulp at the element's own
    magnitude, 2^-9 relative).  A bound "1e-3 of the largest magnitude" cannot be met by any value
    STORED in bf16 (the rounding of an element near the maximum alone is up to 2^-9 = 1.95e-3 of it);
    this bound is the tight form of the same statement: fp32 arithmetic, then a single rounding.
    `roundings=2` is for a reference that was itself rounded to bf16 (the oracle's per-step state)."""
    d, r = dev.detach().double().cpu(), ref32.detach().double().cpu()
    mag = torch.maximum(d.abs(), r.abs()).clamp_min(2.0 ** -126)
    half_ulp = torch.exp2(torch.floor(torch.log2(mag)) - 8.0)        # bf16: 8 significant bits, ulp = 2^(e-7)
    allowed = roundings * half_ulp * (1 + 1e-6) + fp32_tol * float(r.abs().max())
    return float(((d - r).abs() / allowed).max())
