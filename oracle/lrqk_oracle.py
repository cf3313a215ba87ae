"""CPU restatement of the LRQK prefill-factorisation / decode-selection path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is the checker the CUDA kernels are compared against and the thing that is
timed as the CPU baseline.  Floating-point stages are written with torch CPU
ops in fp32 in the same operation order as the reference project, so that on
the same torch build they give the same bits as the reference run on CPU;
integer stages are numpy (and, for large sizes, the C twin in
``lrqk_oracle.c``).  Every function cites the reference file:line it follows
(paths relative to the reference checkout).

Parity status: PINNED.  ``tests/golden/*.npz`` holds traces produced by running
the reference project itself (``tests/golden/make_golden.py``); the CPU test
suite replays them through this module.
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))

# ----------------------------------------------------------------------------
# C twin loader
# ----------------------------------------------------------------------------
_clib = None


def clib():
    """ctypes handle to ``liblrqk_oracle.so`` (built on demand with gcc)."""
    global _clib
    if _clib is None:
        so = os.path.join(_HERE, "liblrqk_oracle.so")
        src = os.path.join(_HERE, "lrqk_oracle.c")
        if not os.path.exists(so) or (os.path.exists(src) and os.path.getmtime(so) < os.path.getmtime(src)):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_lrqk_oracle_build", os.path.join(_HERE, "build_ref.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_c_oracle()
        lib = ctypes.CDLL(so)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p
        lib.oracle_topk_sorted_f32.argtypes = [vp, i64, i64, i64, i32, vp]
        lib.oracle_topk_sorted_f32.restype = ctypes.c_int
        lib.oracle_slot_diff.argtypes = [vp, vp, i64, i32, vp, vp, vp]
        lib.oracle_slot_diff.restype = ctypes.c_int
        lib.oracle_miss_rows.argtypes = [vp, vp, i64, i64, i64, i32, i64, vp]
        lib.oracle_miss_rows.restype = i64
        lib.oracle_gather_rows.argtypes = [vp, vp, vp, i64, i64]
        lib.oracle_gather_rows.restype = None
        lib.oracle_take_along_dim_with_mask.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, i64, i64]
        lib.oracle_take_along_dim_with_mask.restype = i64
        _clib = lib
    return _clib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


# ----------------------------------------------------------------------------
# small helpers
# ----------------------------------------------------------------------------
def expand_kv_heads(x: torch.Tensor, groups: int) -> torch.Tensor:
    """[B,Hkv,S,d] -> [B,Hkv*groups,S,d], each KV head repeated `groups` times in a
    row (q head h reads KV head h // groups): lrqk_attention.py:36-39 (HF repeat_kv)."""
    if groups == 1:
        return x
    b, h, s, d = x.shape
    return x[:, :, None, :, :].expand(b, h, groups, s, d).reshape(b, h * groups, s, d)


def _solve_left(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """X with A X = B (LU with partial pivoting): torch.linalg.solve_ex(A, B)[0]."""
    return torch.linalg.solve_ex(a, b)[0]


def _solve_right(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """X with X A = B: torch.linalg.solve_ex(A, B, left=False)[0]."""
    return torch.linalg.solve_ex(a, b, left=False)[0]


def _t(x: torch.Tensor) -> torch.Tensor:
    return x.transpose(-1, -2)


# ----------------------------------------------------------------------------
# A1: initial factors  (lrqk_attention.py:145-209)
# ----------------------------------------------------------------------------
def init_factors(Q: torch.Tensor, K: torch.Tensor, r: int, method: str = "randn"):
    """Initial A_Q, A_K [B,H,S,r].

    randn  -- two draws from the global torch generator, A_Q first (:145-152)
    top    -- the r columns of Q (resp. K) with the largest column abs-sum (:171-185)
    topcol -- the r columns with the largest |Q|+|K| column abs-sum, same columns
              for both (:154-169)
    """
    b, h, s, _ = Q.shape
    if method == "randn":
        aq = torch.randn((b, h, s, r), dtype=Q.dtype, device=Q.device)
        ak = torch.randn((b, h, s, r), dtype=K.dtype, device=K.device)
        return aq, ak
    qs = Q.abs().sum(dim=2, keepdim=True)
    ks = K.abs().sum(dim=2, keepdim=True)
    if method == "top":
        iq = torch.topk(qs, k=r, dim=-1).indices
        ik = torch.topk(ks, k=r, dim=-1).indices
    elif method == "topcol":
        iq = ik = torch.topk(qs + ks, k=r, dim=-1).indices
    else:
        raise ValueError(f"unknown init method {method!r}")
    aq = torch.gather(Q, -1, iq.expand(-1, -1, Q.shape[2], -1))
    ak = torch.gather(K, -1, ik.expand(-1, -1, K.shape[2], -1))
    return aq, ak


# ----------------------------------------------------------------------------
# A2: alternating least squares over the prompt  (lrqk_attention.py:312-423)
# ----------------------------------------------------------------------------
def _ls_right_factor(A: torch.Tensor, X: torch.Tensor) -> torch.Tensor:
    """B = (A^T A)^-1 A^T X  (:363-370, :416-421)."""
    return _solve_left(_t(A) @ A, _t(A) @ X)


def prefill_factorize(Q: torch.Tensor, K: torch.Tensor, A_Q: torch.Tensor, A_K: torch.Tensor,
                      max_iter: int, tol: float, return_sweeps: bool = False):
    """Unit-weight joint factorisation Q ~ A_Q B_Q, K ~ A_K B_K, A_Q A_K^T ~ Q K^T.

    One sweep (:359-413):
      B_Q, B_K  <- least squares against the current A factors            (:363-370)
      A_Q'      <- Q (K^T A_K + B_Q^T)(A_K^T A_K + B_Q B_Q^T)^-1          (:373-382)
      A_K'      <- K (Q^T A_Q' + B_K^T)(A_Q'^T A_Q' + B_K B_K^T)^-1       (:385-395)
      stop after the sweep if max(mse(A_Q,A_Q'), mse(A_K,A_K')) < tol     (:398-413)
    then B_Q, B_K are recomputed from the final A factors (:416-421).
    All tensors fp32 [B,H,S,*]; K already expanded to the query heads.
    """
    sweeps = 0
    for _ in range(max_iter):
        gram_k = _t(A_K) @ A_K
        B_Q = _solve_left(_t(A_Q) @ A_Q, _t(A_Q) @ Q)
        B_K = _solve_left(gram_k, _t(A_K) @ K)

        rhs_q = _t(K) @ A_K + _t(B_Q)
        new_A_Q = Q @ _solve_right(gram_k + B_Q @ _t(B_Q), rhs_q)

        gram_q = _t(new_A_Q) @ new_A_Q
        rhs_k = _t(Q) @ new_A_Q + _t(B_K)
        new_A_K = K @ _solve_right(gram_q + B_K @ _t(B_K), rhs_k)

        d_q = torch.nn.functional.mse_loss(A_Q, new_A_Q)
        d_k = torch.nn.functional.mse_loss(A_K, new_A_K)
        A_Q, A_K = new_A_Q, new_A_K
        sweeps += 1
        if max(d_q, d_k) < tol:
            break
    B_Q = _ls_right_factor(A_Q, Q)
    B_K = _ls_right_factor(A_K, K)
    if return_sweeps:
        return A_Q, B_Q, A_K, B_K, sweeps
    return A_Q, B_Q, A_K, B_K


def prefill_factorize_weighted(Q: torch.Tensor, K: torch.Tensor, A_Q: torch.Tensor, A_K: torch.Tensor,
                               lambda_q: float, lambda_k: float, max_iter: int, tol: float,
                               return_sweeps: bool = False):
    """The factorisation with weights lambda_Q, lambda_K on the two reconstruction terms
    (lrqk_attention.py:218-309), taken whenever either differs from 1 (:790-797).

    One sweep (:252-300) -- unlike the unit-weight form, BOTH left factors are renewed from the
    factors the sweep started with:
      B_Q, B_K  <- least squares against the current A factors                           (:256-263)
      A_Q'      <- Q (K^T A_K + lambda_Q B_Q^T)(A_K^T A_K + lambda_Q B_Q B_Q^T)^-1       (:266-274)
      A_K'      <- K (Q^T A_Q + lambda_K B_K^T)(A_Q^T A_Q + lambda_K B_K B_K^T)^-1       (:277-288)
      stop after the sweep if max(mse(A_Q,A_Q'), mse(A_K,A_K')) < tol                    (:291-300)
    then B_Q, B_K from the final A factors (:303-308).
    """
    sweeps = 0
    for _ in range(max_iter):
        gram_q = _t(A_Q) @ A_Q
        gram_k = _t(A_K) @ A_K
        B_Q = _solve_left(gram_q, _t(A_Q) @ Q)
        B_K = _solve_left(gram_k, _t(A_K) @ K)

        rhs_q = _t(K) @ A_K + lambda_q * _t(B_Q)
        new_A_Q = Q @ _solve_right(gram_k + lambda_q * (B_Q @ _t(B_Q)), rhs_q)

        rhs_k = _t(Q) @ A_Q + lambda_k * _t(B_K)
        new_A_K = K @ _solve_right(gram_q + lambda_k * (B_K @ _t(B_K)), rhs_k)

        delta = max(torch.nn.functional.mse_loss(A_Q, new_A_Q), torch.nn.functional.mse_loss(A_K, new_A_K))
        A_Q, A_K = new_A_Q, new_A_K
        sweeps += 1
        if delta < tol:
            break
    B_Q = _ls_right_factor(A_Q, Q)
    B_K = _ls_right_factor(A_K, K)
    if return_sweeps:
        return A_Q, B_Q, A_K, B_K, sweeps
    return A_Q, B_Q, A_K, B_K


def cast_prefill(Q: torch.Tensor, K: torch.Tensor, r: int, max_iter: int, tol: float,
                 init: str = "randn", init_factors_override=None, lambda_q: float = 1.0, lambda_k: float = 1.0):
    """fp32 up-cast, initial factors, factorisation (unit-weight form when both weights are 1,
    :790), results rounded to K's dtype: lrqk_attention.py:772-800."""
    out_dtype = K.dtype
    Q32, K32 = Q.to(torch.float32), K.to(torch.float32)
    if init_factors_override is not None:
        aq, ak = (t.to(torch.float32) for t in init_factors_override)
    else:
        aq, ak = init_factors(Q32, K32, r, init)
    if lambda_q == 1.0 and lambda_k == 1.0:
        out = prefill_factorize(Q32, K32, aq, ak, max_iter, tol)
    else:
        out = prefill_factorize_weighted(Q32, K32, aq, ak, lambda_q, lambda_k, max_iter, tol)
    return tuple(o.to(out_dtype) for o in out)


# ----------------------------------------------------------------------------
# A4: per-step rank-r projection and right-factor update  (lrqk_attention.py:522-665)
# ----------------------------------------------------------------------------
def _line_search_step(dB: torch.Tensor, x_hat: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """eta = |dB|^2 / (|x_hat dB|^2 + eps): lrqk_attention.py:651-665."""
    num = dB.square().sum(dim=(2, 3), keepdim=True)
    den = (x_hat @ dB).square().sum(dim=(2, 3), keepdim=True)
    return num / (den + eps)


def decode_project_update(B_Q: torch.Tensor, A_act: torch.Tensor, B_K: torch.Tensor,
                          K_act: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
                          max_iter: int, tol: float, return_iters: bool = False):
    """Unit-weight decode update (all fp32).

      B_Q,B_K [B,H,r,d]; A_act [B,H,n,r] rank-r rows of the active set; K_act [B,H,n,d]
      full keys of the active set; q,k [B,H,1,d].
    Shared terms (:555-565); k_hat0 = k B_K^T (B_K B_K^T)^-1 (:568-569); max(max_iter,1)
    alternations (:552, :572-609)
        q_hat = (q B_Q^T + (q K_act^T) A_act + (q k^T) k_hat)(B_Q B_Q^T + A_act^T A_act + k_hat^T k_hat)^-1
        k_hat'= (k B_K^T + (q k^T) q_hat)(B_K B_K^T + q_hat^T q_hat)^-1
    leaving the loop early once mse(k_hat, k_hat') < tol; then one gradient step
    on each right factor with the exact line-search step (:612-626).
    """
    max_iter = max(max_iter, 1)
    k_bk = k @ _t(B_K)
    gram_bk = B_K @ _t(B_K)
    q_rhs = q @ _t(B_Q) + (q @ _t(K_act)) @ A_act
    gram_q = B_Q @ _t(B_Q) + _t(A_act) @ A_act
    qk = q @ _t(k)

    k_hat = _solve_right(gram_bk, k_bk)
    iters = 0
    for _ in range(max_iter):
        q_hat = _solve_right(gram_q + _t(k_hat) @ k_hat, q_rhs + qk @ k_hat)
        new_k_hat = _solve_right(gram_bk + _t(q_hat) @ q_hat, k_bk + qk @ q_hat)
        delta = torch.nn.functional.mse_loss(k_hat, new_k_hat)
        k_hat = new_k_hat
        iters += 1
        if delta < tol:
            break

    dBQ = _t(q_hat) @ (q_hat @ B_Q - q)
    dBK = _t(k_hat) @ (k_hat @ B_K - k)
    B_Q = B_Q - _line_search_step(dBQ, q_hat) * dBQ
    B_K = B_K - _line_search_step(dBK, k_hat) * dBK
    if return_iters:
        return B_Q, B_K, q_hat, k_hat, iters
    return B_Q, B_K, q_hat, k_hat


def decode_project_update_weighted(B_Q: torch.Tensor, A_act: torch.Tensor, B_K: torch.Tensor,
                                   K_act: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
                                   lambda1: float, lambda2: float, max_iter: int, tol: float,
                                   return_iters: bool = False):
    """The decode update with weights (lrqk_attention.py:433-519), taken whenever either differs
    from 1 (:820-837): lambda2 weighs the active set's terms, lambda1 the new token's own
    q k^T term --
        q_hat = (q B_Q^T + l2 (q K_act^T) A_act + l1 (q k^T) k_hat)(B_Q B_Q^T + l2 A_act^T A_act + l1 k_hat^T k_hat)^-1
        k_hat'= (k B_K^T + l1 (q k^T) q_hat)(B_K B_K^T + l1 q_hat^T q_hat)^-1
    (:462-495); everything else as in the unit-weight form.
    """
    max_iter = max(max_iter, 1)
    k_bk = k @ _t(B_K)
    gram_bk = B_K @ _t(B_K)
    q_rhs = q @ _t(B_Q) + lambda2 * ((q @ _t(K_act)) @ A_act)
    gram_q = B_Q @ _t(B_Q) + lambda2 * (_t(A_act) @ A_act)
    qk = lambda1 * (q @ _t(k))

    k_hat = _solve_right(gram_bk, k_bk)
    iters = 0
    for _ in range(max_iter):
        q_hat = _solve_right(gram_q + lambda1 * (_t(k_hat) @ k_hat), q_rhs + qk @ k_hat)
        new_k_hat = _solve_right(gram_bk + lambda1 * (_t(q_hat) @ q_hat), k_bk + qk @ q_hat)
        delta = torch.nn.functional.mse_loss(k_hat, new_k_hat)
        k_hat = new_k_hat
        iters += 1
        if delta < tol:
            break

    dBQ = _t(q_hat) @ (q_hat @ B_Q - q)
    dBK = _t(k_hat) @ (k_hat @ B_K - k)
    B_Q = B_Q - _line_search_step(dBQ, q_hat) * dBQ
    B_K = B_K - _line_search_step(dBK, k_hat) * dBK
    if return_iters:
        return B_Q, B_K, q_hat, k_hat, iters
    return B_Q, B_K, q_hat, k_hat


def cast_decode(B_Q, A_act, B_K, K_act, q, k, max_iter: int, tol: float,
                lambda_dec_q: float = 1.0, lambda_dec_k: float = 1.0):
    """fp32 up-cast of every operand, update (unit-weight form when both weights are 1, :820),
    results rounded to k's dtype: lrqk_attention.py:803-839."""
    f = torch.float32
    ops = (B_Q.to(f), A_act.to(f), B_K.to(f), K_act.to(f), q.to(f), k.to(f))
    if lambda_dec_q == 1.0 and lambda_dec_k == 1.0:
        out = decode_project_update(*ops, max_iter, tol)
    else:
        out = decode_project_update_weighted(*ops, lambda_dec_q, lambda_dec_k, max_iter, tol)
    return tuple(o.to(k.dtype) for o in out)


# ----------------------------------------------------------------------------
# A6: proxy scores and top-k  (lrqk_attention.py:1235-1273)
# ----------------------------------------------------------------------------
def proxy_scores(A_K: torch.Tensor, q_hat: torch.Tensor) -> torch.Tensor:
    """fp32 scores [B,H,c] = A_K[B,H,c,r] . q_hat[B,H,1,r] (the matmul at :1260-1263,
    evaluated in fp32 from the stored -- possibly bf16 -- operands)."""
    return (A_K.to(torch.float32) @ _t(q_hat.to(torch.float32))).squeeze(-1)


def proxy_scores_lane_order(A_K: torch.Tensor, q_hat: torch.Tensor, lanes: int) -> np.ndarray:
    """Scores in the fixed fp32 summation order of the CUDA scoring kernel: the r columns are
    cut into `lanes` equal runs; within a run the even and the odd columns are summed
    separately, left to right starting from zero, and the two sums are added; the run sums
    are then combined by a butterfly (partner distance 1, 2, 4, ...).  Products of two bf16
    values are exact in fp32, and for fp32 operands a fused multiply-add is emulated in
    float64 (exact product, one rounding), so the order is reproducible bit for bit."""
    a = A_K.to(torch.float32).numpy()
    q = q_hat.to(torch.float32).numpy()
    *lead, c, r = a.shape
    per = r // lanes
    a64 = a.astype(np.float64).reshape(*lead, c, lanes, per)
    q64 = np.broadcast_to(q.astype(np.float64), a.shape).reshape(*lead, c, lanes, per)
    even = np.zeros(a64.shape[:-1], dtype=np.float32)
    odd = np.zeros(a64.shape[:-1], dtype=np.float32)
    for j in range(0, per, 2):
        even = (a64[..., j] * q64[..., j] + even.astype(np.float64)).astype(np.float32)
        odd = (a64[..., j + 1] * q64[..., j + 1] + odd.astype(np.float64)).astype(np.float32)
    run = (even + odd).astype(np.float32)
    dist = 1
    while dist < lanes:
        idx = np.arange(lanes) ^ dist
        run = (run + run[..., idx]).astype(np.float32)
        dist *= 2
    return run[..., 0]


def topk_sorted(scores, k: int) -> np.ndarray:
    """Positions of the k largest scores of each row, ascending; of equal scores the
    lower position wins (the reference's torch.topk + torch.sort at :1266-1272
    with the tie order pinned).  scores [..., c] -> int32 [..., k]."""
    s = np.ascontiguousarray(scores.numpy() if isinstance(scores, torch.Tensor) else scores, dtype=np.float32)
    lead, c = s.shape[:-1], s.shape[-1]
    s2 = s.reshape(-1, c)
    out = np.empty((s2.shape[0], k), dtype=np.int32)
    rc = clib().oracle_topk_sorted_f32(_ptr(s2), s2.shape[0], c, c, k, _ptr(out))
    if rc != 0:
        raise ValueError(f"oracle_topk_sorted_f32 failed ({rc}): k={k} c={c}")
    return out.reshape(*lead, k)


def topk_sorted_numpy(scores, k: int) -> np.ndarray:
    """Same contract as :func:`topk_sorted`, in numpy (stable sort of the negated
    scores; -0.0 and +0.0 compare equal)."""
    s = np.asarray(scores.numpy() if isinstance(scores, torch.Tensor) else scores, dtype=np.float32)
    order = np.argsort(-(s + np.float32(0.0)), axis=-1, kind="stable")[..., :k]
    return np.sort(order, axis=-1).astype(np.int32)


def select_reference_ops(A_K: torch.Tensor, q_hat: torch.Tensor, k: int) -> torch.Tensor:
    """The selection exactly as the reference evaluates it -- matmul in the tensors' own
    dtype, torch.topk, torch.sort (:1249-1273) -- used when pinning against the
    reference's traces and when timing the CPU baseline.  Returns int64 [B,H,k,1]
    (or arange when the candidate range is not longer than k, :1250-1258)."""
    b, h, c, _ = A_K.shape
    if c <= k:
        return torch.arange(0, c, dtype=torch.long).reshape(1, 1, -1, 1).expand(b, h, -1, 1)
    s = A_K @ _t(q_hat)
    return torch.sort(torch.topk(s, k=k, dim=2).indices, dim=2).values


# ----------------------------------------------------------------------------
# A7: hit/miss difference  (lrqk_attention.py:1275-1315)
# ----------------------------------------------------------------------------
def slot_diff_reference_ops(now: torch.Tensor, new: torch.Tensor):
    """The O(k^2) broadcast-compare form the reference runs (:1303-1315); now/new
    int64 [B,H,k,1] -> (updated [B,H,k,1], mask [B,H,k] bool)."""
    b, h = now.shape[:2]
    eq = now.view(b, h, -1, 1) == new.view(b, h, 1, -1)
    evict = ~eq.any(dim=3)
    absent = ~eq.any(dim=2)
    upd = now.clone()
    upd[evict] = new[absent]
    return upd, evict


def slot_diff(now: np.ndarray, new: np.ndarray):
    """Set form of the same update via the C twin.  now/new int32 [..., k] ->
    (updated int32 [..., k], mask uint8 [..., k], miss_count int32 [...])."""
    now = np.ascontiguousarray(now, dtype=np.int32)
    new = np.ascontiguousarray(new, dtype=np.int32)
    k = now.shape[-1]
    n = now.size // k
    upd = np.empty_like(now)
    mask = np.empty(now.shape, dtype=np.uint8)
    cnt = np.empty(now.shape[:-1], dtype=np.int32)
    rc = clib().oracle_slot_diff(_ptr(now), _ptr(new), n, k, _ptr(upd), _ptr(mask), _ptr(cnt))
    if rc != 0:
        raise ValueError("slot_diff: evicted and missing counts differ (duplicate entries?)")
    return upd, mask, cnt


def slot_diff_python(now, new):
    """Pure-Python form for one row (small cases): the docstring example at
    lrqk_attention.py:1279-1290 is now=[0,1,2,6,7], new=[0,2,4,5,6] ->
    updated=[0,4,2,6,5], mask=[0,1,0,0,1]."""
    new_set, now_set = set(int(x) for x in new), set(int(x) for x in now)
    missing = [int(x) for x in new if int(x) not in now_set]
    upd, mask, j = [], [], 0
    for x in now:
        if int(x) in new_set:
            upd.append(int(x)); mask.append(0)
        else:
            upd.append(missing[j]); mask.append(1); j += 1
    assert j == len(missing)
    return upd, mask


# ----------------------------------------------------------------------------
# A8/A9: row numbers and the host gather
# ----------------------------------------------------------------------------
def miss_rows(table: np.ndarray, mask: np.ndarray, kv_heads: int, groups: int, capacity: int) -> np.ndarray:
    """Linear rows of the missed entries, row-major over (b, kv head, group, slot):
    lrqk_attention.py:71-98; table/mask [B, kv_heads*groups, k]."""
    table = np.ascontiguousarray(table, dtype=np.int32)
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    b, _, k = table.shape
    out = np.empty(int(mask.sum()), dtype=np.int64)
    m = clib().oracle_miss_rows(_ptr(table), _ptr(mask), b, kv_heads, groups, k, capacity, _ptr(out))
    assert m == out.size
    return out


def gather_rows(src_flat: np.ndarray, rows: np.ndarray) -> np.ndarray:
    """dst[i] = src[rows[i]] by per-row memcpy: cpp_kernel/take_along_dim_grouped.cpp:133-183."""
    src_flat = np.ascontiguousarray(src_flat)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    out = np.empty((rows.size,) + src_flat.shape[1:], dtype=src_flat.dtype)
    rb = src_flat.dtype.itemsize * int(np.prod(src_flat.shape[1:]))
    clib().oracle_gather_rows(_ptr(out), _ptr(src_flat), _ptr(rows), rows.size, rb)
    return out


def take_along_dim_with_mask(src: np.ndarray, indices: np.ndarray, mask: np.ndarray) -> np.ndarray:
    """src [B,Hkv,S,w], indices/mask [B,Hkv,G,k] -> [sum(mask), w]:
    cpp_kernel/take_along_dim_grouped.cpp:13-124."""
    src = np.ascontiguousarray(src)
    indices = np.ascontiguousarray(indices, dtype=np.int64)
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    b, h, s, w = src.shape
    g, k = indices.shape[2:]
    out = np.empty((int(mask.sum()), w), dtype=src.dtype)
    m = clib().oracle_take_along_dim_with_mask(_ptr(out), _ptr(src), _ptr(indices), _ptr(mask),
                                               b, h, s, g, k, w * src.dtype.itemsize)
    assert m == out.shape[0]
    return out


# ----------------------------------------------------------------------------
# A12: exact attention over the resident rows
# ----------------------------------------------------------------------------
def attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
    """softmax(q K^T / sqrt(d)) V per query head over every resident row, fp32:
    what flash_attn_with_kvcache(q, k, v, causal=True) computes for one query
    (lrqk_attention.py:2326-2327).  q [B,H,1,d], K/V [B,H,n,d] -> [B,H,1,d] fp32."""
    q32, K32, V32 = q.to(torch.float32), K.to(torch.float32), V.to(torch.float32)
    s = (q32 @ _t(K32)) / math.sqrt(q.shape[-1])
    return torch.softmax(s, dim=-1) @ V32


# ----------------------------------------------------------------------------
# A3/A5/A11/A13: the per-layer engine  (lrqk_attention.py:1031-1613)
# ----------------------------------------------------------------------------
@dataclass
class StepTrace:
    q_hat: torch.Tensor = None
    k_hat: torch.Tensor = None
    candidates: int = 0
    wanted: np.ndarray = None       # ascending top-k before the diff, int32 [B,H,k]
    table: np.ndarray = None        # slot table after the diff, int32 [B,H,k]
    mask: np.ndarray = None         # uint8 [B,H,k]
    miss_rows: np.ndarray = None    # int64 [M]
    fetched: torch.Tensor = None    # [M, 2d]
    attn: torch.Tensor = None       # fp32 [B,H,1,d]


class OracleLayer:
    """State machine of one layer: mirrors LightAttentionIndicesFactory
    (lrqk_attention.py:1031-1613), both prompt branches: longer than k + m (:1467-1504) and
    k <= length <= k + m (:1444-1466, every prompt row resident, no selection until the
    context outgrows the resident rows).  A prompt of exactly k + m rows makes the reference
    itself fail at its first decode step (the ring write lands one slot past the ring); here the
    full ring is flushed to the host store at once, which is what :1192-1196 does when a decode
    step fills it.

    `faithful=True` evaluates selection and difference with the reference's own op
    sequence (torch.topk / broadcast compare); `faithful=False` uses the pinned tie
    rule and the set form.  Both agree whenever no two candidate scores are equal.
    """

    def __init__(self, r: int, k: int, m: int, groups: int, max_iter=(2, 2), tol=(1e-2, 1e-2),
                 capacity: int = 4096, init: str = "randn", scaling_ratio: float = 1.5,
                 faithful: bool = False, weights=(1.0, 1.0, 1.0, 1.0)):
        self.r, self.k, self.m, self.groups = r, k, m, groups
        # (lambda_Q, lambda_K, lambda_dec_q, lambda_dec_k): :1040, :1066-1072, used at :1435-1436, :1535-1536
        self.weights = (weights,) * 4 if isinstance(weights, float) else tuple(weights)
        self.max_iter = tuple(max_iter) if isinstance(max_iter, (tuple, list)) else (max_iter, max_iter)
        self.tol = tuple(tol) if isinstance(tol, (tuple, list)) else (tol, tol)
        self.capacity, self.init, self.scaling_ratio, self.faithful = capacity, init, scaling_ratio, faithful
        self.current_len = 0
        self.lite_len = 0
        self.lite_indices: List[int] = [-1] * m
        self.trace: List[StepTrace] = []

    # -- containers: zero-initialised growable stores (lrqk_attention.py:844-963) --
    def _first_capacity(self, length: int) -> int:
        return max(self.capacity, int(length * self.scaling_ratio))      # :880

    def _ensure(self, buf: torch.Tensor, used: int, extra: int) -> torch.Tensor:
        cap = buf.shape[2]
        if used + extra >= cap:                                          # :892-897
            new_cap = cap
            while new_cap <= used + extra:
                new_cap = int(new_cap * self.scaling_ratio)
            shape = list(buf.shape); shape[2] = new_cap
            grown = torch.zeros(shape, dtype=buf.dtype)                  # :913
            grown[:, :, :used] = buf[:, :, :used]
            return grown
        return buf

    # -- prefill: lrqk_attention.py:1385-1504 --
    def prefill(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, init_factors_override=None):
        b, hq, s, d = Q.shape
        assert s >= self.k, "seq_len must be larger than attn_topk"       # :1411
        Krep = expand_kv_heads(K, self.groups)
        self.Kres = torch.zeros((b, hq, self.k + self.m, d), dtype=Q.dtype)
        self.Vres = torch.zeros_like(self.Kres)
        self.current_len = s
        A_Q, B_Q, A_K, B_K = cast_prefill(Q, Krep, self.r, self.max_iter[0], self.tol[0], self.init,
                                          init_factors_override, self.weights[0], self.weights[1])
        self.B_Q, self.B_K = B_Q, B_K
        cap = self._first_capacity(s)
        self.A_K = torch.zeros((b, hq, cap, self.r), dtype=A_K.dtype)
        self.A_K[:, :, :s] = A_K
        self.a_len = s
        self.A_Q_last = A_Q[:, :, -1:, :]
        if s <= self.k + self.m:                                         # :1444-1466
            kk, rem = self.k, s - self.k
            hcap = self._first_capacity(kk)
            self.host = torch.zeros((b, K.shape[1], hcap, 2 * d), dtype=K.dtype)
            self.host[:, :, :kk] = torch.cat([K[:, :, :kk], V[:, :, :kk]], dim=-1)
            self.host_len = kk
            self.lite_len = rem
            self.lite_indices = list(range(kk, kk + rem)) + [-1] * (self.m - rem)
            self.Kres[:, :, :s] = Krep
            self.Vres[:, :, :s] = expand_kv_heads(V, self.groups)
            self.table = np.broadcast_to(np.arange(kk, dtype=np.int32), (b, hq, kk)).copy()
            if rem >= self.m:                                            # see the class docstring
                g = self.groups
                self._host_append(torch.cat([self.Kres[:, ::g, kk:kk + self.m], self.Vres[:, ::g, kk:kk + self.m]], dim=-1))
                self.lite_len = 0
            return self
        self.host = torch.zeros((b, K.shape[1], cap, 2 * d), dtype=K.dtype)
        self.host[:, :, :s] = torch.cat([K, V], dim=-1)                  # :962, :1469
        self.host_len = s
        cand = s - self.m                                                # :1473
        wanted = self._select(A_K[:, :, :cand], self.A_Q_last)
        self.table = wanted.copy()
        idx = torch.from_numpy(wanted.astype(np.int64))[..., None].expand(-1, -1, -1, d)
        self.Kres[:, :, :self.k] = torch.gather(Krep, 2, idx)            # :1339-1351
        self.Vres[:, :, :self.k] = torch.gather(expand_kv_heads(V, self.groups), 2, idx)
        self.lite_indices = list(range(s - self.m, s))                   # :1493-1504
        self.lite_len = 0
        self.Kres[:, :, self.k:] = Krep[:, :, s - self.m:]
        self.Vres[:, :, self.k:] = expand_kv_heads(V, self.groups)[:, :, s - self.m:]
        return self

    def _select(self, A_cand: torch.Tensor, q_hat: torch.Tensor) -> np.ndarray:
        if self.faithful:
            return select_reference_ops(A_cand, q_hat, self.k)[..., 0].numpy().astype(np.int32)
        return topk_sorted(proxy_scores(A_cand, q_hat), self.k)

    def _host_append(self, rows: torch.Tensor):
        n = rows.shape[2]
        self.host = self._ensure(self.host, self.host_len, n)
        self.host[:, :, self.host_len:self.host_len + n] = rows
        self.host_len += n

    # -- one decode step: lrqk_attention.py:1506-1613 --
    def decode(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, want_attention: bool = True):
        kk, m, g = self.k, self.m, self.groups
        d = q.shape[-1]
        tr = StepTrace()
        # lite ring write, :1174-1196
        slot = kk + self.lite_len
        self.Kres[:, :, slot:slot + 1] = expand_kv_heads(k, g)
        self.Vres[:, :, slot:slot + 1] = expand_kv_heads(v, g)
        self.lite_indices[self.lite_len] = self.current_len
        self.lite_len += 1
        self.current_len += 1
        if self.lite_len >= m:
            ring = torch.cat([self.Kres[:, ::g, kk:kk + m], self.Vres[:, ::g, kk:kk + m]], dim=-1)
            self._host_append(ring)
            self.lite_len = 0
        if self.current_len <= kk + m:                                   # :1526-1545
            # every token is still resident: project against all earlier rows, no selection
            n = self.current_len - 1
            B_Q, B_K, q_hat, k_hat = cast_decode(self.B_Q, self.A_K[:, :, :self.a_len], self.B_K, self.Kres[:, :, :n],
                                                 q, expand_kv_heads(k, g), self.max_iter[1], self.tol[1],
                                                 self.weights[2], self.weights[3])
            self.B_Q, self.B_K = B_Q, B_K
            self.A_K = self._ensure(self.A_K, self.a_len, 1)
            self.A_K[:, :, self.a_len:self.a_len + 1] = k_hat
            self.a_len += 1
            tr.q_hat, tr.k_hat, tr.candidates = q_hat, k_hat, -1
            tr.table = self.table
            Kv, Vv = self.Kres[:, :, :self.current_len], self.Vres[:, :, :self.current_len]
            if want_attention:
                tr.attn = attention(q, Kv, Vv)
            self.trace.append(tr)
            return Kv, Vv
        # rank-r rows of the active set out of the zero-initialised store, :1156-1171
        act = np.concatenate([self.table, np.broadcast_to(np.asarray(self.lite_indices, dtype=np.int32),
                                                          self.table.shape[:2] + (m,))], axis=-1)
        idx = torch.from_numpy(act.astype(np.int64))[..., None].expand(-1, -1, -1, self.r)
        A_act = torch.gather(self.A_K, 2, idx)
        B_Q, B_K, q_hat, k_hat = cast_decode(self.B_Q, A_act, self.B_K, self.Kres, q, expand_kv_heads(k, g),
                                             self.max_iter[1], self.tol[1], self.weights[2], self.weights[3])
        self.B_Q, self.B_K = B_Q, B_K
        self.A_K = self._ensure(self.A_K, self.a_len, 1)
        self.A_K[:, :, self.a_len:self.a_len + 1] = k_hat               # :1231
        self.a_len += 1
        tr.q_hat, tr.k_hat = q_hat, k_hat
        # candidates, selection, difference, :1562-1573
        cand = self.lite_indices[self.lite_len] - 1
        tr.candidates = cand
        if cand <= kk:                                                   # :1247-1255: nothing to choose from yet
            wanted = np.broadcast_to(np.arange(cand, dtype=np.int32), self.table.shape[:2] + (cand,)).copy()
        else:
            wanted = self._select(self.A_K[:, :, :cand], q_hat)
        if self.faithful:
            upd, msk = slot_diff_reference_ops(torch.from_numpy(self.table.astype(np.int64))[..., None],
                                               torch.from_numpy(wanted.astype(np.int64))[..., None])
            table, mask = upd[..., 0].numpy().astype(np.int32), msk.numpy().astype(np.uint8)
        else:
            table, mask, _ = slot_diff(self.table, wanted)
        self.table = table
        tr.wanted, tr.table, tr.mask = wanted, table, mask
        # fetch of the misses from the host store into the evicted slots, :1575-1608
        rows = miss_rows(table, mask, k.shape[1], g, self.host.shape[2])
        flat = self.host.view(-1, 2 * d)
        fetched = flat[torch.from_numpy(rows)]
        tr.miss_rows, tr.fetched = rows, fetched
        if fetched.numel() > 0:
            bm = torch.from_numpy(mask.astype(bool))
            self.Kres[:, :, :kk][bm] = fetched[:, :d]
            self.Vres[:, :, :kk][bm] = fetched[:, d:]
        if want_attention:
            tr.attn = attention(q, self.Kres, self.Vres)
        self.trace.append(tr)
        return self.Kres, self.Vres


# ----------------------------------------------------------------------------
# seeded synthetic inputs shared by the oracle, the tests and the benchmark
# ----------------------------------------------------------------------------
def make_prompt(seed: int, bsz: int, hq: int, hkv: int, seq: int, d: int = 128, latent: int = 32,
                noise: float = 0.1, dtype=torch.float32):
    """Keys of approximate rank `latent` plus noise, K = U W + noise*E per KV head with
    U~N(0,1), W~N(0,1/latent), E~N(0,1); values and prompt queries ~N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    U = torch.randn(bsz, hkv, seq, latent, generator=g)
    W = torch.randn(bsz, hkv, latent, d, generator=g) / math.sqrt(latent)
    E = torch.randn(bsz, hkv, seq, d, generator=g)
    K = U @ W + noise * E
    V = torch.randn(bsz, hkv, seq, d, generator=g)
    Q = torch.randn(bsz, hq, seq, d, generator=g)
    return Q.to(dtype), K.to(dtype), V.to(dtype)


def make_step(seed: int, step: int, bsz: int, hq: int, hkv: int, d: int = 128, dtype=torch.float32):
    """One decode step's q [B,Hq,1,d], k, v [B,Hkv,1,d] ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed * 1000003 + 7919 * (step + 1))
    q = torch.randn(bsz, hq, 1, d, generator=g)
    k = torch.randn(bsz, hkv, 1, d, generator=g)
    v = torch.randn(bsz, hkv, 1, d, generator=g)
    return q.to(dtype), k.to(dtype), v.to(dtype)
