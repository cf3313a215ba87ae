"""Device-side state of one layer and thin wrappers over the C-ABI operators.

``LayerState`` owns the tensors a ``LightAttentionIndicesFactory`` keeps in the
reference (lrqk_attention.py:1052-1111) -- the rank-r key factors ``A_K``, the
right factors ``B_Q``/``B_K``, the resident keys/values, the slot table and the
page-locked host K|V store -- and the ``lrqk_layer`` struct that points at them.
torch is used for device memory and streams only; every computation is a call
into ``liblrqk_sm100.so``.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib

_DTYPES = {torch.float32: _lib.LRQK_F32, torch.bfloat16: _lib.LRQK_BF16}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as a cudaStream_t.  (torch.cuda.current_stream() costs
    ~15 us of Python per call -- a third of a decode step's host time; the raw accessor, where this torch has
    it, a fraction of a microsecond.)"""
    if _raw_stream is not None:
        return C.c_void_p(_raw_stream(torch.cuda.current_device()))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# Page-locked buffers released by closed stores, kept for the next store of the same size: pinning
# half a gigabyte takes a fifth of a second, far longer than the prompt kernels of a layer.
_HOST_POOL: dict = {}
_HOST_POOL_BYTES = 0
HOST_POOL_LIMIT_BYTES = 64 << 30


def release_host_pool() -> None:
    """Give the pooled page-locked buffers back to the system."""
    global _HOST_POOL_BYTES
    for bufs in _HOST_POOL.values():
        for ptr in bufs:
            _lib.lib().lrqk_host_free(C.c_void_p(ptr))
    _HOST_POOL.clear()
    _HOST_POOL_BYTES = 0


class HostStore:
    """Page-locked, device-mapped host buffer [B, Hkv, capacity, 2d] holding K|V rows
    (the reference's pinned AutoIncreaseTensorSharedKV, lrqk_attention.py:959-963, :1088-1094).

    The reference's store is zero-initialised (:888).  ``zero=True`` clears the whole buffer on the
    host; a caller that is about to overwrite the first rows anyway passes ``zero=False`` and clears
    only the rest with :meth:`zero_rows_from` (clearing 0.5 GB on one core costs more than every
    prompt kernel of the layer together)."""

    def __init__(self, bsz: int, kv_heads: int, capacity: int, head_dim: int, dtype: torch.dtype, zero: bool = True):
        global _HOST_POOL_BYTES
        self.shape = (bsz, kv_heads, capacity, 2 * head_dim)
        self.dtype = dtype
        self.nbytes = int(np.prod(self.shape)) * torch.empty((), dtype=dtype).element_size()
        pooled = _HOST_POOL.get(self.nbytes)
        fresh = not pooled
        if pooled:
            self.host_ptr = pooled.pop()
            _HOST_POOL_BYTES -= self.nbytes
        else:
            hp = C.c_void_p()
            _lib.check(_lib.lib().lrqk_host_alloc(C.byref(hp), self.nbytes), "lrqk_host_alloc")
            self.host_ptr = hp.value                   # comes zero-filled
        dp = C.c_void_p()
        _lib.check(_lib.lib().lrqk_host_device_ptr(C.c_void_p(self.host_ptr), C.byref(dp)), "lrqk_host_device_ptr")
        self.device_ptr = dp.value
        raw = (C.c_uint8 * self.nbytes).from_address(self.host_ptr)
        self._raw = raw
        self.data = torch.frombuffer(raw, dtype=torch.uint8).view(dtype).view(self.shape)
        self._fresh = fresh
        if zero and not fresh:
            self.data.zero_()  # a pooled buffer still holds its previous contents
        self.current_len = 0

    def zero_rows_from(self, row: int) -> None:
        """Clear rows [row, capacity) of every (batch, KV head) on the host."""
        if row < self.capacity and not self._fresh:
            self.data[:, :, row:].zero_()

    @property
    def capacity(self) -> int:
        return self.shape[2]

    def close(self):
        global _HOST_POOL_BYTES
        if getattr(self, "host_ptr", None):
            self.data = None
            self._raw = None
            if _HOST_POOL_BYTES + self.nbytes <= HOST_POOL_LIMIT_BYTES:
                _HOST_POOL.setdefault(self.nbytes, []).append(self.host_ptr)
                _HOST_POOL_BYTES += self.nbytes
            else:
                _lib.lib().lrqk_host_free(C.c_void_p(self.host_ptr))
            self.host_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_SAME_DEVICE = contextlib.nullcontext()


def on_device(device: torch.device):
    """Context in which `device` is the current CUDA device (nothing to do when it already is).  Every entry
    of the library launches on the CURRENT device, so state that lives on another one must make it current."""
    if device.index is None or torch.cuda.current_device() == device.index:
        return _SAME_DEVICE
    return torch.cuda.device(device)


class LayerState:
    def __init__(self, bsz: int, q_heads: int, kv_heads: int, head_dim: int, r: int, k: int, m: int,
                 a_capacity: int, host_capacity: int, dtype: torch.dtype, device="cuda", max_iter: int = 2,
                 with_host: bool = True, zero_host: bool = True,
                 weights: Tuple[float, float, float, float] = (1.0, 1.0, 1.0, 1.0)):
        if dtype not in _DTYPES:
            raise ValueError(f"unsupported dtype {dtype}: the kernels take float32 or bfloat16")
        if not torch.cuda.is_available():
            raise RuntimeError("lrqk_b200 needs a CUDA device (sm_100); there is no CPU path")
        self.lib = _lib.lib()
        self.weights = tuple(float(w) for w in weights)  # lambda_Q, lambda_K, lambda_dec_q, lambda_dec_k
        if len(self.weights) != 4 or any(not (0.0 <= w < float("inf")) for w in self.weights):
            raise ValueError("weights: four finite, non-negative numbers")
        self.bsz, self.q_heads, self.kv_heads, self.head_dim = bsz, q_heads, kv_heads, head_dim
        self.r, self.k, self.m = r, k, m
        self.dtype, self.device = dtype, torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        n = bsz * q_heads
        z = dict(dtype=dtype, device=self.device)
        self.A_K = torch.zeros((bsz, q_heads, a_capacity, r), **z)          # zero-initialised (:888)
        self.B_Q = torch.zeros((bsz, q_heads, r, head_dim), **z)
        self.B_K = torch.zeros((bsz, q_heads, r, head_dim), **z)
        self.K_res = torch.zeros((bsz, q_heads, k + m, head_dim), **z)      # (:1417-1426)
        self.V_res = torch.zeros((bsz, q_heads, k + m, head_dim), **z)
        self.table = torch.zeros((bsz, q_heads, k), dtype=torch.int32, device=self.device)
        self.lite_pos = torch.full((m,), -1, dtype=torch.int32, device=self.device)
        self.host = HostStore(bsz, kv_heads, host_capacity, head_dim, dtype, zero=zero_host) if with_host else None
        # per-step outputs and scratch
        self.q_hat = torch.zeros((bsz, q_heads, r), **z)
        self.wanted = torch.zeros((bsz, q_heads, k), dtype=torch.int32, device=self.device)
        self.mask = torch.zeros((bsz, q_heads, k), dtype=torch.uint8, device=self.device)
        self.miss_count = torch.zeros((bsz, q_heads), dtype=torch.int32, device=self.device)
        self.miss_list = torch.zeros((n * k, 3), dtype=torch.int32, device=self.device)
        self.counters = torch.zeros((4,), dtype=torch.int32, device=self.device)
        self.attn_out = torch.zeros((bsz, q_heads, head_dim), **z)
        self._rebuild_struct()
        self.max_iter_ws = max(1, max_iter)
        nb = self.lib.lrqk_decode_project_update_workspace_bytes(C.byref(self.c), self.max_iter_ws)
        self.project_ws = torch.zeros((max(nb, 16),), dtype=torch.uint8, device=self.device)
        nb = self.lib.lrqk_flash_decode_workspace_bytes(C.byref(self.c), k + m)
        self.attn_ws = torch.zeros((max(nb, 16),), dtype=torch.uint8, device=self.device)
        self._step_args = None
        self._qkv_in = None
        self._size_score_ws()

    def _size_score_ws(self):
        """Scratch of the scoring stage's two-kernel plan (few heads); empty where one kernel is the plan."""
        nb = self.lib.lrqk_score_topk_workspace_bytes(C.byref(self.c), self.A_K.shape[2])
        self.score_ws = torch.empty((nb,), dtype=torch.uint8, device=self.device) if nb else None
        self._step_args = None

    def _rebuild_struct(self):
        c = _lib.Layer()
        c.dtype = _DTYPES[self.dtype]
        c.bsz, c.q_heads, c.kv_heads, c.head_dim = self.bsz, self.q_heads, self.kv_heads, self.head_dim
        c.r, c.k, c.m = self.r, self.k, self.m
        c.a_capacity = self.A_K.shape[2]
        c.host_capacity = self.host.capacity if self.host is not None else 0
        c.A_K, c.B_Q, c.B_K = self.A_K.data_ptr(), self.B_Q.data_ptr(), self.B_K.data_ptr()
        c.K_res, c.V_res = self.K_res.data_ptr(), self.V_res.data_ptr()
        c.table, c.lite_pos = self.table.data_ptr(), self.lite_pos.data_ptr()
        c.host_kv = self.host.device_ptr if self.host is not None else None
        c.weights[:] = self.weights
        self.c = c

    # ---- operators -------------------------------------------------------------------------
    def _chk(self, t: torch.Tensor, shape, name: str):
        if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous() or tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: expected contiguous {self.dtype} CUDA tensor of shape {tuple(shape)}, "
                             f"got {t.dtype} {tuple(t.shape)} on {t.device}")

    def lite_append(self, k_new, v_new, lite_slot: int, position: int, flush_rows: int = 0, host_row: int = 0):
        self._chk(k_new, (self.bsz, self.kv_heads, self.head_dim), "k_new")
        self._chk(v_new, (self.bsz, self.kv_heads, self.head_dim), "v_new")
        _lib.check(self.lib.lrqk_lite_append(C.byref(self.c), _ptr(k_new), _ptr(v_new), lite_slot, position,
                                             flush_rows, host_row, _stream()), "lrqk_lite_append")

    def project_update(self, q, k_new, max_iter: int, tol: float, append_row: int):
        self._chk(q, (self.bsz, self.q_heads, self.head_dim), "q")
        self._chk(k_new, (self.bsz, self.kv_heads, self.head_dim), "k_new")
        if max(1, max_iter) > self.max_iter_ws:
            raise ValueError("max_iter exceeds the workspace this state was sized for")
        _lib.check(self.lib.lrqk_decode_project_update(
            C.byref(self.c), _ptr(q), _ptr(k_new), max_iter, tol, append_row, _ptr(self.q_hat),
            C.c_void_p(self.counters.data_ptr() + 8), _ptr(self.project_ws), _stream()),
            "lrqk_decode_project_update")
        return self.q_hat

    def project(self, q, k_new, max_iter: int, append_row: int):
        """First half of ``project_update``: the alternating solves; every alternation's iterates stay in the
        projection workspace (nothing else is written)."""
        self._chk(q, (self.bsz, self.q_heads, self.head_dim), "q")
        self._chk(k_new, (self.bsz, self.kv_heads, self.head_dim), "k_new")
        if max(1, max_iter) > self.max_iter_ws:
            raise ValueError("max_iter exceeds the workspace this state was sized for")
        _lib.check(self.lib.lrqk_decode_project(C.byref(self.c), _ptr(q), _ptr(k_new), max_iter, append_row,
                                                _ptr(self.q_hat), _ptr(self.project_ws), _stream()), "lrqk_decode_project")

    def update(self, q, k_new, max_iter: int, tol: float, append_row: int):
        """Second half: early-exit decision, ``B_Q``/``B_K``, ``q_hat`` and the new row of ``A_K`` from the iterates
        ``project`` left."""
        self._chk(q, (self.bsz, self.q_heads, self.head_dim), "q")
        self._chk(k_new, (self.bsz, self.kv_heads, self.head_dim), "k_new")
        _lib.check(self.lib.lrqk_decode_update(
            C.byref(self.c), _ptr(q), _ptr(k_new), max_iter, tol, append_row, _ptr(self.q_hat),
            C.c_void_p(self.counters.data_ptr() + 8), _ptr(self.project_ws), _stream()), "lrqk_decode_update")
        return self.q_hat

    def score_topk(self, q_hat, candidates: int, scores_out: Optional[torch.Tensor] = None):
        self._chk(q_hat, (self.bsz, self.q_heads, self.r), "q_hat")
        stride = 0
        if scores_out is not None:
            assert scores_out.dtype == torch.float32 and scores_out.is_contiguous()
            stride = scores_out.shape[-1]
        ws = self.score_ws
        _lib.check(self.lib.lrqk_score_topk(C.byref(self.c), _ptr(q_hat), candidates, _ptr(self.wanted),
                                            _ptr(scores_out), stride, _ptr(ws), 0 if ws is None else ws.numel(),
                                            _stream()), "lrqk_score_topk")
        return self.wanted

    def slot_diff(self, wanted: Optional[torch.Tensor] = None):
        wanted = self.wanted if wanted is None else wanted
        self.counters[:2].zero_()
        _lib.check(self.lib.lrqk_slot_diff(C.byref(self.c), _ptr(wanted), _ptr(self.mask), _ptr(self.miss_count),
                                           _ptr(self.miss_list), _ptr(self.counters),
                                           C.c_void_p(self.counters.data_ptr() + 4), _stream()), "lrqk_slot_diff")
        return self.mask

    def miss_gather(self):
        _lib.check(self.lib.lrqk_miss_gather(C.byref(self.c), _ptr(self.miss_list), _ptr(self.counters), _stream()),
                   "lrqk_miss_gather")

    def flash_decode(self, q, rows: Optional[int] = None, scale: Optional[float] = None, exchange=None):
        """Attention over the first `rows` resident rows; with `exchange` (a sharding.HeadExchange) the
        kernel's epilogue also stores the rows into every rank's exchange buffer."""
        self._chk(q, (self.bsz, self.q_heads, self.head_dim), "q")
        rows = self.k + self.m if rows is None else rows
        scale = self.head_dim ** -0.5 if scale is None else scale
        if exchange is not None:
            _lib.check(self.lib.lrqk_flash_decode_push(C.byref(self.c), _ptr(q), _ptr(self.attn_out), rows, scale,
                                                       _ptr(self.attn_ws), C.byref(exchange.c), exchange.seq.next_push(),
                                                       _stream()), "lrqk_flash_decode_push")
            return self.attn_out
        _lib.check(self.lib.lrqk_flash_decode(C.byref(self.c), _ptr(q), _ptr(self.attn_out), rows, scale,
                                              _ptr(self.attn_ws), _stream()), "lrqk_flash_decode")
        return self.attn_out

    def fetch_attend(self, q, scale: Optional[float] = None, exchange=None):
        """``miss_gather()`` followed by ``flash_decode(q)`` as ONE kernel: the threads that attend to a slot
        whose mask byte is set read that row from the host store themselves (and refill the slot on the
        side).  Same results bit for bit."""
        self._chk(q, (self.bsz, self.q_heads, self.head_dim), "q")
        scale = self.head_dim ** -0.5 if scale is None else scale
        peers, seq = (None, 0) if exchange is None else (C.byref(exchange.c), exchange.seq.next_push())
        _lib.check(self.lib.lrqk_fetch_attend(C.byref(self.c), _ptr(self.mask), _ptr(q), _ptr(self.attn_out), scale,
                                              _ptr(self.attn_ws), peers, seq, _stream()), "lrqk_fetch_attend")
        return self.attn_out

    def make_step_args(self, q, k_new, v_new, lite_slot: int, position: int, flush_rows: int, host_row: int,
                       candidates: int, max_iter: int, tol: float, scale: Optional[float] = None,
                       attention: bool = True) -> _lib.StepArgs:
        a = self._step_args
        if a is None:                      # the buffers below live as long as the state: fill them in once
            a = self._step_args = _lib.StepArgs()
            a.q_hat, a.wanted, a.mask = self.q_hat.data_ptr(), self.wanted.data_ptr(), self.mask.data_ptr()
            a.miss_count, a.miss_list = self.miss_count.data_ptr(), self.miss_list.data_ptr()
            a.counters = self.counters.data_ptr()
            a.project_workspace, a.attn_workspace = self.project_ws.data_ptr(), self.attn_ws.data_ptr()
            a.score_workspace = None if self.score_ws is None else self.score_ws.data_ptr()
            a.score_workspace_bytes = 0 if self.score_ws is None else self.score_ws.numel()
            self._attn_out_ptr, self._default_scale = self.attn_out.data_ptr(), self.head_dim ** -0.5
        a.q, a.k_new, a.v_new = q.data_ptr(), k_new.data_ptr(), v_new.data_ptr()
        a.attn_out = self._attn_out_ptr if attention else None
        a.lite_slot, a.position, a.flush_rows, a.host_row = lite_slot, position, flush_rows, host_row
        a.candidates, a.max_iter, a.tol = candidates, max_iter, tol
        a.scale = self._default_scale if scale is None else scale
        a.peers, a.push_seq = None, 0
        return a

    def layer_step(self, args: _lib.StepArgs):
        _lib.check(self.lib.lrqk_layer_step(C.byref(self.c), C.byref(args), _stream()), "lrqk_layer_step")

    def rope_qkv(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, bsz: int, q_heads: int, kv_heads: int,
                 b0: int = 0, kvh0: int = 0):
        """Split the fused projection of one new token per sequence (qkv [bsz, 1, (q_heads + 2 kv_heads) d] of
        the WHOLE model) into this state's heads -- batch entries b0.., KV heads kvh0.. -- and rotate q and k by
        cos, sin ([bsz or 1, 1, d]).  Returns views [B,Hq,1,d], [B,Hkv,1,d], [B,Hkv,1,d] of buffers that the next
        call overwrites."""
        d = self.head_dim
        if self._qkv_in is None:
            z = dict(dtype=self.dtype, device=self.device)
            self._qkv_in = (torch.empty((self.bsz, self.q_heads, d), **z), torch.empty((self.bsz, self.kv_heads, d), **z),
                            torch.empty((self.bsz, self.kv_heads, d), **z))
        self._chk(qkv, (bsz, 1, (q_heads + 2 * kv_heads) * d), "qkv")
        rows = cos.shape[0]
        self._chk(cos, (rows, 1, d), "cos")
        self._chk(sin, (rows, 1, d), "sin")
        q, k, v = self._qkv_in
        _lib.check(self.lib.lrqk_rope_qkv(_ptr(qkv), _ptr(cos), _ptr(sin), rows, _DTYPES[self.dtype], bsz, q_heads, kv_heads,
                                          d, b0, self.bsz, kvh0, self.kv_heads, _ptr(q), _ptr(k), _ptr(v), _stream()),
                   "lrqk_rope_qkv")
        return q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2)

    def kv_pack_host(self, keys, values, host_row: int = 0):
        s = keys.shape[2]
        self._chk(keys, (self.bsz, self.kv_heads, s, self.head_dim), "keys")
        self._chk(values, (self.bsz, self.kv_heads, s, self.head_dim), "values")
        _lib.check(self.lib.lrqk_kv_pack_host(C.byref(self.c), _ptr(keys), _ptr(values), s, host_row, _stream()),
                   "lrqk_kv_pack_host")

    def fill_resident(self, keys, values):
        s = keys.shape[2]
        self._chk(keys, (self.bsz, self.kv_heads, s, self.head_dim), "keys")
        self._chk(values, (self.bsz, self.kv_heads, s, self.head_dim), "values")
        _lib.check(self.lib.lrqk_prefill_fill_resident(C.byref(self.c), _ptr(keys), _ptr(values), s, _stream()),
                   "lrqk_prefill_fill_resident")

    # ---- device-side status words ----------------------------------------------------------
    def status_words(self) -> torch.Tensor:
        """int32 [3] (a fresh device tensor): the hit/miss difference's mismatch flag, the attention kernel's
        and the projection kernel's bounded-wait words (LRQK_ETIMEOUT when a wait ran out)."""
        attn = self.attn_ws.view(torch.int32)[self.bsz * self.q_heads]
        proj = self.project_ws.view(torch.int32)[(self.project_ws.numel() - 16) // 4]
        return torch.stack([self.counters[1], attn, proj])

    def check_status(self) -> None:
        """Synchronising check of the words above; raises LrqkError for the first that is set."""
        diff, attn, proj = (int(x) for x in self.status_words().tolist())
        if diff != 0:
            raise _lib.LrqkError(_lib.EINVAL, "lrqk_slot_diff", "a head's evicted and missing counts differ "
                                 "(the wanted set holds duplicates or the slot table is corrupt)")
        for code, where in ((attn, "lrqk_flash_decode"), (proj, "lrqk_decode_project_update")):
            if code != 0:
                raise _lib.LrqkError(code, where, self.lib.lrqk_strerror(code).decode())

    def close(self):
        if self.host is not None:
            torch.cuda.synchronize()
            self.host.close()
            self.host = None
