"""Host-side mirror of the reference's ``lrqk_attention`` module for the decode path.

Same class names, constructor arguments, defaults and return conventions as the reference
(paths below are relative to its checkout):

* ``InitAQAK``                         -- lrqk_attention.py:140-143
* ``AutoIncreaseTensor`` (+ ``SharedKV``), ``PreAllocatedTensor``, ``_CacheQKV``
                                       -- lrqk_attention.py:844-1028
* ``LightAttentionIndicesFactory``     -- lrqk_attention.py:1031-1613
* ``LightAttentionIndicesNoHitMiss``   -- lrqk_attention.py:1683-1775
* ``DynamicLRQKCache``                 -- lrqk_attention.py:1778-1970

What differs is where the work happens: every numerical or data-moving stage is a CUDA kernel
of ``liblrqk_sm100.so`` working on pre-allocated state (``LayerState``); Python keeps only the
integer bookkeeping the reference also keeps in Python (ring slot, lengths, candidate count).
A decode step performs no host synchronisation.  There is no CPU path: without a CUDA device
the constructors of the compute classes raise.
"""
from __future__ import annotations

import ctypes as C
import enum
from collections import defaultdict
from typing import Dict, List, Optional, Tuple, Union

import torch

from . import _lib
from .state import HostStore, LayerState, _ptr, _stream, on_device

try:  # HF is only needed for the Cache base class
    from transformers import cache_utils as _cache_utils
    _CacheBase = _cache_utils.Cache
except Exception:  # pragma: no cover
    _cache_utils = None
    _CacheBase = object


def _pair(x):
    if isinstance(x, (tuple, list)):
        if len(x) != 2:
            raise AssertionError("must be a tuple or list of length 2")
        return tuple(x)
    return (x, x)


class InitAQAK(enum.Enum):
    randn = enum.auto()
    top = enum.auto()
    topcol = enum.auto()


def _resolve_init(method: Union[InitAQAK, str]) -> InitAQAK:
    if isinstance(method, str):
        if method not in InitAQAK.__members__:
            raise ValueError(f"Unknown init_method: {method}. Current support {list(InitAQAK.__members__.keys())}")
        return InitAQAK[method]
    if not isinstance(method, InitAQAK):
        raise ValueError(f"Unknown init_method: {method}")
    return method


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,Hkv,S,d] -> [B,Hkv*n_rep,S,d] (view-expand then reshape), as HF's repeat_kv."""
    if n_rep == 1:
        return x
    b, h, s, d = x.shape
    return x[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)


# ------------------------------------------------------------------------------------------------
# containers
# ------------------------------------------------------------------------------------------------
class AutoIncreaseTensor:
    """Growable, zero-initialised tensor along one axis (lrqk_attention.py:844-956): first
    allocation ``max(capacity, int(len * scaling_ratio))``, later growth by ``scaling_ratio``
    until the data fits, new space zeroed."""

    def __init__(self, capacity: int = 4096, dim: int = 0, scaling_ratio: float = 1.5,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None,
                 pin_memory: bool = False):
        self.capacity, self.dim, self.scaling_ratio = capacity, dim, scaling_ratio
        self.device, self.dtype, self.pin_memory = device, dtype, pin_memory
        self.data: Optional[torch.Tensor] = None
        self.current_len = 0

    def _alloc(self, shape):
        pin = self.pin_memory and torch.cuda.is_available()
        return torch.zeros(shape, device=self.device, dtype=self.dtype, pin_memory=pin)

    def reserve(self, target_length: int) -> bool:
        """Make room for `target_length` entries; True if the buffer was reallocated."""
        if self.data is None or target_length < self.capacity:
            return False
        new_cap = self.capacity
        while new_cap <= target_length:
            new_cap = int(new_cap * self.scaling_ratio)
        shape = list(self.data.shape)
        shape[self.dim] = new_cap
        grown = self._alloc(shape)
        grown.narrow(self.dim, 0, self.current_len).copy_(self.data.narrow(self.dim, 0, self.current_len))
        self.data, self.capacity = grown, new_cap
        return True

    @torch.no_grad()
    def append(self, x: torch.Tensor):
        if self.device is None:
            self.device = x.device
        if self.dtype is None:
            self.dtype = x.dtype
        length = x.size(self.dim)
        if self.data is None:
            cap = max(self.capacity, int(length * self.scaling_ratio))
            shape = list(x.shape)
            shape[self.dim] = cap
            self.data, self.capacity = self._alloc(shape), cap
        else:
            self.reserve(self.current_len + length)
        self.data.narrow(self.dim, self.current_len, length).copy_(x.to(self.device, self.dtype))
        self.current_len += length

    def has_data(self):
        return self.data is not None

    @property
    def shape(self) -> torch.Size:
        s = list(self.data.shape)
        s[self.dim] = self.current_len
        return torch.Size(s)

    def tensor(self) -> torch.Tensor:
        return self.data.narrow(self.dim, 0, self.current_len)

    def __len__(self):
        return self.current_len

    def __getitem__(self, idx):
        if self.data is None:
            raise IndexError("Cache is empty")
        return self.tensor()[idx]

    def take_along_dim(self, indices: torch.Tensor, dim: int = None, out=None) -> torch.Tensor:
        if self.data is None:
            raise IndexError("Cache is empty")
        return torch.take_along_dim(self.data, indices, self.dim if dim is None else dim, out=out)


class AutoIncreaseTensorSharedKV(AutoIncreaseTensor):
    """K and V concatenated on the last axis (lrqk_attention.py:959-963)."""

    def append(self, k: torch.Tensor, v: torch.Tensor):
        return super().append(torch.cat([k, v], dim=-1))


class PreAllocatedTensor:
    """Fixed-capacity tensor for prompts shorter than the active set (lrqk_attention.py:966-1011)."""

    def __init__(self, capacity: int, dim: int, dtype: torch.dtype = None, device: torch.device = None):
        self.capacity, self.dim, self.dtype, self.device = capacity, dim, dtype, device
        self.data = None
        self.current_len = 0

    @classmethod
    def from_tensor(cls, capacity: int, dim: int, data: torch.Tensor):
        out = cls(capacity, dim, data.dtype, data.device)
        out.append(data)
        return out

    def append(self, x: torch.Tensor):
        self.dtype = x.dtype if self.dtype is None else self.dtype
        self.device = x.device if self.device is None else self.device
        n = x.shape[self.dim]
        if self.data is None:
            shape = list(x.shape)
            shape[self.dim] = self.capacity
            self.data = torch.empty(shape, dtype=self.dtype, device=self.device)
        if self.current_len + n > self.capacity:
            raise ValueError("Not enough capacity to store the tensor")
        self.data.narrow(self.dim, self.current_len, n).copy_(x)
        self.current_len += n

    def has_data(self):
        return self.data is not None

    def tensor(self) -> torch.Tensor:
        return self.data.narrow(self.dim, 0, self.current_len)

    def __len__(self):
        return self.current_len

    def __getitem__(self, idx):
        return self.tensor()[idx]


class _CacheQKV:
    def __init__(self, capacity: int, dim: int, dtype: torch.dtype = None, device: torch.device = None):
        self.Q = PreAllocatedTensor(capacity, dim, dtype, device)
        self.K = PreAllocatedTensor(capacity, dim, dtype, device)
        self.V = PreAllocatedTensor(capacity, dim, dtype, device)

    def append(self, Q, K, V):
        self.Q.append(Q)
        self.K.append(K)
        self.V.append(V)
        return self.Q.tensor(), self.K.tensor(), self.V.tensor()

    def __len__(self):
        return self.Q.current_len


class _HostKVView:
    """What the reference exposes as ``factory.KVcpu``: ``.data`` [B,Hkv,capacity,2d] in
    page-locked host memory and the filled length."""

    def __init__(self, store: HostStore):
        self._store = store

    @property
    def data(self) -> torch.Tensor:
        return self._store.data

    @property
    def current_len(self) -> int:
        return self._store.current_len

    @property
    def capacity(self) -> int:
        return self._store.capacity

    def tensor(self) -> torch.Tensor:
        return self._store.data.narrow(2, 0, self._store.current_len)

    def __len__(self):
        return self._store.current_len


# ------------------------------------------------------------------------------------------------
# the per-layer engine
# ------------------------------------------------------------------------------------------------
class LightAttentionIndicesFactory:
    """Per-layer selection engine: lrqk_attention.py:1031-1613.

    ``prefill(q, k, v)`` factorises the prompt, stores K|V in page-locked host memory, selects
    the first resident set and fills the lite ring.  ``decode(q, k, v)`` performs one step and
    returns the resident ``(K, V)`` of shape [B,Hq,k+m,d] exactly like the reference;
    ``decode_attend`` additionally runs the attention kernel and returns its output, which is
    what the patched attention modules use.

    ``weights`` = (lambda_Q, lambda_K, lambda_dec_q, lambda_dec_k) as in the reference (:1040,
    :1435-1436, :1535-1536): with either weight of a pair different from 1 the prompt factorisation /
    the decode projection take the reference's general forms (:218-309 / :433-519), which the same
    kernels evaluate.

    Prompts of ``attn_topk .. attn_topk + num_lite_tokens`` rows take the reference's short branch
    (:1444-1466): every prompt row stays resident (slot = position), nothing is selected, and decode
    steps project against all earlier rows (:1526-1545) until the context outgrows the resident rows.
    The same kernels serve it: lite slots that hold no token yet point at a row of ``A_K`` that is
    still zero, so they add nothing to any sum.  A prompt of exactly ``attn_topk + num_lite_tokens``
    rows makes the reference fail at its first decode step (its ring write lands one slot past the
    ring); here the full ring is flushed to the host store at once, as a decode step that fills it
    would (:1192-1196).
    """

    def __init__(self, num_lite_tokens: int = 1, attn_topk: int = 128, num_key_value_groups: int = 1,
                 r: int = 16, max_iter: Union[int, Tuple[int, int]] = 2,
                 tol: Union[float, Tuple[float, float]] = 1e-4,
                 weights: Tuple[float, float, float, float] = (1.0, 1.0, 1.0, 1.0), capacity: int = 4096,
                 init_aq_ak_method: Union[InitAQAK, str] = InitAQAK.randn, scaling_ratio: float = 1.5,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        self.num_lite_tokens, self.attn_topk, self.dim = num_lite_tokens, attn_topk, 2
        self.num_key_value_groups, self.r = num_key_value_groups, r
        self.max_iter, self.tol = _pair(max_iter), _pair(tol)
        self.init_aq_ak_method = init_aq_ak_method
        self.gpu_capacity = attn_topk + num_lite_tokens
        self.prefill_length = 0
        self.current_len = 0
        if isinstance(weights, float):
            weights = (weights,) * 4
        if not isinstance(weights, tuple) or len(weights) != 4:
            raise ValueError("weights must be a float or a tuple of length 4")
        if any(not (0.0 <= float(w) < float("inf")) for w in weights):
            raise ValueError("weights must be finite and non-negative")
        self.weights = tuple(float(w) for w in weights)
        self.capacity, self.scaling_ratio = capacity, scaling_ratio
        self.device, self.dtype = device, dtype
        self.lite_len = 0
        self.lite_indices: List[int] = [-1] * num_lite_tokens
        self.resident_rows = self.gpu_capacity           # rows of Kgpu/Vgpu the last decode step attended to
        self.state: Optional[LayerState] = None
        self.verbose = False
        self._hook = type(self).only_indices_in_cpu is not LightAttentionIndicesFactory.only_indices_in_cpu

    # ---- views on the device state (names as in the reference) ---------------------------------
    def __len__(self):
        return self.current_len

    @property
    def Kgpu(self):
        return None if self.state is None else self.state.K_res

    @property
    def Vgpu(self):
        return None if self.state is None else self.state.V_res

    @property
    def B_Q(self):
        return None if self.state is None else self.state.B_Q

    @property
    def B_K(self):
        return None if self.state is None else self.state.B_K

    @property
    def A_K(self):
        return self.state.A_K.narrow(2, 0, self.current_len)

    @property
    def KVcpu(self):
        self._await_host_store(on_host=True)
        return _HostKVView(self.state.host)

    @property
    def hit_indices(self) -> Optional[torch.Tensor]:
        """int64 [B,Hq,k,1], the position held by each selected slot (a copy of the device table)."""
        return None if self.state is None else self.state.table.to(torch.int64).unsqueeze(-1)

    @property
    def Klite(self):
        return self.Kgpu[:, ::self.num_key_value_groups, self.attn_topk:self.gpu_capacity, :]

    @property
    def Vlite(self):
        return self.Vgpu[:, ::self.num_key_value_groups, self.attn_topk:self.gpu_capacity, :]

    # ---- selection primitives kept callable, as in the reference -----------------------------------
    def compute_hit_indices(self, query_states: torch.Tensor, key_states: torch.Tensor) -> torch.Tensor:
        """Ascending top-k positions of key_states . query_states (lrqk_attention.py:1235-1273).
        query_states [B,H,1,r]; key_states [B,H,c,r] must be a prefix view of this layer's A_K."""
        st = self.state
        b, h, c, _ = key_states.shape
        if c <= self.attn_topk:
            return torch.arange(0, c, device=query_states.device, dtype=torch.long).reshape(1, 1, -1, 1).expand(b, h, -1, 1)
        if key_states.data_ptr() != st.A_K.data_ptr():
            raise ValueError("compute_hit_indices scores this layer's own A_K buffer")
        st.score_topk(query_states.reshape(b, h, self.r).contiguous(), c)
        return st.wanted.to(torch.int64).unsqueeze(-1)

    def only_indices_in_cpu(self, now_indices: torch.Tensor, new_indices: torch.Tensor):
        """Set difference of the wanted positions against the resident ones
        (lrqk_attention.py:1275-1315): returns (updated_indices, mask of refilled slots).
        Subclasses may override it (the reference's hit-rate counter does); the fused step then
        falls back to calling this method between the kernels."""
        st = self.state
        saved = st.table.clone()
        st.table.copy_(now_indices.reshape(st.table.shape).to(torch.int32))
        st.slot_diff(new_indices.reshape(st.table.shape).to(torch.int32).contiguous())
        updated = st.table.to(torch.int64).reshape(now_indices.shape)
        mask = st.mask.to(torch.bool).clone()
        st.table.copy_(saved)
        return updated, mask

    # ---- prefill --------------------------------------------------------------------------------
    def _initial_factors(self, Q: torch.Tensor, K: torch.Tensor):
        """fp32 [B,Hq,S,r] starting factors (lrqk_attention.py:145-209); K is per KV head here and
        is expanded only for the column gathers."""
        method = _resolve_init(self.init_aq_ak_method)
        b, hq, s, d = Q.shape
        if method == InitAQAK.randn:
            aq = torch.randn((b, hq, s, self.r), dtype=torch.float32, device=Q.device)
            ak = torch.randn((b, hq, s, self.r), dtype=torch.float32, device=Q.device)
            return aq, ak
        g = self.num_key_value_groups
        qs = Q.float().abs().sum(dim=2, keepdim=True)
        ks = repeat_kv(K.float().abs().sum(dim=2, keepdim=True), g)
        if method == InitAQAK.top:
            iq = torch.topk(qs, k=self.r, dim=-1).indices
            ik = torch.topk(ks, k=self.r, dim=-1).indices
        else:
            iq = ik = torch.topk(qs + ks, k=self.r, dim=-1).indices
        aq = torch.gather(Q, -1, iq.expand(-1, -1, s, -1)).float()
        ik_kv = ik.view(b, K.shape[1], g, 1, self.r)
        ak = torch.gather(K[:, :, None].expand(-1, -1, g, -1, -1), -1, ik_kv.expand(-1, -1, -1, s, -1))
        return aq.contiguous(), ak.reshape(b, hq, s, self.r).float().contiguous()

    def _new_state(self, bsz, hq, hkv, d, seq_len, dtype, device) -> LayerState:
        cap = max(self.capacity, int(seq_len * self.scaling_ratio))   # first allocation, :880
        # the first seq_len rows of the host store are written by the prompt copy: clear only the rest
        st = LayerState(bsz, hq, hkv, d, self.r, self.attn_topk, self.num_lite_tokens, a_capacity=cap,
                        host_capacity=cap, dtype=dtype, device=device, max_iter=self.max_iter[1], zero_host=False,
                        weights=self.weights)
        st.host.zero_rows_from(seq_len)
        return st

    _side_streams: Dict[torch.device, "torch.cuda.Stream"] = {}

    @classmethod
    def _side_stream(cls, device) -> "torch.cuda.Stream":
        device = torch.device(device)
        if device not in cls._side_streams:
            cls._side_streams[device] = torch.cuda.Stream(device=device)
        return cls._side_streams[device]

    @torch.no_grad()
    def prefill(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor):
        with on_device(query_states.device):
            return self._prefill(query_states, key_states, value_states)

    def _prefill(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor):
        bsz, hq, seq_len, d = query_states.shape
        hkv = key_states.shape[1]
        assert seq_len >= self.attn_topk, "seq_len must be larger than attn_topk"
        if hq != hkv * self.num_key_value_groups:
            raise ValueError("num_key_value_groups does not match the head counts of q and k")
        q = query_states.contiguous()
        k = key_states.contiguous()
        v = value_states.contiguous()
        if seq_len <= self.gpu_capacity:
            return self._prefill_short(q, k, v)
        st = self.state = self._new_state(bsz, hq, hkv, d, seq_len, q.dtype, q.device)
        self.prefill_length = self.current_len = seq_len
        # the prompt's K|V rows go to the page-locked host store on a second stream: that copy is bound
        # by the host link and overlaps the factorisation, which is bound by HBM and the tensor cores
        main, side = torch.cuda.current_stream(), self._side_stream(q.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            st.kv_pack_host(k, v, 0)
        k.record_stream(side)
        v.record_stream(side)
        a_q_last = self._factorize(st, q, k, seq_len)
        st.host.current_len = seq_len
        st.score_topk(a_q_last, seq_len - self.num_lite_tokens)       # candidates 0 .. S-m-1, :1471-1474
        st.table.copy_(st.wanted)
        st.fill_resident(k, v)
        self.lite_indices = list(range(seq_len - self.num_lite_tokens, seq_len))
        self.lite_len = 0
        # The copy to the host store may still be running when this returns: nothing on the main stream reads the
        # store before the layer's first decode step, which waits for this event (as does any host-side look at
        # KVcpu), so the copy also overlaps whatever the caller enqueues next -- the next layer's prompt pass.
        self._host_ready = torch.cuda.Event()
        self._host_ready.record(side)

    def _await_host_store(self, on_host: bool):
        """Order what follows after the prompt's copy into the host store: the current stream waits
        (``on_host=False``), or the calling thread does."""
        ev = getattr(self, "_host_ready", None)
        if ev is not None:
            if on_host:
                ev.synchronize()
            else:
                torch.cuda.current_stream().wait_event(ev)
            self._host_ready = None

    def _factorize(self, st: LayerState, q, k, seq_len: int) -> torch.Tensor:
        """Prompt factorisation into st.A_K[:seq_len], st.B_Q, st.B_K; returns the last row of A_Q."""
        aq, ak = self._initial_factors(q, k)
        nb = st.lib.lrqk_prefill_factorize_workspace_bytes(C.byref(st.c), seq_len)
        ws = torch.empty((max(nb, 16),), dtype=torch.uint8, device=q.device)
        a_q_last = torch.empty((q.shape[0], q.shape[1], self.r), dtype=q.dtype, device=q.device)
        _lib.check(st.lib.lrqk_prefill_factorize(C.byref(st.c), _ptr(q), _ptr(k), _ptr(aq), _ptr(ak), seq_len,
                                                 self.max_iter[0], self.tol[0], _ptr(a_q_last), None, _ptr(ws),
                                                 _stream()), "lrqk_prefill_factorize")
        return a_q_last

    def _prefill_short(self, q, k, v):
        """attn_topk <= seq_len <= attn_topk + num_lite_tokens (lrqk_attention.py:1444-1466): the first
        attn_topk rows go to the host store, ALL rows stay resident in position order, the slot table
        is 0..attn_topk-1 and the remaining rows are the first entries of the lite ring."""
        bsz, hq, seq_len, d = q.shape
        hkv, kk, m, g = k.shape[1], self.attn_topk, self.num_lite_tokens, self.num_key_value_groups
        # host capacity follows the rows it is first given (:880): the first attn_topk rows
        cap_a = max(self.capacity, int(seq_len * self.scaling_ratio), self.gpu_capacity + 2)
        cap_h = max(self.capacity, int(kk * self.scaling_ratio), self.gpu_capacity + 2)
        st = self.state = LayerState(bsz, hq, hkv, d, self.r, kk, m, a_capacity=cap_a, host_capacity=cap_h,
                                     dtype=q.dtype, device=q.device, max_iter=self.max_iter[1], zero_host=True,
                                     weights=self.weights)
        self.prefill_length = self.current_len = seq_len
        self._factorize(st, q, k, seq_len)
        st.kv_pack_host(k[:, :, :kk].contiguous(), v[:, :, :kk].contiguous(), 0)
        st.host.current_len = kk
        st.K_res[:, :, :seq_len].copy_(repeat_kv(k, g))
        st.V_res[:, :, :seq_len].copy_(repeat_kv(v, g))
        st.table.copy_(torch.arange(kk, dtype=torch.int32, device=q.device).expand(bsz, hq, kk))
        rem = seq_len - kk
        self.lite_len = rem
        self.lite_indices = list(range(kk, kk + rem)) + [-1] * (m - rem)
        # device copy of the ring positions: an empty slot points at row attn_topk + num_lite_tokens of
        # A_K, which stays zero until every slot has been filled (that position is appended last)
        st.lite_pos.copy_(torch.tensor([p if p >= 0 else self.gpu_capacity for p in self.lite_indices],
                                       dtype=torch.int32))
        if rem >= m:      # full ring: flush it now (the reference fails here, see the class docstring)
            ring = torch.cat([st.K_res[:, ::g, kk:kk + m], st.V_res[:, ::g, kk:kk + m]], dim=-1)
            torch.cuda.current_stream().synchronize()
            st.host.data[:, :, kk:kk + m].copy_(ring)
            st.host.current_len = kk + m
            self.lite_len = 0

    def load_state(self, *, A_K, B_Q, B_K, keys, values, table, dtype=None):
        """Adopt factors and a first resident set produced elsewhere (same layout as after
        ``prefill``): A_K [B,Hq,S,r], B_Q/B_K [B,Hq,r,d], keys/values [B,Hkv,S,d] on the device,
        table int [B,Hq,k] ascending.  Fills the host store, the slots and the lite ring."""
        bsz, hq, seq_len, _ = A_K.shape
        hkv, d = keys.shape[1], keys.shape[3]
        dtype = keys.dtype if dtype is None else dtype
        st = self.state = self._new_state(bsz, hq, hkv, d, seq_len, dtype, keys.device)
        self.prefill_length = self.current_len = seq_len
        st.A_K[:, :, :seq_len].copy_(A_K)
        st.B_Q.copy_(B_Q)
        st.B_K.copy_(B_K)
        st.table.copy_(table)
        k, v = keys.to(dtype).contiguous(), values.to(dtype).contiguous()
        st.kv_pack_host(k, v, 0)
        st.host.current_len = seq_len
        st.fill_resident(k, v)
        self.lite_indices = list(range(seq_len - self.num_lite_tokens, seq_len))
        self.lite_len = 0

    # ---- save / resume ----------------------------------------------------------------------------
    # (The reference keeps no cache state across runs; this is the dump a serving host needs to park a long
    # context and pick it up again.)
    def state_dict(self) -> dict:
        """Everything ``load_state_dict`` needs to go on decoding bit for bit: the rank-r key factors of all
        tokens so far, the right factors, the resident rows, slot table and ring positions, the filled rows of
        the host store, and the host-side counters.  Tensors are CPU copies (this call synchronises)."""
        st = self.state
        if st is None:
            raise RuntimeError("nothing to save before prefill")
        self._await_host_store(on_host=True)
        with on_device(st.device):
            torch.cuda.synchronize()
        rows = st.host.current_len
        return {
            "format": 1,
            "shape": dict(bsz=st.bsz, q_heads=st.q_heads, kv_heads=st.kv_heads, head_dim=st.head_dim, r=st.r,
                          k=st.k, m=st.m, a_capacity=st.A_K.shape[2], host_capacity=st.host.capacity,
                          dtype=str(st.dtype).replace("torch.", ""), weights=list(st.weights)),
            "counters": dict(current_len=self.current_len, prefill_length=self.prefill_length, lite_len=self.lite_len,
                             lite_indices=list(self.lite_indices), resident_rows=self.resident_rows, host_len=rows),
            "A_K": st.A_K[:, :, :self.current_len].cpu(), "B_Q": st.B_Q.cpu(), "B_K": st.B_K.cpu(),
            "K_res": st.K_res.cpu(), "V_res": st.V_res.cpu(), "table": st.table.cpu(), "lite_pos": st.lite_pos.cpu(),
            "host": st.host.data[:, :, :rows].clone(),
        }

    def load_state_dict(self, sd: dict, device=None) -> None:
        """Rebuild the layer from ``state_dict()`` output on ``device`` (default: this factory's, else the
        current CUDA device).  The factory must have been built with the same ``attn_topk``, ``num_lite_tokens``,
        ``r`` and ``num_key_value_groups``."""
        if sd.get("format") != 1:
            raise ValueError("not a state this version wrote")
        sh, c = sd["shape"], sd["counters"]
        if (sh["k"], sh["m"], sh["r"]) != (self.attn_topk, self.num_lite_tokens, self.r) or \
                sh["q_heads"] != sh["kv_heads"] * self.num_key_value_groups:
            raise ValueError("the saved state was produced with other settings (attn_topk, num_lite_tokens, r, groups)")
        if tuple(float(w) for w in sh["weights"]) != tuple(self.weights):
            raise ValueError("the saved state was produced with other weights")
        dtype = getattr(torch, sh["dtype"])
        device = torch.device(device if device is not None else (self.device if self.device is not None else "cuda"))
        if self.state is not None:
            self.close()
        with on_device(device if device.index is not None else torch.device("cuda", torch.cuda.current_device())):
            st = self.state = LayerState(sh["bsz"], sh["q_heads"], sh["kv_heads"], sh["head_dim"], sh["r"], sh["k"], sh["m"],
                                         a_capacity=sh["a_capacity"], host_capacity=sh["host_capacity"], dtype=dtype,
                                         device=device, max_iter=self.max_iter[1], zero_host=True, weights=self.weights)
            st.A_K[:, :, :c["current_len"]].copy_(sd["A_K"])
            for name in ("B_Q", "B_K", "K_res", "V_res", "table", "lite_pos"):
                getattr(st, name).copy_(sd[name])
            st.host.data[:, :, :c["host_len"]].copy_(sd["host"])
            st.host.current_len = c["host_len"]
            torch.cuda.synchronize()
        self.current_len, self.prefill_length = c["current_len"], c["prefill_length"]
        self.lite_len, self.lite_indices = c["lite_len"], list(c["lite_indices"])
        self.resident_rows = c["resident_rows"]

    # ---- decode ---------------------------------------------------------------------------------
    def _reserve(self):
        st = self.state
        if self.current_len + 1 >= st.A_K.shape[2]:                     # growth rule, :892-897
            new_cap = st.A_K.shape[2]
            while new_cap <= self.current_len + 1:
                new_cap = int(new_cap * self.scaling_ratio)
            grown = torch.zeros((st.bsz, st.q_heads, new_cap, st.r), dtype=st.dtype, device=st.device)
            grown[:, :, :self.current_len].copy_(st.A_K[:, :, :self.current_len])
            st.A_K = grown
            st._rebuild_struct()
            st._size_score_ws()
        if st.host.current_len + self.num_lite_tokens >= st.host.capacity:
            torch.cuda.synchronize()
            new_cap = st.host.capacity
            while new_cap <= st.host.current_len + self.num_lite_tokens:
                new_cap = int(new_cap * self.scaling_ratio)
            new = HostStore(st.bsz, st.kv_heads, new_cap, st.head_dim, st.dtype)
            new.data[:, :, :st.host.current_len].copy_(st.host.data[:, :, :st.host.current_len])
            new.current_len = st.host.current_len
            st.host.close()
            st.host = new
            st._rebuild_struct()

    def _step_counters(self):
        """Advance the Python-side counters exactly as _append does (lrqk_attention.py:1174-1196)
        and derive the candidate count of this step (:1562-1568)."""
        m = self.num_lite_tokens
        slot, position = self.lite_len, self.current_len
        self.lite_indices[slot] = position
        self.lite_len += 1
        self.current_len += 1
        flush_rows, host_row = 0, self.state.host.current_len
        if self.lite_len >= m:
            flush_rows = m
            self.state.host.current_len += m
            self.lite_len = 0
        candidates = self.lite_indices[self.lite_len] - 1
        return slot, position, flush_rows, host_row, candidates

    def _flat(self, x: torch.Tensor, heads: int) -> torch.Tensor:
        st = self.state
        if x.shape[0] != st.bsz or x.shape[1] != heads or x.shape[-1] != st.head_dim or x.numel() != st.bsz * heads * st.head_dim:
            raise ValueError(f"decode expects [B,{heads},1,{st.head_dim}], got {tuple(x.shape)}")
        return x.reshape(st.bsz, heads, st.head_dim).contiguous()

    @torch.no_grad()
    def _decode(self, query_states, key_states, value_states, attention: bool, exchange=None):
        st = self.state
        if st is None:
            raise RuntimeError("decode before prefill")
        if query_states.device != st.device:
            raise ValueError(f"this layer's state lives on {st.device}, the step's tensors on {query_states.device}")
        with on_device(st.device):
            return self._decode_on_device(query_states, key_states, value_states, attention, exchange)

    def _decode_on_device(self, query_states, key_states, value_states, attention: bool, exchange=None):
        st = self.state
        self._await_host_store(on_host=False)
        self._reserve()
        q = self._flat(query_states.to(st.dtype), st.q_heads)
        k = self._flat(key_states.to(st.dtype), st.kv_heads)
        v = self._flat(value_states.to(st.dtype), st.kv_heads)
        slot, position, flush_rows, host_row, candidates = self._step_counters()
        self.resident_rows = self.gpu_capacity
        if self.current_len <= self.gpu_capacity or candidates <= self.attn_topk:
            # Every token is still resident (lrqk_attention.py:1526-1545), or the context has just outgrown
            # the resident rows and there are no more candidates than slots yet (:1247-1255): ring write and
            # projection only, nothing to select or fetch.  Empty ring slots are zero rows (see prefill).
            st.lite_append(k, v, slot, position, flush_rows, host_row)
            st.project_update(q, k, self.max_iter[1], self.tol[1], position)
            st.mask.zero_()
            st.miss_count.zero_()
            self.resident_rows = min(self.current_len, self.gpu_capacity)
            if attention:
                st.flash_decode(q, rows=self.resident_rows, exchange=exchange)
            return st
        if not self._hook:
            args = st.make_step_args(q, k, v, slot, position, flush_rows, host_row, candidates,
                                     self.max_iter[1], self.tol[1], attention=attention)
            if exchange is not None:      # push, and the wait for all ranks' rows, in the same call
                args.peers, args.push_seq = exchange.struct_ptr(), exchange.seq.next_push()
                args.gathered_out, args.wait_status = exchange.gathered.data_ptr(), exchange.status.data_ptr()
                exchange.seq.next_wait()
            else:
                args.gathered_out = args.wait_status = None
            st.layer_step(args)
        else:
            if exchange is not None:
                raise NotImplementedError("the stage-by-stage path does not push to other ranks")
            # a subclass observes or replaces the difference: run the stages one by one
            st.lite_append(k, v, slot, position, flush_rows, host_row)
            st.project_update(q, k, self.max_iter[1], self.tol[1], position)
            st.score_topk(st.q_hat, candidates)
            now = st.table.to(torch.int64).unsqueeze(-1)
            new = st.wanted.to(torch.int64).unsqueeze(-1)
            updated, mask = self.only_indices_in_cpu(now, new)
            mask = mask.reshape(st.table.shape)
            st.table.copy_(updated.reshape(st.table.shape).to(torch.int32))
            st.mask.copy_(mask.to(torch.uint8))
            idx = mask.reshape(-1, st.k).nonzero()
            n = idx.shape[0]
            st.miss_list[:n, 0] = idx[:, 0].int()
            st.miss_list[:n, 1] = idx[:, 1].int()
            st.miss_list[:n, 2] = st.table.reshape(-1, st.k)[idx[:, 0], idx[:, 1]]
            st.counters[0] = n
            st.miss_gather()
            if attention:
                st.flash_decode(q)
        return st

    def decode(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor):
        """One step; returns the resident (K, V) [B,Hq,k+m,d] (lrqk_attention.py:1506-1613)."""
        st = self._decode(query_states, key_states, value_states, attention=False)
        if self.resident_rows < self.gpu_capacity:           # short prompt: the filled rows only, :1541-1544
            return st.K_res.narrow(2, 0, self.resident_rows), st.V_res.narrow(2, 0, self.resident_rows)
        return st.K_res, st.V_res

    def decode_attend(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                      ) -> torch.Tensor:
        """One step including the attention over the resident rows; returns [B,Hq,1,d] (a view
        of a buffer that the next step overwrites)."""
        st = self._decode(query_states, key_states, value_states, attention=True)
        return st.attn_out.unsqueeze(2)

    def decode_attend_push(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                           exchange) -> torch.Tensor:
        """decode_attend for a head-sharded layer: the attention kernel also stores this rank's rows
        into every rank's exchange buffer (``exchange``: a sharding.HeadExchange), and the same call
        enqueues the bounded wait for all ranks' rows, which are then in ``exchange.gathered``
        ([world, heads_per_rank, d]); ``exchange.rows()`` returns them."""
        st = self._decode(query_states, key_states, value_states, attention=True, exchange=exchange)
        return st.attn_out.unsqueeze(2)

    def miss_counts(self) -> torch.Tensor:
        """int32 [B,Hq]: slots refilled by the last step (device tensor; reading it synchronises)."""
        return self.state.miss_count

    def close(self):
        if self.state is not None:
            self._await_host_store(on_host=True)
            self.state.close()
            self.state = None


def cast_lrqk_prefill(Q: torch.Tensor, K: torch.Tensor, r: int, lambda_Q: float = 1.0, lambda_K: float = 1.0,
                      max_iter: int = 8, tol: float = 1e-5, init_method: Union[InitAQAK, str] = InitAQAK.randn):
    """The reference's functional form of the prompt factorisation (lrqk_attention.py:772-800) on the prompt
    kernels: ``Q, K`` [B,H,S,d] (``K`` already repeated to the query heads, as the reference passes it).  Returns
    ``(A_Q, B_Q, A_K, B_K)`` in ``K``'s dtype; the full ``A_Q``, which the kernels never materialise, is one
    library product ``Q X_Q`` with the d x r map the factorisation leaves.  A convenience (scratch state per call)."""
    bsz, heads, seq_len, d = Q.shape
    dtype = K.dtype
    if max_iter > 8:
        raise ValueError("at most 8 sweeps")
    with on_device(K.device):
        st = LayerState(bsz, heads, heads, d, r, 1, 1, a_capacity=seq_len, host_capacity=1, dtype=dtype, device=K.device,
                        with_host=False, weights=(float(lambda_Q), float(lambda_K), 1.0, 1.0))
        try:
            fac = LightAttentionIndicesFactory(r=r, init_aq_ak_method=init_method, num_key_value_groups=1)
            q, k = Q.to(dtype).contiguous(), K.to(dtype).contiguous()
            aq, ak = fac._initial_factors(q, k)
            nb = st.lib.lrqk_prefill_factorize_workspace_bytes(C.byref(st.c), seq_len)
            ws = torch.empty((max(nb, 16),), dtype=torch.uint8, device=K.device)
            last = torch.empty((bsz, heads, r), dtype=dtype, device=K.device)
            n_sw = torch.zeros(1, dtype=torch.int32, device=K.device)
            sweeps = max(1, max_iter)
            _lib.check(st.lib.lrqk_prefill_factorize(C.byref(st.c), _ptr(q), _ptr(k), _ptr(aq), _ptr(ak), seq_len, sweeps,
                                                     tol, _ptr(last), _ptr(n_sw), _ptr(ws), _stream()), "lrqk_prefill_factorize")
            x_q = torch.empty((bsz, heads, d, r), dtype=torch.float32, device=K.device)
            _lib.check(st.lib.lrqk_prefill_factor_maps(C.byref(st.c), seq_len, sweeps, _ptr(n_sw), _ptr(ws), _ptr(x_q), None,
                                                       _stream()), "lrqk_prefill_factor_maps")
            A_Q = (q.float() @ x_q).to(dtype)
            out = (A_Q, st.B_Q.clone(), st.A_K[:, :, :seq_len].clone(), st.B_K.clone())
        finally:
            st.close()
    return out


def cast_lrqk_decode(B_Q: torch.Tensor, A_K: torch.Tensor, B_K: torch.Tensor, K__: torch.Tensor, q: torch.Tensor,
                     k: torch.Tensor, lambda_dec_q: float = 1.0, lambda_dec_k: float = 1.0, max_iter: int = 8,
                     tol: float = 1e-5):
    """The reference's functional form of the decode projection (lrqk_attention.py:803-839) on the projection
    kernel: ``B_Q, B_K`` [B,H,r,d]; ``A_K`` [B,H,n,r] and ``K__`` [B,H,n,d], the rank-r rows and the keys of the
    active set; ``q, k`` [B,H,1,d] (``k`` already repeated to the query heads).  Returns ``(B_Q', B_K', q_hat,
    k_hat)`` with ``q_hat, k_hat`` [B,H,1,r], everything in ``k``'s dtype.  A convenience for code written
    against the reference's functions: it builds a scratch layer state per call; the cache objects above are the
    fast path."""
    bsz, heads, n, r = A_K.shape
    d = K__.shape[-1]
    if n < 2:
        raise ValueError("the active set needs at least two rows")
    if max_iter > 8:
        raise ValueError("at most 8 alternations")
    dtype = k.dtype
    with on_device(k.device):
        st = LayerState(bsz, heads, heads, d, r, n - 1, 1, a_capacity=n + 1, host_capacity=1, dtype=dtype,
                        device=k.device, max_iter=max(1, max_iter), with_host=False,
                        weights=(1.0, 1.0, float(lambda_dec_q), float(lambda_dec_k)))
        try:
            st.A_K[:, :, :n].copy_(A_K)
            st.B_Q.copy_(B_Q)
            st.B_K.copy_(B_K)
            st.K_res.copy_(K__)
            st.table.copy_(torch.arange(n - 1, dtype=torch.int32, device=k.device).expand(bsz, heads, n - 1))
            st.lite_pos.fill_(n - 1)
            q_hat = st.project_update(q.reshape(bsz, heads, d).to(dtype).contiguous(),
                                      k.reshape(bsz, heads, d).to(dtype).contiguous(), max_iter, tol, n)
            out = (st.B_Q.clone(), st.B_K.clone(), q_hat.clone().unsqueeze(2), st.A_K[:, :, n:n + 1].clone())
            st.check_status()
        finally:
            st.close()
    return out


class LightAttentionIndicesNoHitMiss(LightAttentionIndicesFactory):
    """Comparison mode without the hit/miss table (lrqk_attention.py:1683-1775): every selected
    row is fetched from the host store on every step."""

    def only_indices_in_cpu(self, now_indices: torch.Tensor, new_indices: torch.Tensor):
        return new_indices.clone(), torch.ones(new_indices.shape[:3], dtype=torch.bool, device=new_indices.device)


# ------------------------------------------------------------------------------------------------
# the cache object handed to HF models
# ------------------------------------------------------------------------------------------------
class DynamicLRQKCache(_CacheBase):
    """Per-layer state machine pending -> collecting -> decoding: lrqk_attention.py:1778-1970.

    ``update(q, k, v, layer_idx, attention_mask=None)`` returns the un-repeated prompt K, V while
    prefilling and the resident [B,Hq,k+m,d] pair while decoding.  ``attend(...)`` is the fused
    variant for patched attention modules: while decoding it returns the attention output
    itself instead of K, V."""

    class State(enum.Enum):
        pending = 0
        collecting = 1
        decoding = 2

    def __init__(self, r: int = 16, num_active_tokens: int = 512, lambda_Q: float = 1.0, lambda_K: float = 1.0,
                 max_iter: Union[int, Tuple[int, int]] = 2, lite_tokens: int = 16,
                 tol: Union[float, Tuple[float, float]] = 1e-2, max_sequence_length: int = 4096,
                 num_key_value_groups: int = 1, lwattn_factory=LightAttentionIndicesFactory,
                 init_aq_ak_method: Union[InitAQAK, str] = InitAQAK.randn):
        if _CacheBase is not object:
            try:
                super().__init__(layers=[])
            except TypeError:  # older HF: Cache.__init__ takes no arguments
                super().__init__()
        self.num_key_value_groups, self.r, self.num_active_tokens = num_key_value_groups, r, num_active_tokens
        self.lambda_Q, self.lambda_K = lambda_Q, lambda_K
        self.max_iter, self.tol, self.lite_tokens = _pair(max_iter), _pair(tol), lite_tokens
        self.lwattn: Dict[int, LightAttentionIndicesFactory] = defaultdict(lambda: lwattn_factory(
            num_lite_tokens=lite_tokens, attn_topk=num_active_tokens, num_key_value_groups=num_key_value_groups,
            r=r, max_iter=max_iter, tol=tol, capacity=max_sequence_length, init_aq_ak_method=init_aq_ak_method))
        self.temp_buff_cache_qkv: Dict[int, _CacheQKV] = defaultdict(lambda: _CacheQKV(num_active_tokens, 2))
        self.sequence_state = defaultdict(lambda: DynamicLRQKCache.State.pending)
        self.sharding = None

    def shard_heads(self, group=None, sharding=None):
        """Run every layer for this rank's share of the (batch x KV head) units only (one process per
        GPU, ``group`` = the ranks taking part, default the whole process group).  ``update`` and
        ``attend`` keep taking the full [B, H, L, d] tensors, identical on every rank; ``attend``
        still returns the rows of ALL heads (the attention kernel stores them into every rank's
        exchange buffer), ``update`` returns this rank's K, V.  The reference is single-GPU."""
        from .sharding import HeadSharding
        if self.sequence_state:
            raise RuntimeError("shard_heads() must be called before the first layer sees a prompt")
        self.sharding = sharding if sharding is not None else HeadSharding(group)
        return self.sharding

    def _local(self, query_states, key_states, value_states, attention_mask=None):
        sh, hkv = self.sharding, key_states.shape[1]
        q, k, v = (sh.local(x, hkv).contiguous() for x in (query_states, key_states, value_states))
        return q, k, v, sh.local_rows(attention_mask, hkv)

    def __getitem__(self, layer_idx: int):
        raise NotImplementedError("DynamicLRQKCache does not support indexing")

    def __iter__(self):
        raise NotImplementedError("DynamicLRQKCache does not support iteration")

    def __len__(self):
        return len(self.sequence_state)

    def get_seq_length(self, layer_idx=0):
        return len(self.lwattn[layer_idx])

    def get_max_cache_shape(self, *a, **kw) -> Optional[int]:
        return None

    @property
    def seen_tokens(self):
        return self.get_seq_length()

    def is_decoding(self, layer_idx: int) -> bool:
        return self.sequence_state[layer_idx] == self.State.decoding

    def _prefill_states(self, query_states, key_states, value_states, layer_idx, attention_mask):
        state = self.sequence_state[layer_idx]
        bsz, _, seq_len, _ = key_states.shape
        if state == self.State.pending:
            if attention_mask is not None:                       # zero padded positions, :1901-1903
                key_states.mul_(attention_mask.view(bsz, 1, seq_len, 1))
                value_states.mul_(attention_mask.view(bsz, 1, seq_len, 1))
            if seq_len < self.num_active_tokens:                 # too short to factorise, :1910-1918
                self.temp_buff_cache_qkv[layer_idx].append(query_states, key_states, value_states)
                self.sequence_state[layer_idx] = self.State.collecting
            else:
                self.lwattn[layer_idx].prefill(query_states, key_states, value_states)
                self.sequence_state[layer_idx] = self.State.decoding
            return key_states, value_states
        buf = self.temp_buff_cache_qkv[layer_idx]                # collecting, :1928-1958
        if len(buf) + seq_len < self.num_active_tokens:
            _, k_all, v_all = buf.append(query_states, key_states, value_states)
            return k_all, v_all
        q_all, k_all, v_all = buf.append(query_states, key_states, value_states)
        self.lwattn[layer_idx].prefill(q_all, k_all, v_all)
        self.sequence_state[layer_idx] = self.State.decoding
        del self.temp_buff_cache_qkv[layer_idx]
        return k_all, v_all

    def update(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
               layer_idx: int, attention_mask: Optional[torch.Tensor] = None):
        if any(c is None for c in (query_states, key_states, value_states)):
            raise ValueError("None of query_states, key_states, and value_states can be None")
        if self.sharding is not None:
            query_states, key_states, value_states, attention_mask = self._local(query_states, key_states,
                                                                                 value_states, attention_mask)
        if self.sequence_state[layer_idx] != self.State.decoding:
            return self._prefill_states(query_states, key_states, value_states, layer_idx, attention_mask)
        return self.lwattn[layer_idx].decode(query_states, key_states, value_states)

    def attend(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
               layer_idx: int) -> torch.Tensor:
        """Decode-state only: one step plus attention, returns [B,Hq,1,d]."""
        if self.sequence_state[layer_idx] != self.State.decoding:
            raise RuntimeError("attend() is only valid once the layer is decoding; use update() before")
        fac = self.lwattn[layer_idx]
        if self.sharding is None:
            return fac.decode_attend(query_states, key_states, value_states)
        bsz, hq, hkv = query_states.shape[0], query_states.shape[1], key_states.shape[1]
        q, k, v, _ = self._local(query_states, key_states, value_states)
        exchange = self.sharding.exchange(q.shape[0] * q.shape[1], q.shape[-1], fac.state.dtype)
        fac.decode_attend_push(q, k, v, exchange)
        return self.sharding.gather_step(bsz, hkv, hq).unsqueeze(2)

    def attend_qkv(self, qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, layer_idx: int, q_heads: int,
                   kv_heads: int) -> torch.Tensor:
        """``attend`` from the fused projection of the new token: qkv [B, 1, (q_heads + 2 kv_heads) d] holds the
        un-rotated q, k and v heads of the whole model, cos / sin [B or 1, 1, d] the position's rotary factors.
        One kernel rotates q and k and cuts out this rank's heads; returns the rows of all heads [B,Hq,1,d]."""
        if self.sequence_state[layer_idx] != self.State.decoding:
            raise RuntimeError("attend_qkv() is only valid once the layer is decoding; use update() before")
        fac, bsz = self.lwattn[layer_idx], qkv.shape[0]
        if self.sharding is None:
            q, k, v = fac.state.rope_qkv(qkv, cos, sin, bsz, q_heads, kv_heads)
            return fac.decode_attend(q, k, v)
        mine = self.sharding.shard(bsz, kv_heads)
        q, k, v = fac.state.rope_qkv(qkv, cos, sin, bsz, q_heads, kv_heads, b0=mine.b0, kvh0=mine.h0)
        exchange = self.sharding.exchange(q.shape[0] * q.shape[1], q.shape[-1], fac.state.dtype)
        fac.decode_attend_push(q, k, v, exchange)
        return self.sharding.gather_step(bsz, kv_heads, q_heads).unsqueeze(2)

    def state_dict(self) -> dict:
        """The whole cache for ``load_state_dict``: every decoding layer's ``state_dict()`` and the prompt rows of
        layers that are still collecting a short prompt."""
        layers = {}
        for idx, state in self.sequence_state.items():
            if state == DynamicLRQKCache.State.decoding:
                layers[idx] = {"state": "decoding", "layer": self.lwattn[idx].state_dict()}
            elif state == DynamicLRQKCache.State.collecting:
                buf = self.temp_buff_cache_qkv[idx]
                layers[idx] = {"state": "collecting", "Q": buf.Q.tensor().cpu(), "K": buf.K.tensor().cpu(), "V": buf.V.tensor().cpu()}
        return {"format": 1, "layers": layers,
                "settings": dict(r=self.r, num_active_tokens=self.num_active_tokens, lite_tokens=self.lite_tokens,
                                 num_key_value_groups=self.num_key_value_groups)}

    def load_state_dict(self, sd: dict, device=None) -> None:
        """Restore what ``state_dict()`` wrote into this (fresh, identically configured) cache."""
        if sd.get("format") != 1:
            raise ValueError("not a state this version wrote")
        mine = dict(r=self.r, num_active_tokens=self.num_active_tokens, lite_tokens=self.lite_tokens,
                    num_key_value_groups=self.num_key_value_groups)
        if sd["settings"] != mine:
            raise ValueError(f"the saved cache was configured as {sd['settings']}, this one as {mine}")
        for idx, entry in sd["layers"].items():
            idx = int(idx)
            if entry["state"] == "decoding":
                self.lwattn[idx].load_state_dict(entry["layer"], device=device)
                self.sequence_state[idx] = DynamicLRQKCache.State.decoding
            else:
                dev = torch.device(device if device is not None else "cuda")
                self.temp_buff_cache_qkv[idx].append(entry["Q"].to(dev), entry["K"].to(dev), entry["V"].to(dev))
                self.sequence_state[idx] = DynamicLRQKCache.State.collecting

    def save(self, path: str) -> None:
        """``torch.save`` of ``state_dict()``."""
        torch.save(self.state_dict(), path)

    def load(self, path: str, device=None) -> None:
        self.load_state_dict(torch.load(path, map_location="cpu", weights_only=False), device=device)

    def check_status(self) -> None:
        """Synchronising check of every layer's device-side status words (the hit/miss difference's mismatch flag,
        the bounded waits of the attention and projection kernels) and of the exchange's arrival wait; raises
        LrqkError for the first that is set.  Off the hot path: ``close()`` calls it, a serving loop may call it
        once per request."""
        for fac in self.lwattn.values():
            if fac.state is not None:
                fac.state.check_status()
        if self.sharding is not None and self.sharding._exchange is not None:
            self.sharding._exchange.check_status()

    def close(self, check: bool = True):
        """Free every layer's device and page-locked host memory and the exchange buffers (after a last look at
        the status words, unless ``check=False``)."""
        try:
            if check:
                self.check_status()
        finally:
            self._free()

    def _free(self):
        for fac in self.lwattn.values():
            fac.close()
        if self.sharding is not None:
            self.sharding.close()
