"""Comparison modes and measurement helpers of the reference, around the CUDA path.

* ``LightAttentionIndicesOffloadPrefill`` -- lrqk_attention.py:1616-1680: between the prompt pass
  and the first decode step a layer's device state (resident K/V, rank-r key factors) is parked in
  page-locked host memory, so that a many-layer prompt pass never holds every layer's state on
  the GPU at once.
* ``FullOffloadCache``                    -- lrqk_attention.py:1973-2026: the "keep everything on the
  host, bring everything back every step" baseline of the reference's throughput table.
* ``WrapForwardTimer``                    -- lrqk_attention.py:2031-2105: prompt / decode tokens per
  second around a model's ``forward`` (CUDA events here, wall clock there).
* ``HitRateCounter``                      -- wikitext_hitrate.py:36-51: a factory that records the miss
  rate of every step (from the device-side miss counts of the fused step here, through an
  ``only_indices_in_cpu`` override there; that override hook keeps working too).
* ``tps_estimate`` / ``run_task``         -- tps_estimate.py:41-142: the throughput driver; prompts are
  synthetic token ids of the requested lengths (the reference reads RULER prompts from disk).

The copies in the first two classes are plain ``torch`` transfers on a side stream: they are
set-up / baseline traffic, not part of the per-step selection path.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from .lrqk_attention import (DynamicLRQKCache, LightAttentionIndicesFactory, LightAttentionIndicesNoHitMiss,
                             _CacheBase)


class LightAttentionIndicesOffloadPrefill(LightAttentionIndicesFactory):
    """Do not keep K/V (and A_K) on the GPU between the prompt pass and the first decode step."""

    _PARKED = ("K_res", "V_res", "A_K")

    def prefill(self, query_states, key_states, value_states):
        super().prefill(query_states, key_states, value_states)
        st = self.state
        self.stream_temp = torch.cuda.Stream(query_states.device)
        self.stream_temp.wait_stream(torch.cuda.current_stream())
        self._parked: Dict[str, torch.Tensor] = {}
        with torch.cuda.stream(self.stream_temp):
            for name in self._PARKED:
                t = getattr(st, name)
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                host.copy_(t, non_blocking=True)
                t.record_stream(self.stream_temp)
                self._parked[name] = host
                setattr(st, name, None)          # the caching allocator may reuse the memory once the copy is done

    def _restore(self):
        if getattr(self, "_parked", None):
            st = self.state
            self.stream_temp.synchronize()
            with torch.cuda.stream(self.stream_temp):
                for name, host in self._parked.items():
                    setattr(st, name, host.to(st.device, non_blocking=True))
            self.stream_temp.synchronize()
            self._parked = None
            st._rebuild_struct()

    def _decode(self, *args, **kwargs):
        self._restore()
        return super()._decode(*args, **kwargs)


class _HostKV:
    """K and V of one layer in two page-locked host buffers [B, Hkv, capacity, d], grown by half when full."""

    def __init__(self, like: torch.Tensor, first_rows: int, capacity: int):
        b, h, _, d = like.shape
        self.rows = 0
        self.capacity = max(capacity, first_rows + first_rows // 2)
        self.k = torch.empty((b, h, self.capacity, d), dtype=like.dtype, pin_memory=True)
        self.v = torch.empty_like(self.k, pin_memory=True)

    def reserve(self, rows: int):
        if rows <= self.capacity:
            return
        torch.cuda.current_stream().synchronize()          # earlier copies out of the old buffers must be done
        cap = self.capacity
        while cap < rows:
            cap += cap // 2 + 1
        for name in ("k", "v"):
            old = getattr(self, name)
            new = torch.empty(old.shape[:2] + (cap, old.shape[3]), dtype=old.dtype, pin_memory=True)
            new[:, :, :self.rows].copy_(old[:, :, :self.rows])
            setattr(self, name, new)
        self.capacity = cap


class FullOffloadCache(_CacheBase):
    """The "everything on the host" row of the reference's throughput table (lrqk_attention.py:1973-2026):
    no K/V row stays on the GPU between calls.  ``update(key_states, value_states, layer_idx)`` stores the
    new rows in the layer's page-locked host buffers and returns ALL rows of that layer on the device.

    The device side is one staging pair shared by every layer, as large as the longest layer so far: the
    tensors ``update`` returns are views of it and stay valid until the next ``update`` call (the copies
    and the attention that reads them are ordered on the current stream)."""

    def __init__(self, capacity: int = 4096) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("FullOffloadCache stages through a CUDA device; none is available")
        if _CacheBase is not object:
            try:
                super().__init__(layers=[])
            except TypeError:
                super().__init__()
        self._capacity = capacity
        self._layers: Dict[int, _HostKV] = {}
        self._stage_k: Optional[torch.Tensor] = None
        self._stage_v: Optional[torch.Tensor] = None

    def __len__(self):
        return len(self._layers)

    def get_seq_length(self, layer_idx=0):
        lay = self._layers.get(layer_idx)
        return 0 if lay is None else lay.rows

    def get_max_cache_shape(self, *a, **kw) -> Optional[int]:
        return None

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        """(kv_length, kv_offset) for the mask builder of transformers 5.x: every stored row plus the new tokens."""
        q = int(query_length.shape[0]) if hasattr(query_length, "shape") else int(query_length)
        return self.get_seq_length(layer_idx) + q, 0

    def _staging(self, like: torch.Tensor, rows: int):
        s = self._stage_k
        if s is None or s.shape[2] < rows or s.shape[:2] != like.shape[:2] or s.dtype != like.dtype:
            cap = max(rows + rows // 2, self._capacity)
            shape = like.shape[:2] + (cap, like.shape[3])
            self._stage_k = torch.empty(shape, dtype=like.dtype, device=like.device)
            self._stage_v = torch.empty(shape, dtype=like.dtype, device=like.device)
        return self._stage_k, self._stage_v

    @torch.no_grad()
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int, *args, **kwargs):
        new_rows = key_states.shape[2]
        lay = self._layers.get(layer_idx)
        if lay is None:
            lay = self._layers[layer_idx] = _HostKV(key_states, new_rows, self._capacity)
        total = lay.rows + new_rows
        lay.reserve(total)
        dk, dv = self._staging(key_states, total)
        # the layer's stored rows come up from the host, the new rows are appended on both sides
        if lay.rows:
            dk[:, :, :lay.rows].copy_(lay.k[:, :, :lay.rows], non_blocking=True)
            dv[:, :, :lay.rows].copy_(lay.v[:, :, :lay.rows], non_blocking=True)
        dk[:, :, lay.rows:total].copy_(key_states)
        dv[:, :, lay.rows:total].copy_(value_states)
        lay.k[:, :, lay.rows:total].copy_(key_states, non_blocking=True)
        lay.v[:, :, lay.rows:total].copy_(value_states, non_blocking=True)
        lay.rows = total
        return dk[:, :, :total], dv[:, :, :total]


class WrapForwardTimer:
    """Prompt and decode throughput of a model, from CUDA events recorded around its ``forward``.

    Same use as the reference's timer (lrqk_attention.py:2031-2105): ``timer, model = WrapForwardTimer.wrap(model)``;
    the first timed call after ``wrap`` / ``reset`` is the prompt pass, every later call one decode step;
    ``prefill_tps()`` is prompt tokens per second, ``decode_tps()`` decode steps per second; ``remove_wrapper()``
    restores the model.  The times are device times: an event before and after each call on the current
    stream, no synchronisation inside the timed loop.  Decode time is the span from the first decode call's
    start to the last one's end, so host-side gaps between the steps (sampling, launch overhead) count too."""

    def __init__(self, module: torch.nn.Module):
        self.module = module
        self.seq_len = 0
        self._prompt = None            # (begin, end) events of the prompt pass
        self._decode = []              # (begin, end) events of every decode step
        self._inner = None
        self._shadowed = None

    # -- results ------------------------------------------------------------------------------
    @staticmethod
    def _seconds(begin, end) -> float:
        end.synchronize()
        return begin.elapsed_time(end) * 1e-3

    def prefill_tps(self) -> float:
        if self._prompt is None:
            return 0.0
        return self.seq_len / self._seconds(*self._prompt)

    def decode_tps(self) -> float:
        if not self._decode:
            return 0.0
        return len(self._decode) / self._seconds(self._decode[0][0], self._decode[-1][1])

    @property
    def decode_time_list(self):
        """Seconds of each decode step (device time inside the call)."""
        return [self._seconds(b, e) for b, e in self._decode]

    def reset(self):
        self.seq_len, self._prompt = 0, None
        self._decode.clear()

    # -- installation -------------------------------------------------------------------------
    def _timed(self, *args, **kwargs):
        first = self._prompt is None
        if first:
            ids = kwargs.get("input_ids")
            if ids is None:
                raise ValueError("the timed forward takes input_ids as a keyword argument")
            self.seq_len = ids.shape[1]
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        result = self._inner(*args, **kwargs)
        end.record()
        if first:
            self._prompt = (begin, end)
        else:
            self._decode.append((begin, end))
        return result

    @classmethod
    def wrap(cls, module: torch.nn.Module):
        timer = getattr(module, "_lrqk_forward_timer", None)
        if timer is None:
            timer = cls(module)
            timer._shadowed = module.__dict__.get("forward")      # an instance-level forward, if one was set
            timer._inner = module.forward
            module.forward = timer._timed
            module._lrqk_forward_timer = timer
        return timer, module

    def remove_wrapper(self):
        if self._inner is not None:
            if self._shadowed is not None:
                self.module.forward = self._shadowed
            else:
                del self.module.__dict__["forward"]               # the class's own forward shows again
            self._inner = None
            del self.module._lrqk_forward_timer


class HitRateCounter(LightAttentionIndicesFactory):
    """A factory that logs the miss rate of every selecting decode step (what the reference's
    ``wikitext_hitrate.py:36-51`` collects by overriding ``only_indices_in_cpu``).

    Here the step's hit/miss difference already leaves a per-head miss count on the device, so the
    counter keeps the fused step and appends ``sum(miss_count) / (heads * attn_topk)`` to a device-side
    log after each step, without a host synchronisation; ``miss_rates`` copies the log to the host."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._log: Optional[torch.Tensor] = None
        self._logged = 0

    def _decode(self, *args, **kwargs):
        st = super()._decode(*args, **kwargs)
        if self.current_len > self.gpu_capacity:            # a step that ran the difference (:1571-1573)
            if self._log is None or self._logged == self._log.numel():
                grown = torch.zeros(max(256, 2 * self._logged), dtype=torch.float32, device=st.device)
                if self._log is not None:
                    grown[:self._logged].copy_(self._log)
                self._log = grown
            self._log[self._logged] = st.miss_count.sum() / float(st.miss_count.numel() * st.k)
            self._logged += 1
        return st

    @property
    def miss_rates(self):
        return [] if self._log is None else self._log[:self._logged].tolist()

    def average_miss_rate(self) -> float:
        return float(self._log[:self._logged].mean()) if self._logged else float("nan")


task_dict = {
    "lrqk_default": LightAttentionIndicesFactory,
    "lrqk_offload": LightAttentionIndicesOffloadPrefill,
    "lrqk_no_hitmiss": LightAttentionIndicesNoHitMiss,
    "gpu_only": None,
    "cpu_offload": None,
}


def tps_estimate(model, past_key_values_factory: Optional[Callable] = None, prompt_lens=(4096,), max_new_tokens: int = 32,
                 vocab_size: Optional[int] = None, seed: int = 0) -> dict:
    """Prompt and decode tokens per second of greedy generation for each prompt length
    (tps_estimate.py:41-85), on seeded uniform-random token ids."""
    wrapper, _ = WrapForwardTimer.wrap(model)
    vocab = vocab_size or model.config.vocab_size
    device = next(model.parameters()).device
    out = {}
    try:
        for n in prompt_lens:
            g = torch.Generator().manual_seed(seed + n)
            ids = torch.randint(0, vocab, (1, n), generator=g).to(device)
            wrapper.reset()
            cache = past_key_values_factory() if past_key_values_factory is not None else None
            with torch.no_grad():
                logits = model(input_ids=ids, past_key_values=cache, use_cache=True)
                cache = logits.past_key_values
                tok = logits.logits[:, -1].argmax(-1, keepdim=True)
                for _ in range(max_new_tokens):
                    res = model(input_ids=tok, past_key_values=cache, use_cache=True)
                    tok = res.logits[:, -1].argmax(-1, keepdim=True)
            out[str(n)] = {"prefill_tps": wrapper.prefill_tps(), "decode_tps": wrapper.decode_tps()}
    finally:
        wrapper.remove_wrapper()
    return out


def run_task(name: str, model, *, r: int = 16, num_active_tokens: int = 1024, lite_tokens: int = 16, prompt_lens=(4096,),
             max_new_tokens: int = 32, out_path: Optional[str] = None) -> dict:
    """One row of the reference's throughput table (tps_estimate.py:126-142): ``name`` in ``task_dict``.
    Like the reference's driver (:127-130), a row whose ``out_path`` already exists is not measured again: the
    file's records are returned."""
    if name not in task_dict:
        raise ValueError(f"Unknown task {name}")
    if out_path and os.path.exists(out_path):
        with open(out_path) as f:
            return json.load(f)
    groups = model.config.num_attention_heads // model.config.num_key_value_heads
    if name == "cpu_offload":
        factory = FullOffloadCache
    elif name == "gpu_only":
        factory = None
    else:
        cls = task_dict[name]
        factory = lambda: DynamicLRQKCache(r=r, num_active_tokens=num_active_tokens, lite_tokens=lite_tokens,  # noqa: E731
                                           max_sequence_length=max(prompt_lens) + max_new_tokens + 64,
                                           num_key_value_groups=groups, lwattn_factory=cls)
    records = tps_estimate(model, factory, prompt_lens=prompt_lens, max_new_tokens=max_new_tokens)
    if out_path:
        with open(out_path, "w") as f:
            json.dump(records, f, indent=4)
    return records
