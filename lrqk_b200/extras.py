"""Comparison modes and measurement helpers of the reference, around the CUDA path.

* ``LightAttentionIndicesOffloadPrefill`` -- lrqk_attention.py:1616-1680: between the prompt pass
  and the first decode step a layer's device state (resident K/V, rank-r key factors) is parked in
  page-locked host memory, so that a many-layer prompt pass never holds every layer's state on
  the GPU at once.
* ``FullOffloadCache``                    -- lrqk_attention.py:1973-2026: the "keep everything on the
  host, bring everything back every step" baseline of the reference's throughput table.
* ``WrapForwardTimer``                    -- lrqk_attention.py:2031-2105: wall-clock prompt / decode
  tokens per second around a model's ``forward``.
* ``HitRateCounter``                      -- wikitext_hitrate.py:36-51: a factory that records the miss
  rate of every step through the overridable ``only_indices_in_cpu`` hook.
* ``tps_estimate`` / ``run_task``         -- tps_estimate.py:41-142: the throughput driver; prompts are
  synthetic token ids of the requested lengths (the reference reads RULER prompts from disk).

The copies in the first two classes are plain ``torch`` transfers on a side stream: they are
set-up / baseline traffic, not part of the per-step selection path.
"""
from __future__ import annotations

import json
import time
from collections import defaultdict
from typing import Callable, Dict, Optional

import numpy as np
import torch

from .lrqk_attention import (AutoIncreaseTensorSharedKV, DynamicLRQKCache, LightAttentionIndicesFactory,
                             LightAttentionIndicesNoHitMiss, _CacheBase)


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


class FullOffloadCache(_CacheBase):
    """Every layer's K|V lives in page-locked host memory; ``update`` appends the new rows and returns
    the whole K and V on the device (lrqk_attention.py:1973-2026)."""

    def __init__(self) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("OffloadedCache can only be used with a GPU")
        if _CacheBase is not object:
            try:
                super().__init__(layers=[])
            except TypeError:
                super().__init__()
        self.KVcpu = defaultdict(lambda: AutoIncreaseTensorSharedKV(capacity=4096, dim=2, device="cpu", pin_memory=True))

    def __len__(self):
        return len(self.KVcpu)

    def get_seq_length(self, layer_idx=0):
        return len(self.KVcpu[layer_idx])

    def get_max_cache_shape(self, *a, **kw) -> Optional[int]:
        return None

    def get_mask_sizes(self, query_length, layer_idx: int = 0):
        """(kv_length, kv_offset) for the mask builder of transformers 5.x: everything cached so far plus the new tokens."""
        q = int(query_length.shape[0]) if hasattr(query_length, "shape") else int(query_length)
        return self.get_seq_length(layer_idx) + q, 0

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int, *args, **kwargs):
        kv = self.KVcpu[layer_idx]
        kv.append(key_states, value_states)
        hdim = key_states.shape[-1]
        full = kv.tensor()
        return (full.narrow(3, 0, hdim).to(key_states.device), full.narrow(3, hdim, hdim).to(value_states.device))


class WrapForwardTimer:
    """Wall-clock timer around ``module.forward``: the first call is the prompt pass, every later
    call one decode step (lrqk_attention.py:2031-2105)."""

    def __init__(self, module: torch.nn.Module):
        self.module = module
        self.prefill_begin = None
        self.prefill_end = None
        self.decode_begin = None
        self.decode_time_list = []
        self.seq_len = 0
        self.original_method = None

    def prefill_tps(self):
        """Prefill token per second"""
        if self.prefill_begin is None:
            return 0.0
        return self.seq_len / (self.prefill_end - self.prefill_begin)

    def decode_tps(self):
        """Decode token per second"""
        if len(self.decode_time_list) == 0:
            return 0.0
        return len(self.decode_time_list) / sum(self.decode_time_list)

    def remove_wrapper(self):
        setattr(self.module, "forward", self.original_method)
        del self.original_method
        setattr(self.module, "manual_time_wrapped", False)

    def reset(self):
        self.prefill_begin = None
        self.prefill_end = None
        self.decode_begin = None
        self.decode_time_list.clear()
        self.seq_len = 0

    @classmethod
    def wrap(cls, module: torch.nn.Module):
        wraper = cls(module)
        if getattr(module, "manual_time_wrapped", False):
            return wraper, wraper.module
        original_method = getattr(module, "forward")
        wraper.original_method = original_method
        setattr(wraper.module, "manual_time_wrapped", True)

        def __new_method(self, *args, **kwargs):
            if wraper.prefill_begin is None:
                input_ids = kwargs.get("input_ids", None)
                if input_ids is None:
                    raise ValueError("input_ids is None")
                wraper.seq_len = input_ids.shape[1]
                wraper.prefill_begin = time.time()
            else:
                wraper.decode_begin = time.time()
            result = original_method(*args, **kwargs)
            torch.cuda.synchronize()   # the step's work is asynchronous here: wait for it before reading the clock
            if wraper.prefill_end is None:
                wraper.prefill_end = time.time()
            else:
                wraper.decode_time_list.append(time.time() - wraper.decode_begin)
            return result

        setattr(wraper.module, "forward", __new_method.__get__(wraper.module))
        return wraper, wraper.module


class HitRateCounter(LightAttentionIndicesFactory):
    """Records the miss rate of every decode step (wikitext_hitrate.py:36-51).  Overriding
    ``only_indices_in_cpu`` switches the object to the stage-by-stage path with int64 tensors of the
    reference's shapes."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.miss_rates = []

    def only_indices_in_cpu(self, now_indices: torch.Tensor, new_indices: torch.Tensor):
        updated_indices, now_in_new = super().only_indices_in_cpu(now_indices, new_indices)
        self.miss_rates.append((torch.sum(now_in_new) / now_in_new.numel()).item())   # 1 = miss: loaded from the host
        return updated_indices, now_in_new

    def average_miss_rate(self):
        return float(np.mean(self.miss_rates))


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
    """One row of the reference's throughput table (tps_estimate.py:126-142): ``name`` in ``task_dict``."""
    if name not in task_dict:
        raise ValueError(f"Unknown task {name}")
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
