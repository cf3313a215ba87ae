"""Hugging Face integration: attention forward for Llama / Qwen2 / Mistral decoder layers that
routes through ``DynamicLRQKCache``, and the reference's loader functions.

Mirrors the reference's patched attention classes and loaders (paths relative to its checkout):

* ``LRQK_LlamaFlashAttention2.forward``   -- lrqk_attention.py:2222-2335
* ``LRQK_Qwen2FlashAttention2.forward``   -- lrqk_attention.py:2108-2219
* ``LRQK_MistralFlashAttention2.forward`` -- lrqk_attention.py:2338-2458
* ``load_model_hack`` / ``load_tokenizer`` / ``load_lrqk_model`` / ``load_model``
                                          -- lrqk_attention.py:2595-2743

The reference replaces the ``flash_attention_2`` class of transformers 4.47; the attention
modules of transformers 5.x are a single class per family with one ``forward(hidden_states,
position_embeddings, attention_mask, past_key_values, **kwargs)``, so here that bound method is
replaced on every decoder layer (the reference's second pass does the same, :2661-2665).  The
three families share the code below: q/k/v projections (Qwen2's carry biases), rotary embedding
from the family's own ``apply_rotary_pos_emb``, the cache call, the output projection.

What the patched forward does with the cache:

* layer still prefilling (``pending`` / ``collecting``): ``cache.update(q, k, v, layer_idx,
  attention_mask)`` -- the reference's call (:2284-2286) -- returns the prompt's K, V and
  exact causal attention over them is taken with ``scaled_dot_product_attention`` (the prompt
  attention is a dense library operation outside the selection path);
* layer decoding: ``cache.attend(q, k, v, layer_idx)`` runs the whole per-layer step (ring
  write, rank-r projection, proxy scoring + top-k, hit/miss, miss fetch, attention over the
  resident rows) in the CUDA library and returns the attention output directly.

With ``cache.shard_heads()`` (one process per GPU) the dense parts run replicated on every rank,
each rank's cache holds its share of the (batch x KV head) units, the prompt's attention is taken
for those heads only and all-gathered, and ``cache.attend`` returns all heads' rows through the
exchange fused into the attention kernel.

Any other cache type falls through to the family's original forward.
"""
from __future__ import annotations

import sys
import types
import warnings
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .lrqk_attention import DynamicLRQKCache

SUPPORTED_FAMILIES = ("qwen", "llama", "mistral")


def _causal_attention(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, scaling: float,
                      pad_mask: Optional[torch.Tensor], mask4d: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Exact attention of q [B,Hq,L,d] over K, V [B,Hkv,S,d] (S >= L; the queries are the last L
    positions), causal.  ``mask4d`` -- the [B,1,L,S] mask transformers built for this call, boolean
    or additive -- is used as it is when its shape fits; otherwise the causal pattern is rebuilt
    here, combined with the [B,S] padding mask (1 = token) if there is one.  Returns [B,L,Hq,d]."""
    L, S = q.shape[2], K.shape[2]
    mask = None
    if mask4d is not None and mask4d.dim() == 4 and mask4d.shape[-2] == L and mask4d.shape[-1] == S:
        mask = mask4d if mask4d.dtype == torch.bool else mask4d.to(q.dtype)
    elif pad_mask is not None or (L > 1 and L != S):
        idx_q = torch.arange(S - L, S, device=q.device)[:, None]
        idx_k = torch.arange(S, device=q.device)[None, :]
        mask = (idx_k <= idx_q)[None, None]                      # [1,1,L,S]
        if pad_mask is not None:
            mask = mask & pad_mask[:, None, None, -S:].to(torch.bool)
    out = F.scaled_dot_product_attention(q, K, V, attn_mask=mask, is_causal=(mask is None and L > 1),
                                         scale=scaling, enable_gqa=K.shape[1] != q.shape[1])
    return out.transpose(1, 2)


def _padding_mask(attention_mask: Optional[torch.Tensor], seq_len: int) -> Optional[torch.Tensor]:
    """The [B,S] token mask the reference's cache expects (:1901-1903).  transformers 5.x hands the
    attention modules a [B,1,L,S] mask (or none at all when nothing is padded): its last query row
    tells which keys are real tokens."""
    if attention_mask is None:
        return None
    if attention_mask.dim() == 2:
        return attention_mask[:, -seq_len:].to(torch.bool)
    if attention_mask.dim() == 4 and attention_mask.shape[-1] >= seq_len:
        row = attention_mask[:, 0, -1, -seq_len:]
        return row if row.dtype == torch.bool else (row == 0)
    return None


def _fused_qkv(attn):
    """(weight [(Hq + 2 Hkv) d, hidden], bias or None) of one projection that yields q|k|v, or None when the
    module's projections are not three plain ``nn.Linear`` of one dtype.  Built once: the three weights are
    concatenated and each projection's parameter is re-pointed to its rows of the fused tensor, so no memory is
    added and the separate projections keep working."""
    f = getattr(attn, "_lrqk_qkv", None)
    if f is not None:
        if f is False or attn.q_proj.weight.data_ptr() == f[0].data_ptr():
            return f or None
    projs = (attn.q_proj, attn.k_proj, attn.v_proj)
    ok = (all(type(p) is torch.nn.Linear for p in projs)
          and len({(p.weight.dtype, p.weight.device, p.in_features, p.bias is None) for p in projs}) == 1)
    if not ok:
        attn._lrqk_qkv = False
        return None
    with torch.no_grad():
        w = torch.cat([p.weight.data for p in projs], 0)
        b = None if projs[0].bias is None else torch.cat([p.bias.data for p in projs], 0)
        off = 0
        for p in projs:
            n = p.out_features
            p.weight.data = w[off:off + n]
            if b is not None:
                p.bias.data = b[off:off + n]
            off += n
    attn._lrqk_qkv = (w, b)
    return attn._lrqk_qkv


def lrqk_attention_forward(self, hidden_states: torch.Tensor,
                           position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                           attention_mask: Optional[torch.Tensor] = None, past_key_values=None, **kwargs):
    """Replacement for ``{Llama,Qwen2,Mistral}Attention.forward`` of transformers 5.x."""
    if not isinstance(past_key_values, DynamicLRQKCache):
        return self._lrqk_original_forward(hidden_states, position_embeddings=position_embeddings,
                                           attention_mask=attention_mask, past_key_values=past_key_values, **kwargs)
    cache: DynamicLRQKCache = past_key_values
    input_shape = hidden_states.shape[:-1]
    hidden_shape = (*input_shape, -1, self.head_dim)
    if hidden_states.shape[1] == 1 and cache.is_decoding(self.layer_idx):
        # decode step: one fused projection, then one kernel that rotates q and k and hands this rank's heads
        # to the layer step (instead of three projections and the dozen element-wise launches of the rotary op)
        fused = _fused_qkv(self)
        cos, sin = position_embeddings
        state = cache.lwattn[self.layer_idx].state
        if (fused is not None and hidden_states.dtype == fused[0].dtype == state.dtype == cos.dtype
                and cos.shape[-1] == self.head_dim):
            qkv = F.linear(hidden_states, fused[0], fused[1])
            kv_heads = self.k_proj.out_features // self.head_dim
            q_heads = self.q_proj.out_features // self.head_dim
            attn_output = cache.attend_qkv(qkv, cos.contiguous(), sin.contiguous(), self.layer_idx, q_heads, kv_heads)
            attn_output = attn_output.transpose(1, 2).reshape(*input_shape, -1).contiguous()
            return self.o_proj(attn_output), None
    query_states = self.q_proj(hidden_states).view(hidden_shape).transpose(1, 2)
    key_states = self.k_proj(hidden_states).view(hidden_shape).transpose(1, 2)
    value_states = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
    cos, sin = position_embeddings
    rope = sys.modules[type(self).__module__].apply_rotary_pos_emb
    query_states, key_states = rope(query_states, key_states, cos, sin)

    q_len = query_states.shape[2]
    if cache.is_decoding(self.layer_idx):
        if q_len != 1:
            raise NotImplementedError("a decoding LRQK layer takes one new token per call, like the reference's "
                                      "LightAttentionIndicesFactory.decode")
        attn_output = cache.attend(query_states, key_states, value_states, self.layer_idx).transpose(1, 2)
    else:
        pad = _padding_mask(attention_mask, key_states.shape[2])
        K, V = cache.update(query_states, key_states.contiguous(), value_states.contiguous(), self.layer_idx,
                            attention_mask=None if pad is None else pad.to(key_states.dtype))
        pad_all, sh = _padding_mask(attention_mask, K.shape[2]), getattr(cache, "sharding", None)
        if sh is None:
            attn_output = _causal_attention(query_states, K, V, self.scaling, pad_all, mask4d=attention_mask)
        else:
            # head-sharded cache: K, V are this rank's; attend for its query heads, then every rank
            # receives the rows of all heads
            hkv, mask4d = key_states.shape[1], attention_mask
            if mask4d is not None and mask4d.dim() == 4 and mask4d.shape[0] == query_states.shape[0]:
                mask4d = sh.local_rows(mask4d, hkv)
            local = _causal_attention(sh.local(query_states, hkv), K, V, self.scaling, sh.local_rows(pad_all, hkv),
                                      mask4d=mask4d)
            attn_output = sh.gather_prompt(local, query_states.shape[0], hkv, query_states.shape[1])
    attn_output = attn_output.reshape(*input_shape, -1).contiguous()
    return self.o_proj(attn_output), None


# ------------------------------------------------------------------------------------------------
# decode-time decoder layer: the element-wise glue around the attention call as two fused kernels
# ------------------------------------------------------------------------------------------------
def _lrqk_dtype(t: torch.Tensor):
    from .state import _DTYPES
    return _DTYPES.get(t.dtype)


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, want_sum: bool = True):
    """(x + delta, weight * rmsnorm(x + delta)) for [..., hidden] tensors in one launch (``lrqk_add_rmsnorm``);
    ``delta=None``: no add, and no sum is returned unless asked."""
    import ctypes as C
    from . import _lib
    from .state import _ptr, _stream
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    normed = torch.empty_like(x)
    total = torch.empty_like(x) if (want_sum and delta is not None) else None
    _lib.check(_lib.lib().lrqk_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(weight), float(eps), _lrqk_dtype(x), rows, hidden,
                                           _ptr(total), _ptr(normed), _stream()), "lrqk_add_rmsnorm")
    return (x if delta is None else total), normed


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up of the fused gate|up projection [..., 2 * inter] in one launch (``lrqk_swiglu``)."""
    from . import _lib
    from .state import _ptr, _stream
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * inter)
    out = torch.empty(gate_up.shape[:-1] + (inter,), dtype=gate_up.dtype, device=gate_up.device)
    _lib.check(_lib.lib().lrqk_swiglu(_ptr(gate_up), _lrqk_dtype(gate_up), rows, inter, _ptr(out), _stream()), "lrqk_swiglu")
    return out


def _fused_gate_up(mlp):
    """Weight [2 * inter, hidden] of one projection that yields gate|up, or None when the MLP is not the plain
    bias-free SwiGLU of these families.  Built once; the two projections are re-pointed into the fused tensor."""
    f = getattr(mlp, "_lrqk_gate_up", None)
    if f is not None:
        if f is False or mlp.gate_proj.weight.data_ptr() == f.data_ptr():
            return None if f is False else f
    ok = (all(hasattr(mlp, n) and type(getattr(mlp, n)) is torch.nn.Linear for n in ("gate_proj", "up_proj", "down_proj"))
          and mlp.gate_proj.bias is None and mlp.up_proj.bias is None
          and mlp.gate_proj.weight.dtype == mlp.up_proj.weight.dtype
          and mlp.gate_proj.weight.shape == mlp.up_proj.weight.shape
          and type(getattr(mlp, "act_fn", None)).__name__ in ("SiLU", "SiLUActivation"))
    if not ok:
        mlp._lrqk_gate_up = False
        return None
    with torch.no_grad():
        w = torch.cat([mlp.gate_proj.weight.data, mlp.up_proj.weight.data], 0)
        n = mlp.gate_proj.out_features
        mlp.gate_proj.weight.data = w[:n]
        mlp.up_proj.weight.data = w[n:]
    mlp._lrqk_gate_up = w
    return w


def _norm_params(norm):
    """(weight, eps) of an RMSNorm module of these families, or None for anything else."""
    eps = getattr(norm, "variance_epsilon", None)
    w = getattr(norm, "weight", None)
    if eps is None or w is None or not type(norm).__name__.endswith("RMSNorm"):
        return None
    return w, float(eps)


def lrqk_decoder_layer_forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None,
                               past_key_values=None, use_cache=False, position_embeddings=None, **kwargs):
    """Replacement for ``{Llama,Qwen2,Mistral}DecoderLayer.forward``: while the layer's LRQK state is decoding one
    token per sequence, the two RMSNorms, the two residual adds and the SwiGLU activation run as four launches of
    this library instead of some twenty eager ones (same rounding points); anything else takes the module's own
    forward."""
    cache = past_key_values
    n1 = n2 = gate_up = None
    if (isinstance(cache, DynamicLRQKCache) and hidden_states.shape[1] == 1 and cache.is_decoding(self.self_attn.layer_idx)
            and _lrqk_dtype(hidden_states) is not None and hidden_states.is_contiguous()):
        n1, n2 = _norm_params(self.input_layernorm), _norm_params(self.post_attention_layernorm)
        gate_up = _fused_gate_up(self.mlp)
    if n1 is None or n2 is None or gate_up is None or n1[0].dtype != hidden_states.dtype or gate_up.dtype != hidden_states.dtype:
        return self._lrqk_original_layer_forward(hidden_states, attention_mask=attention_mask, position_ids=position_ids,
                                                 past_key_values=past_key_values, use_cache=use_cache,
                                                 position_embeddings=position_embeddings, **kwargs)
    _, normed = add_rmsnorm(hidden_states, None, n1[0], n1[1])
    attn_out, _ = self.self_attn(hidden_states=normed, attention_mask=attention_mask, position_ids=position_ids,
                                 past_key_values=past_key_values, use_cache=use_cache,
                                 position_embeddings=position_embeddings, **kwargs)
    hidden_states, normed = add_rmsnorm(hidden_states, attn_out.contiguous(), n2[0], n2[1])
    act = swiglu(F.linear(normed, gate_up))
    return hidden_states + self.mlp.down_proj(act)


def family_of(model_name: str) -> str:
    """Model family by substring of the name, in the reference's order (:2611-2632)."""
    mn = model_name.lower()
    for fam in SUPPORTED_FAMILIES:
        if fam in mn:
            return fam
    raise ValueError(f"Unknown model name: {model_name}")


def patch_model(model) -> int:
    """Replace ``self_attn.forward`` of every decoder layer; returns the number of layers patched."""
    n = 0
    for layer in model.model.layers:
        attn = getattr(layer, "self_attn", None)
        if attn is None:
            continue
        if not hasattr(attn, "_lrqk_original_forward"):
            attn._lrqk_original_forward = attn.forward
            attn.forward = types.MethodType(lrqk_attention_forward, attn)
        if not hasattr(layer, "_lrqk_original_layer_forward") and hasattr(layer, "mlp") and hasattr(layer, "input_layernorm"):
            layer._lrqk_original_layer_forward = layer.forward
            layer.forward = types.MethodType(lrqk_decoder_layer_forward, layer)
        n += 1
    return n


def load_model_hack(model_name: str, device=None, yarn=None, base_model=None):
    """The model with its ``self_attn.forward`` replaced (lrqk_attention.py:2595-2671).

    - model_name: the model name (also selects the family: qwen / llama / mistral)
    - device: the device to load the model on (``device_map="auto"`` when None)
    - yarn: additional keyword arguments for ``from_pretrained``
    - base_model: use this model instead of loading one
    """
    import transformers
    family_of(model_name)
    if yarn is None:
        yarn = {}
    if base_model is not None:
        model = base_model
    else:
        model = transformers.AutoModelForCausalLM.from_pretrained(
            model_name, attn_implementation="sdpa", dtype=torch.bfloat16, trust_remote_code=True,
            device_map="auto" if device is None else device, **yarn)
    patch_model(model)
    return model.eval()


def load_tokenizer(model_name: str, max_length=None):
    """Left-padding tokenizer with a pad token (lrqk_attention.py:2674-2685)."""
    import transformers
    tokenizer = transformers.AutoTokenizer.from_pretrained(model_name, padding_side="left", max_length=max_length)
    if tokenizer.pad_token is None:
        tokenizer.pad_token = tokenizer.eos_token
        tokenizer.pad_token_id = tokenizer.eos_token_id
    return tokenizer


def load_lrqk_model(model_name: str, max_length=None, device=None, yarn=None, base_model=None):
    """(model, tokenizer) with the LRQK attention forward (lrqk_attention.py:2687-2699)."""
    model = load_model_hack(model_name, device, yarn=yarn, base_model=base_model)
    return model, load_tokenizer(model_name, max_length)


def load_model(model_name: str, lrqk=True, max_length=None, device=None, yarn=None, base_model=None):
    """(model, tokenizer); ``lrqk=False`` loads the plain model (lrqk_attention.py:2702-2743)."""
    import transformers
    if yarn is None:
        yarn = {}
    if device is None:
        warnings.warn("When device is None, device_map=auto is used: layers may land on several GPUs.  Each layer's "
                      "LRQK state then lives on, and runs with, that layer's device; name one device to keep the "
                      "model on a single GPU.")
    if lrqk:
        model = load_model_hack(model_name, device, yarn=yarn, base_model=base_model)
    elif base_model is not None:
        model = base_model
    else:
        model = transformers.AutoModelForCausalLM.from_pretrained(
            model_name, dtype=torch.bfloat16, trust_remote_code=True, attn_implementation="sdpa",
            device_map="auto" if device is None else device, **yarn)
    model = model.eval()
    return model, load_tokenizer(model_name, max_length)
