"""The patched attention forward inside real Hugging Face decoder stacks (random-init, tiny):
Llama, Qwen2 (QKV bias) and Mistral.  Checks that the prompt pass is exact attention, that the
decode steps run through ``DynamicLRQKCache.attend`` (the CUDA path) and stay close to the
full-attention model when almost every token is resident, and that the loaders' helpers behave
like the reference's (family by substring, forward replaced on every layer)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(family: str):
    import transformers
    common = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=4096)
    if family == "llama":
        cfg = transformers.LlamaConfig(**common, head_dim=64, rope_theta=500000.0)
    elif family == "qwen":
        cfg = transformers.Qwen2Config(**common, rope_theta=1e6)
    else:
        cfg = transformers.MistralConfig(**common, head_dim=64, sliding_window=None)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(3)
    model = transformers.AutoModelForCausalLM.from_config(cfg).to(torch.bfloat16).cuda().eval()
    return model


@pytest.mark.parametrize("family", ["llama", "qwen", "mistral"])
def test_patched_stack_prefills_exactly_and_decodes_through_the_cuda_path(family):
    from lrqk_b200 import DynamicLRQKCache, load_model_hack
    from lrqk_b200.hf_models import family_of
    model = _tiny(family)
    assert family_of({"llama": "meta-llama/Llama-3-8B", "qwen": "Qwen/Qwen2.5-7B", "mistral": "mistralai/Mistral-7B"}[family]) == family
    k, m, S = 256, 16, 290
    ids = torch.randint(0, 512, (2, S), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        ref_prompt = model(input_ids=ids, use_cache=False).logits
        nxt = ref_prompt[:, -1].argmax(-1, keepdim=True)
        ref_step = model(input_ids=torch.cat([ids, nxt], 1), use_cache=False).logits[:, -1]
    patched = load_model_hack(f"tiny-{family}", base_model=model)
    assert patched is model and all(hasattr(l.self_attn, "_lrqk_original_forward") for l in model.model.layers)
    cache = DynamicLRQKCache(r=16, num_active_tokens=k, lite_tokens=m, max_iter=2, tol=1e-2, max_sequence_length=1024,
                             num_key_value_groups=2, init_aq_ak_method="top")
    with torch.no_grad():
        out = model(input_ids=ids, past_key_values=cache, use_cache=True)
        # the prompt pass is exact attention: same logits as the unpatched path up to bf16 noise
        assert torch.allclose(out.logits.float(), ref_prompt.float(), atol=3e-2, rtol=3e-2)
        assert all(cache.is_decoding(i) for i in range(2)) and cache.get_seq_length() == S
        step = model(input_ids=nxt, past_key_values=cache, use_cache=True).logits[:, -1]
        assert cache.get_seq_length() == S + 1
        # 272 of the 291 tokens are resident: the decode logits stay close to full attention
        cos = torch.nn.functional.cosine_similarity(step.float(), ref_step.float(), dim=-1)
        assert torch.isfinite(step).all() and float(cos.min()) > 0.97, cos
        tok = step.argmax(-1, keepdim=True)
        for _ in range(20):                                      # ring wraps once (m = 16)
            tok = model(input_ids=tok, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
        assert cache.get_seq_length() == S + 21
    # any other cache type takes the family's own forward
    with torch.no_grad():
        plain = model(input_ids=ids, use_cache=True).logits
    assert torch.allclose(plain.float(), ref_prompt.float(), atol=3e-2, rtol=3e-2)
    for fac in cache.lwattn.values():
        fac.close()


def test_generate_and_left_padded_prompts():
    """``model.generate(..., past_key_values=DynamicLRQKCache(...))`` -- the reference's usage -- and a
    left-padded batch: the prompt pass honours the mask transformers builds (same logits as the
    unpatched model on the real tokens) and the padded keys and values are zeroed in the cache,
    as the reference does (lrqk_attention.py:1901-1903)."""
    from lrqk_b200 import DynamicLRQKCache, patch_model
    model = _tiny("llama")
    S, pad = 300, 7
    ids = torch.randint(1, 512, (2, S), generator=torch.Generator().manual_seed(2)).cuda()
    mask = torch.ones_like(ids)
    mask[1, :pad] = 0                                           # second sequence is left-padded
    with torch.no_grad():
        ref = model(input_ids=ids, attention_mask=mask, use_cache=False).logits
    patch_model(model)
    mk = lambda: DynamicLRQKCache(r=16, num_active_tokens=256, lite_tokens=16, max_sequence_length=1024,  # noqa: E731
                                  num_key_value_groups=2, init_aq_ak_method="top")
    cache = mk()
    with torch.no_grad():
        out = model(input_ids=ids, attention_mask=mask, past_key_values=cache, use_cache=True).logits
    assert torch.allclose(out[0].float(), ref[0].float(), atol=3e-2, rtol=3e-2)
    assert torch.allclose(out[1, pad:].float(), ref[1, pad:].float(), atol=3e-2, rtol=3e-2)
    host = cache.lwattn[0].KVcpu.data
    assert not host[1, :, :pad].any() and host[1, :, pad:S].any() and host[0, :, :pad].any()
    cache2 = mk()
    gen = model.generate(input_ids=ids, attention_mask=mask, past_key_values=cache2, max_new_tokens=12, do_sample=False,
                         pad_token_id=0)
    assert gen.shape == (2, S + 12) and cache2.get_seq_length() == S + 11
    for c in (cache, cache2):
        for fac in c.lwattn.values():
            fac.close()


def test_unknown_family_is_rejected_like_the_reference():
    from lrqk_b200.hf_models import family_of
    with pytest.raises(ValueError):
        family_of("gpt2")


def _sharded_rank(rank, world, port, out_dir):
    """One rank of a head-sharded tiny Llama stack; rank 0 also runs the unsharded cache on the same
    weights and compares prompt logits and a run of decode logits."""
    import os
    import torch.distributed as dist
    from lrqk_b200 import DynamicLRQKCache, patch_model
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        model = _tiny("llama")                                   # same seed: same weights on every rank
        patch_model(model)
        S, n_steps = 290, 20
        ids = torch.randint(0, 512, (2, S), generator=torch.Generator().manual_seed(1)).cuda()
        mk = lambda: DynamicLRQKCache(r=16, num_active_tokens=256, lite_tokens=16, max_iter=2, tol=1e-2,  # noqa: E731
                                      max_sequence_length=1024, num_key_value_groups=2, init_aq_ak_method="top")

        def run(cache):
            logits = []
            with torch.no_grad():
                out = model(input_ids=ids, past_key_values=cache, use_cache=True).logits
                logits.append(out[:, -1].float())
                tok = out[:, -1].argmax(-1, keepdim=True)
                for _ in range(n_steps):
                    if cache.sharding is not None:
                        dist.broadcast(tok, 0)
                    step = model(input_ids=tok, past_key_values=cache, use_cache=True).logits[:, -1]
                    logits.append(step.float())
                    tok = step.argmax(-1, keepdim=True)
            return torch.stack(logits)

        sharded = mk()
        sharded.shard_heads()
        got = run(sharded)
        mine = sharded.sharding.shard(2, 2)
        ok = sharded.lwattn[0].state.kv_heads == mine.kv_heads == 1 and sharded.get_seq_length() == S + n_steps
        sharded.sharding._exchange.check_status()
        sharded.close()
        if rank == 0:
            plain = mk()
            want = run(plain)
            plain.close()
            cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
            ok = ok and bool(torch.isfinite(got).all()) and float(cos.min()) > 0.995
            detail = f"cos_min={float(cos.min()):.5f} max_abs={float((got - want).abs().max()):.4f}"
        else:
            detail = ""
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(("ok " if ok else "mismatch ") + detail)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_head_sharded_stack_on_two_gpus_matches_the_unsharded_one(tmp_path):
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_sharded_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert (tmp_path / f"rank{r}.txt").read_text().startswith("ok"), (tmp_path / f"rank{r}.txt").read_text()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shared_position", [False, True])
def test_rope_qkv_kernel_equals_the_eager_rotary_chain_bit_for_bit(dtype, shared_position):
    """One launch = split of the fused projection into heads + rotate-half rotary embedding + cut-out of a
    (batch, KV head) shard; compared with transformers' apply_rotary_pos_emb on the separate tensors."""
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    from lrqk_b200.state import LayerState
    B, Hq, Hkv, d = 4, 8, 2, 128
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(B, 1, (Hq + 2 * Hkv) * d, generator=g).to(dtype).cuda()
    rows = 1 if shared_position else B
    ang = torch.rand(rows, 1, d // 2, generator=g) * 6.28
    cos = torch.cat([ang.cos(), ang.cos()], -1).to(dtype).cuda()
    sin = torch.cat([ang.sin(), ang.sin()], -1).to(dtype).cuda()
    q, k, v = qkv.split([Hq * d, Hkv * d, Hkv * d], dim=-1)
    q, k, v = (t.view(B, 1, -1, d).transpose(1, 2) for t in (q, k, v))
    q_ref, k_ref = apply_rotary_pos_emb(q, k, cos, sin)
    for b0, bc, h0, hc in ((0, B, 0, Hkv), (2, 2, 1, 1), (0, 4, 1, 1)):
        st = LayerState(bc, hc * (Hq // Hkv), hc, d, 16, 64, 16, a_capacity=128, host_capacity=128, dtype=dtype,
                        device="cuda", with_host=False)
        qo, ko, vo = st.rope_qkv(qkv, cos, sin, B, Hq, Hkv, b0=b0, kvh0=h0)
        G = Hq // Hkv
        assert torch.equal(qo, q_ref[b0:b0 + bc, h0 * G:(h0 + hc) * G])
        assert torch.equal(ko, k_ref[b0:b0 + bc, h0:h0 + hc])
        assert torch.equal(vo, v[b0:b0 + bc, h0:h0 + hc])


def test_fused_projection_shares_storage_with_the_separate_ones():
    from lrqk_b200.hf_models import _fused_qkv
    model = _tiny("qwen")                                     # QKV bias
    attn = model.model.layers[0].self_attn
    before = [p.weight.detach().clone() for p in (attn.q_proj, attn.k_proj, attn.v_proj)]
    w, b = _fused_qkv(attn)
    assert b is not None and w.shape[0] == sum(t.shape[0] for t in before)
    assert attn.q_proj.weight.data_ptr() == w.data_ptr() and _fused_qkv(attn)[0] is w      # built once
    x = torch.randn(2, 1, w.shape[1], device="cuda", dtype=w.dtype)
    fused = torch.nn.functional.linear(x, w, b)
    sep = torch.cat([attn.q_proj(x), attn.k_proj(x), attn.v_proj(x)], -1)
    assert torch.allclose(fused.float(), sep.float(), atol=2e-2, rtol=2e-2)
    for p, t in zip((attn.q_proj, attn.k_proj, attn.v_proj), before):
        assert torch.equal(p.weight, t)


@pytest.mark.parametrize("dtype,rows,hidden,inter", [(torch.bfloat16, 1, 4096, 14336), (torch.bfloat16, 8, 3584, 18944),
                                                     (torch.float32, 3, 256, 512)])
def test_fused_layer_glue_matches_the_eager_modules(dtype, rows, hidden, inter):
    """lrqk_add_rmsnorm / lrqk_swiglu against the transformers modules they stand in for during decode: the
    residual add and the activation are element-wise and must agree bit for bit; the normalised row may differ
    by one unit in the last place where the variance was summed in another order."""
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    from lrqk_b200.hf_models import add_rmsnorm, swiglu
    g = torch.Generator(device="cuda").manual_seed(hidden)
    x = torch.randn(rows, 1, hidden, generator=g, device="cuda").to(dtype)
    d = (torch.randn(rows, 1, hidden, generator=g, device="cuda") * 0.3).to(dtype)
    norm = LlamaRMSNorm(hidden, eps=1e-5).to("cuda", dtype)
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(hidden, generator=g, device="cuda")).to(dtype))
        ref_sum = x + d
        ref = norm(ref_sum)
        total, normed = add_rmsnorm(x, d, norm.weight, norm.variance_epsilon)
        assert torch.equal(total, ref_sum)
        _, plain = add_rmsnorm(x, None, norm.weight, norm.variance_epsilon)
        ref_plain = norm(x)
    for got, want in ((normed, ref), (plain, ref_plain)):
        if dtype == torch.bfloat16:
            ulps = (got.view(torch.int16).int() - want.view(torch.int16).int()).abs()
            assert int(ulps.max()) <= 1 and float((ulps == 0).float().mean()) > 0.995
        else:
            assert float((got - want).abs().max() / want.abs().max()) < 1e-6
    gu = torch.randn(rows, 1, 2 * inter, generator=g, device="cuda").to(dtype) * 2
    want = torch.nn.functional.silu(gu[..., :inter]) * gu[..., inter:]
    got = swiglu(gu)
    if dtype == torch.bfloat16:
        ulps = (got.view(torch.int16).int() - want.view(torch.int16).int()).abs()
        assert int(ulps.max()) <= 1 and float((ulps == 0).float().mean()) > 0.999
    else:
        assert float((got - want).abs().max() / want.abs().max()) < 1e-6


def test_patched_decoder_layer_uses_the_fused_glue_only_while_decoding():
    import transformers
    from lrqk_b200 import DynamicLRQKCache, patch_model
    cfg = transformers.LlamaConfig(vocab_size=300, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=2048)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(3)
    model = transformers.AutoModelForCausalLM.from_config(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 300, (1, 400), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        ref_logits = []                                      # attention patched only: eager glue
        patch_model(model)
        for layer in model.model.layers:
            layer.forward = layer._lrqk_original_layer_forward
        cache = DynamicLRQKCache(r=16, num_active_tokens=128, lite_tokens=8, max_sequence_length=1024, num_key_value_groups=2,
                                 init_aq_ak_method="top")
        out = model(input_ids=ids, past_key_values=cache, use_cache=True)
        tok = out.logits[:, -1].argmax(-1, keepdim=True)
        for _ in range(4):
            out = model(input_ids=tok, past_key_values=cache, use_cache=True)
            ref_logits.append(out.logits[:, -1].float())
            tok = out.logits[:, -1].argmax(-1, keepdim=True)
        cache.close()
        for layer in model.model.layers:                     # now with the fused glue
            del layer._lrqk_original_layer_forward
            del layer.__dict__["forward"]
        patch_model(model)
        assert all(hasattr(l, "_lrqk_original_layer_forward") for l in model.model.layers)
        cache = DynamicLRQKCache(r=16, num_active_tokens=128, lite_tokens=8, max_sequence_length=1024, num_key_value_groups=2,
                                 init_aq_ak_method="top")
        out = model(input_ids=ids, past_key_values=cache, use_cache=True)
        tok = out.logits[:, -1].argmax(-1, keepdim=True)
        for i in range(4):
            out = model(input_ids=tok, past_key_values=cache, use_cache=True)
            got = out.logits[:, -1].float()
            assert float((got - ref_logits[i]).abs().max()) <= 3e-2 * float(ref_logits[i].abs().max())
            assert int(got.argmax()) == int(ref_logits[i].argmax())
            tok = got.argmax(-1, keepdim=True)
        cache.close()
