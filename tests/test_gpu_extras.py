"""Comparison modes and drivers mirrored from the reference: the offload-prefill factory gives the
same steps as the default one, the hit-rate hook sees every step, and the throughput driver runs
each row of the reference's table on a tiny random-init Llama."""
import pytest
import torch

import lrqk_oracle as orc

pytestmark = pytest.mark.gpu


def _run(factory_cls, steps=6, device="cuda"):
    c = dict(seed=31, bsz=1, hq=4, hkv=2, seq=900, d=128, r=16, k=64, m=4)
    Q, K, V = orc.make_prompt(c["seed"], c["bsz"], c["hq"], c["hkv"], c["seq"], c["d"])
    fac = factory_cls(num_lite_tokens=c["m"], attn_topk=c["k"], num_key_value_groups=2, r=c["r"], max_iter=(2, 2),
                      tol=1e-2, capacity=c["seq"] + 64, init_aq_ak_method="top")
    fac.prefill(Q.to(device), K.to(device), V.to(device))
    outs = []
    for s in range(steps):
        q, k, v = orc.make_step(c["seed"], s, c["bsz"], c["hq"], c["hkv"], c["d"])
        outs.append(fac.decode_attend(q.to(device), k.to(device), v.to(device)).clone())
    torch.cuda.synchronize(device)
    fac.state.check_status()
    return fac, outs


def test_layers_on_two_devices_of_one_process():
    """One process, layer states on cuda:0 and cuda:1 (what device_map="auto" does to a large model): every entry
    runs with the state's device current, whatever the caller's current device is."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from lrqk_b200 import LightAttentionIndicesFactory
    assert torch.cuda.current_device() == 0
    a, outs_a = _run(LightAttentionIndicesFactory)
    b, outs_b = _run(LightAttentionIndicesFactory, device="cuda:1")      # cuda:0 stays current throughout
    assert torch.cuda.current_device() == 0 and b.state.device == torch.device("cuda", 1)
    assert all(torch.equal(x.cpu(), y.cpu()) for x, y in zip(outs_a, outs_b))
    assert torch.equal(a.state.table.cpu(), b.state.table.cpu())
    q, k, v = orc.make_step(31, 99, 1, 4, 2, 128)
    with pytest.raises(ValueError):
        b.decode_attend(q.cuda(), k.cuda(), v.cuda())                   # tensors of another device are refused
    a.close(); b.close()


def test_offload_prefill_factory_matches_the_default_factory():
    from lrqk_b200 import LightAttentionIndicesFactory, LightAttentionIndicesOffloadPrefill
    a, outs_a = _run(LightAttentionIndicesFactory)
    b, outs_b = _run(LightAttentionIndicesOffloadPrefill)
    assert all(torch.equal(x, y) for x, y in zip(outs_a, outs_b))
    assert torch.equal(a.state.table, b.state.table) and torch.equal(a.state.K_res, b.state.K_res)
    a.close(); b.close()


def test_hit_rate_counter_sees_every_step():
    from lrqk_b200 import HitRateCounter
    fac, outs = _run(HitRateCounter, steps=5)
    assert len(fac.miss_rates) == 5 and all(0.0 <= r <= 1.0 for r in fac.miss_rates)
    assert 0.0 < fac.average_miss_rate() <= 1.0
    fac.close()


def test_throughput_driver_runs_every_row_of_the_table():
    import transformers
    from lrqk_b200 import patch_model, run_task
    from lrqk_b200.extras import task_dict
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=4096)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(cfg).to(torch.bfloat16).cuda().eval()
    patch_model(model)
    for name in task_dict:
        rec = run_task(name, model, r=16, num_active_tokens=256, lite_tokens=16, prompt_lens=(320,), max_new_tokens=8)
        assert rec["320"]["prefill_tps"] > 0 and rec["320"]["decode_tps"] > 0, name
    with pytest.raises(ValueError):
        run_task("nope", model)


@pytest.mark.parametrize("seq,dtype", [(900, torch.bfloat16), (70, torch.float32)])
def test_layer_state_dict_resumes_bit_for_bit(seq, dtype):
    """state_dict() after a few steps, load_state_dict() into a fresh factory: the following steps -- ring
    flushes and, for the short prompt, the change from all-resident to selecting included -- give the same
    attention rows, slot table, resident rows and host rows as the run that was never interrupted."""
    import lrqk_oracle as orc
    from lrqk_b200 import LightAttentionIndicesFactory
    bsz, hq, hkv, d, k, m = 2, 4, 2, 128, 64, 8
    Q, K, V = orc.make_prompt(3, bsz, hq, hkv, seq, d, dtype=dtype)
    make = lambda: LightAttentionIndicesFactory(num_lite_tokens=m, attn_topk=k, num_key_value_groups=hq // hkv, r=8,
                                                max_iter=(2, 2), tol=1e-2, capacity=seq + 64, init_aq_ak_method="top",
                                                weights=(1.0, 1.0, 1.0, 1.0))
    steps = [tuple(t.to(dtype).cuda() for t in orc.make_step(3, s, bsz, hq, hkv, d)) for s in range(30)]
    a = make()
    a.prefill(Q.cuda(), K.cuda(), V.cuda())
    for q, kk, v in steps[:7]:
        a.decode_attend(q, kk, v)
    sd = a.state_dict()
    outs_a = [a.decode_attend(q, kk, v).clone() for q, kk, v in steps[7:]]
    torch.cuda.synchronize()
    b = make()
    b.load_state_dict(sd)
    assert (b.current_len, b.lite_len, b.lite_indices) == (sd["counters"]["current_len"], sd["counters"]["lite_len"],
                                                           sd["counters"]["lite_indices"])
    outs_b = [b.decode_attend(q, kk, v).clone() for q, kk, v in steps[7:]]
    torch.cuda.synchronize()
    for x, y in zip(outs_a, outs_b):
        assert torch.equal(x.view(torch.uint8), y.view(torch.uint8))
    sa, sb = a.state, b.state
    for name in ("B_Q", "B_K", "K_res", "V_res", "table", "lite_pos"):
        assert torch.equal(getattr(sa, name), getattr(sb, name)), name
    assert torch.equal(sa.A_K[:, :, :a.current_len], sb.A_K[:, :, :b.current_len])
    assert len(a.KVcpu) == len(b.KVcpu) and torch.equal(a.KVcpu.tensor(), b.KVcpu.tensor())
    assert a.lite_indices == b.lite_indices and a.current_len == b.current_len
    # other settings are refused
    other = LightAttentionIndicesFactory(num_lite_tokens=m + 1, attn_topk=k, num_key_value_groups=hq // hkv, r=8)
    with pytest.raises(ValueError):
        other.load_state_dict(sd)
    a.close()
    b.close()


def test_cache_save_and_load(tmp_path):
    """DynamicLRQKCache.save()/load(): one layer decoding, one still collecting a short prompt."""
    import lrqk_oracle as orc
    from lrqk_b200 import DynamicLRQKCache
    bsz, hq, hkv, d, k, m = 1, 4, 2, 128, 64, 8
    make = lambda: DynamicLRQKCache(r=8, num_active_tokens=k, lite_tokens=m, max_iter=(2, 2), tol=1e-2,
                                    max_sequence_length=2048, num_key_value_groups=hq // hkv, init_aq_ak_method="top")
    Q, K, V = orc.make_prompt(5, bsz, hq, hkv, 700, d, dtype=torch.bfloat16)
    Qs, Ks, Vs = orc.make_prompt(6, bsz, hq, hkv, 20, d, dtype=torch.bfloat16)      # shorter than num_active_tokens
    steps = [tuple(t.to(torch.bfloat16).cuda() for t in orc.make_step(5, s, bsz, hq, hkv, d)) for s in range(12)]
    a = make()
    a.update(Q.cuda(), K.cuda(), V.cuda(), 0)
    a.update(Qs.cuda(), Ks.cuda(), Vs.cuda(), 1)
    for q, kk, v in steps[:4]:
        a.attend(q, kk, v, 0)
    path = str(tmp_path / "cache.pt")
    a.save(path)
    b = make()
    b.load(path)
    assert b.is_decoding(0) and not b.is_decoding(1)
    assert b.sequence_state[1] == DynamicLRQKCache.State.collecting and len(b.temp_buff_cache_qkv[1]) == 20
    for q, kk, v in steps[4:]:
        x, y = a.attend(q, kk, v, 0), b.attend(q, kk, v, 0)
        assert torch.equal(x.view(torch.uint8), y.view(torch.uint8))
        ka, va = a.update(q, kk, v, 1)
        kb, vb = b.update(q, kk, v, 1)
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    torch.cuda.synchronize()
    a.close()
    b.close()
