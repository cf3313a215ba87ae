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
