"""Host-side logic of the multi-GPU path, without a GPU: shard planning, slicing and assembly, the
push/wait sequence discipline, and a world-size-2 run over gloo in which every rank computes the
attention of its own heads with the CPU oracle and the gathered rows are assembled into model
order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import lrqk_oracle as orc
from lrqk_b200 import sharding


def test_plan_shards_kv_heads_first_then_batch():
    # Llama-3-8B shape: 8 KV heads over 1, 2, 4, 8 ranks
    for world in (1, 2, 4, 8):
        sh = sharding.plan_shards(1, 8, world)
        assert [s.kv_heads for s in sh] == [8 // world] * world
        assert [s.h0 for s in sh] == [r * (8 // world) for r in range(world)]
        assert all(s.bsz == 1 and s.b0 == 0 for s in sh)
    # Qwen2.5-7B shape: 4 KV heads, batch 8: heads at 2 and 4 ranks, batch x heads at 8
    sh = sharding.plan_shards(8, 4, 8)
    assert [(s.b0, s.bsz, s.h0, s.kv_heads) for s in sh] == [(0, 4, h, 1) for h in range(4)] + [(4, 4, h, 1) for h in range(4)]
    units = sorted((b, h) for s in sh for b in range(s.b0, s.b0 + s.bsz) for h in range(s.h0, s.h0 + s.kv_heads))
    assert units == [(b, h) for b in range(8) for h in range(4)]          # every unit exactly once
    with pytest.raises(ValueError):
        sharding.plan_shards(1, 8, 3)
    with pytest.raises(ValueError):
        sharding.plan_shards(3, 4, 8)


def test_slice_and_assemble_round_trip():
    bsz, hkv, groups, d = 4, 2, 3, 8
    x = torch.arange(bsz * hkv * groups * d, dtype=torch.float32).reshape(bsz, hkv * groups, d)
    for world in (1, 2, 4):
        sh = sharding.plan_shards(bsz, hkv, world)
        parts = torch.stack([sharding.slice_for_shard(x, s, groups).contiguous() for s in sh])
        assert torch.equal(sharding.assemble(parts, sh, bsz, hkv * groups, groups), x)


def test_push_sequence_discipline():
    seq = sharding.PushSequence()
    with pytest.raises(RuntimeError):
        seq.next_wait()                      # nothing pushed yet
    assert seq.next_push() == 1
    with pytest.raises(RuntimeError):
        seq.next_push()                      # push 1 not waited for: would overwrite a half in use
    assert seq.next_wait() == 1
    assert seq.next_push() == 2 and seq.next_wait() == 2
    assert (seq.next_push() & 1) == 1        # halves alternate


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bsz, hq, hkv, d, rows = 2, 8, 4, 16, 40
        groups = hq // hkv
        g = torch.Generator().manual_seed(5)          # every rank draws the same full problem
        q = torch.randn(bsz, hq, 1, d, generator=g)
        K = torch.randn(bsz, hq, rows, d, generator=g)
        V = torch.randn(bsz, hq, rows, d, generator=g)
        shards = sharding.plan_shards(bsz, hkv, world)
        mine = shards[rank]
        local = orc.attention(*(sharding.slice_for_shard(t, mine, groups) for t in (q, K, V)))[:, :, 0]
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local.contiguous())
        full = sharding.assemble(torch.stack(gathered), shards, bsz, hq, groups)
        ref = orc.attention(q, K, V)[:, :, 0]
        ok = torch.allclose(full, ref, atol=1e-6)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo_assemble_the_unsharded_result(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def _prompt_rank_main(rank: int, world: int, port: int, out_dir: str):
    """The prompt pass of a head-sharded decoder layer as the patched forward runs it: attention of
    this rank's heads, all-gather, model order -- for heads-only and batch-x-heads splits, with a
    left-padded sequence."""
    from lrqk_b200.hf_models import _causal_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        for bsz, hq, hkv in ((2, 8, 4), (2, 3, 1)):                # second: ranks outnumber KV heads
            S, d = 24, 16
            g = torch.Generator().manual_seed(7)
            q = torch.randn(bsz, hq, S, d, generator=g)
            K = torch.randn(bsz, hkv, S, d, generator=g)
            V = torch.randn(bsz, hkv, S, d, generator=g)
            pad = torch.ones(bsz, S, dtype=torch.bool)
            pad[1, :5] = False
            sh = sharding.HeadSharding()
            assert (sh.rank, sh.world) == (rank, world)
            local = _causal_attention(sh.local(q, hkv), sh.local(K, hkv), sh.local(V, hkv), d ** -0.5,
                                      sh.local_rows(pad, hkv))
            full = sh.gather_prompt(local, bsz, hkv, hq)
            ref = _causal_attention(q, K, V, d ** -0.5, pad)
            real = pad[:, :, None, None].expand_as(ref)               # rows of padded queries are undefined
            ok = ok and full.shape == ref.shape and torch.allclose(full[real], ref[real], atol=1e-5)
            # one decode row per head through the same assembly
            rows = torch.randn(bsz, hq, d, generator=g)
            mine = sh.local(rows, hkv).contiguous()
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            ok = ok and torch.equal(sh._assemble(torch.stack(parts), bsz, hkv, hq), rows)
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_head_sharded_prompt_pass_over_gloo(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_prompt_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def test_cache_refuses_to_shard_after_the_first_prompt():
    from lrqk_b200 import DynamicLRQKCache
    cache = DynamicLRQKCache(num_key_value_groups=2)
    cache.sequence_state[0] = cache.State.decoding
    with pytest.raises(RuntimeError):
        cache.shard_heads(sharding=sharding.HeadSharding(rank=0, world=2))
    fresh = DynamicLRQKCache(num_key_value_groups=2)
    sh = fresh.shard_heads(sharding=sharding.HeadSharding(rank=1, world=2))
    assert fresh.sharding is sh and sh.shard(1, 8).h0 == 4
    x = torch.arange(2 * 8 * 3 * 4.0).reshape(2, 8, 3, 4)
    q, k, v, mask = fresh._local(x, x[:, :4], x[:, :4], torch.ones(2, 3))
    assert torch.equal(q, x[:, 4:]) and torch.equal(k, x[:, 2:4]) and mask.shape == (2, 3)


def test_cpulist_parsing_and_missing_topology(tmp_path):
    assert sharding._parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert sharding._parse_cpulist("") == []
    # no CUDA device / no sysfs entry: the helpers report "unknown" and change nothing
    assert sharding.gpu_numa_cpus(0, sysfs=str(tmp_path)) is None
