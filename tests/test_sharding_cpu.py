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


def test_cpulist_parsing_and_missing_topology(tmp_path):
    assert sharding._parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert sharding._parse_cpulist("") == []
    # no CUDA device / no sysfs entry: the helpers report "unknown" and change nothing
    assert sharding.gpu_numa_cpus(0, sysfs=str(tmp_path)) is None
