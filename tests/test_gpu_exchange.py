"""The attention kernel's push epilogue and the bounded wait (lrqk_flash_decode_push,
lrqk_allgather_wait), on one GPU with emulated ranks and -- when two GPUs are visible -- with two
processes exchanging over CUDA IPC."""
import ctypes as C
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk_state(seed, bsz, hq, d, rows, dtype):
    from lrqk_b200.state import LayerState
    g = torch.Generator().manual_seed(seed)
    st = LayerState(bsz, hq, hq, d, 16, rows - 8, 8, a_capacity=64, host_capacity=16, dtype=dtype, with_host=False)
    st.K_res.copy_(torch.randn(bsz, hq, rows, d, generator=g).to(dtype))
    st.V_res.copy_(torch.randn(bsz, hq, rows, d, generator=g).to(dtype))
    q = torch.randn(bsz, hq, d, generator=g).to(dtype).cuda()
    return st, q


def _push(st, q, ex, lib, _lib):
    seq = ex.seq.next_push()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.lrqk_flash_decode_push(C.byref(st.c), C.c_void_p(q.data_ptr()), C.c_void_p(st.attn_out.data_ptr()),
                                          st.k + st.m, st.head_dim ** -0.5, C.c_void_p(st.attn_ws.data_ptr()),
                                          C.byref(ex.c), seq, stream), "lrqk_flash_decode_push")


@pytest.mark.parametrize("dtype,world,hq,d", [(torch.bfloat16, 2, 4, 128), (torch.float32, 4, 2, 64)])
def test_emulated_ranks_push_and_wait(dtype, world, hq, d):
    from lrqk_b200 import _lib, sharding
    lib = _lib.lib()
    group = sharding.HeadExchange.local_group(world, hq, d, dtype)
    states = [_mk_state(100 + r, 1, hq, d, 300, dtype) for r in range(world)]
    for step in range(3):                                   # three pushes: both halves get reused
        expect = []
        for r, (st, q) in enumerate(states):
            q.add_(0.25 * step)
            expect.append(st.flash_decode(q).clone())       # the plain entry point is the reference here
            _push(st, q, group[r], lib, _lib)               # all pushes are enqueued before any wait
        for r in range(world):
            got = group[r].wait().clone()
            torch.cuda.synchronize()
            group[r].check_status()
            for src in range(world):
                assert torch.equal(got[src], expect[src][0]), (step, r, src)
    for ex in reversed(group):
        ex.close()


def test_push_without_a_local_output_buffer():
    """`out` may be NULL: the rows then only exist in the exchange buffers."""
    from lrqk_b200 import _lib, sharding
    lib = _lib.lib()
    group = sharding.HeadExchange.local_group(1, 4, 128, torch.bfloat16)
    st, q = _mk_state(3, 1, 4, 128, 200, torch.bfloat16)
    expect = st.flash_decode(q).clone()
    seq = group[0].seq.next_push()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.lrqk_flash_decode_push(C.byref(st.c), C.c_void_p(q.data_ptr()), None, st.k + st.m, 128 ** -0.5,
                                          C.c_void_p(st.attn_ws.data_ptr()), C.byref(group[0].c), seq, stream), "push")
    got = group[0].wait().clone()
    torch.cuda.synchronize()
    group[0].check_status()
    assert torch.equal(got[0], expect[0])
    group[0].close()


def test_wait_runs_out_and_reports_without_hanging():
    from lrqk_b200 import _lib, sharding
    lib = _lib.lib()
    group = sharding.HeadExchange.local_group(2, 2, 64, torch.float32)
    st, q = _mk_state(7, 1, 2, 64, 40, torch.float32)
    _push(st, q, group[0], lib, _lib)                       # rank 1 never pushes
    assert lib.lrqk_peer_set_wait_polls(2000) == 0          # a couple of milliseconds
    try:
        got = group[0].wait()
        torch.cuda.synchronize()                            # returns: the wait is bounded
        assert bool(torch.isnan(got).all())                 # no stale rows: what did not arrive reads as NaN
        with pytest.raises(_lib.LrqkError) as e:
            group[0].check_status()
        assert e.value.code == _lib.ETIMEOUT
        x = torch.ones(4, device="cuda") * 2                # the context is still usable
        assert float(x.sum()) == 8.0
    finally:
        lib.lrqk_peer_set_wait_polls(1 << 22)
        for ex in reversed(group):
            ex.close()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_gpu_rank(rank, world, port, out_dir):
    import torch.distributed as dist
    from lrqk_b200 import _lib, sharding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = "ok"
    try:
        lib = _lib.lib()
        hq, d, dtype = 4, 128, torch.bfloat16
        ex = sharding.HeadExchange(hq, d, dtype)
        states = [_mk_state(100 + r, 1, hq, d, 300, dtype) for r in range(world)]   # every rank can recompute all
        for step in range(4):
            expect = []
            for st, q in states:
                q.add_(0.25)
                expect.append(st.flash_decode(q).clone())
            st, q = states[rank]
            _push(st, q, ex, lib, _lib)
            got = ex.wait().clone()
            torch.cuda.synchronize()
            ex.check_status()
            for src in range(world):
                if not torch.equal(got[src], expect[src][0]):
                    ok = f"mismatch step {step} src {src}"
            dist.barrier()
        ex.close()
    except Exception as e:  # reported through the file so that the parent sees it
        ok = f"error: {e!r}"
    finally:
        with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
            f.write(ok)
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_exchange_over_ipc(tmp_path):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_two_gpu_rank, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
